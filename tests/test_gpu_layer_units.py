"""Full-size parity of the benchmarked path: the units of the encoder-layer workload, computed through the batched
calls the layer driver makes (shared launch sequences, grouped loop iterations), must carry the residues the CPU
oracle produced for the same units one at a time (digests in tests/golden/golden.json, made by make_golden.py)."""
import importlib
import json
import os

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu
PKG = "encryption-friendly_llm_architecture_b200"


def _golden():
    return json.load(open(os.path.join(ROOT, "tests", "golden", "golden.json"))).get("layer_units", {})


def _tag(wl, name):
    if "/" in name:
        s, w, j = name.split("/")
        return ("p", s, w, int(j))
    return ("c", wl.unit_index(name))


@pytest.mark.parametrize("schedule", [2, 0])
def test_layer_units_match_oracle_digests(pkg, gpu_full, schedule):
    gold = _golden()
    want = gold.get(f"schedule{schedule}", {})
    if not want:
        pytest.skip("no recorded digests for this schedule")
    layer = importlib.import_module(PKG + ".layer")
    H = pkg.open_hemmer(gpu_full)
    H.set_schedule(schedule)
    wl = layer.LayerWorkload(H, layer.synthetic(gold["seed"]))
    tags = {_tag(wl, n): n for n in want}
    # a reduced layer that keeps the batching structure: the recorded ct x ct units together with further units of
    # each transpose group (so that the joint transpose, the per-group transforms and the shared product loop all
    # see batches > 1), and the whole 768-wide ct x pt sublayer of the recorded output tile (both of its K-groups)
    keep = {i for t, i in ((t[0], t[1]) for t in tags) if t == "c"}
    extra = {False: 2, True: 1, "left": 1}
    for i, u in enumerate(wl.units):
        if u[0] == "ccmm" and i not in keep and extra.get(u[4], 0) > 0:
            keep.add(i); extra[u[4]] -= 1
    sub = {t[1] for t in tags if t[0] == "p"}
    keep |= {i for i, u in enumerate(wl.units) if u[0] == "pcmm" and u[1] in sub}
    wl.mine = sorted(keep)
    out = wl._compute(wl._encrypt_all(gold["nonce0"]))
    dig = wl.output_digests(out)
    for tag, name in tags.items():
        assert dig[tag] == want[name], f"schedule {schedule}: unit {name} differs from the oracle"
    # the unit computed on its own through the unbatched calls gives the same bits as its batch member
    i = wl.unit_index("sv0")
    alone = wl.ccmm_alone(i, gold["nonce0"])
    assert layer.sha(gpu_full.ct_export(alone.ct)[0]) == dig[("c", i)]
    err = wl._decrypt_all(out, check=True)
    assert err < 2.0 ** -14


def test_graph_replay_reproduces_the_pass(pkg, gpu_full):
    """A recorded pass replayed twice leaves the bits of a host-launched pass; recording refuses host copies."""
    layer = importlib.import_module(PKG + ".layer")
    g = gpu_full
    H = pkg.open_hemmer(g)
    H.set_schedule(2)
    wl = layer.LayerWorkload(H, layer.synthetic(7))
    wl.mine = [wl.unit_index("sv1"), wl.unit_index("qk1"), wl.unit_index("wo", 1)]
    wl.prepare()
    first = wl.output_digests(wl.step_resident())
    graph, out = wl.record_graph()
    assert g.graph_kernels(graph) > 100
    for _ in range(2):
        g.graph_launch(graph)
    g.sync()
    assert wl.output_digests(out) == first
    g.graph_begin()
    with pytest.raises(pkg.HBError):
        g.ct_export(out["ccmm"]["all"][1].ct)
    g.graph_end()
