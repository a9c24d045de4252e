"""Generates tests/golden/golden.json from the CPU oracle.

The reference holds no golden vectors for this path (its arithmetic library is closed and never seeded), so
the fixtures pin this repository's own specification: SHA-256 digests of the ciphertext residues the oracle
produces for seeded cases.  tests/test_golden_cpu.py checks that the oracle still reproduces the small cases;
tests/test_gpu_parity.py checks the CUDA library against the full-size ones without re-running the oracle.

Run from the repository root:  python tests/golden/make_golden.py   (a few minutes: one full-size 128x128 ct x ct product)
and  python tests/golden/make_golden.py --layer-units 0 ; python tests/golden/make_golden.py --layer-units 2
(one product of every kind of the encoder-layer workload, in the reference's rotation sequence and in the
benchmarked schedule; about ten minutes per unit)
"""
import hashlib
import importlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
pkg = importlib.import_module("encryption-friendly_llm_architecture_b200")
import cases  # noqa: E402
from conftest import SMALL, rand_ct_residues  # noqa: E402

ORACLE = os.path.join(ROOT, "oracle", "_build", "liboracle.so")


def digest(arr):
    return hashlib.sha256(np.ascontiguousarray(arr, dtype=np.uint64).tobytes()).hexdigest()


def small_cases():
    o = pkg.capi.Lib(ORACLE, "orc_", pkg.make_params(**SMALL))
    o.keygen()
    H = pkg.Hemmer(o)
    out = {}
    for name in sorted(cases.SCENARIOS):
        exports, err = cases.SCENARIOS[name](o, H)
        out[name] = {"digests": [digest(e) for e in exports], "max_abs_err": err}
    return out


def full_cases():
    o = pkg.capi.Lib(ORACLE, "orc_", pkg.make_params())
    o.keygen()
    o.gen_rot_keys([1, 128, 4096])
    out = {"primes": [int(q) for q in o.primes], "scales": [float(s) for s in o.scales]}
    prim = {}
    for lvl in (12, 4, 1):
        data = rand_ct_residues(o, lvl, 2, 1, seed=500 + lvl)
        ct = o.ct_create(lvl, 2, 1)
        o.ct_import(ct, data)
        pt = o.encode(np.random.default_rng(600 + lvl).uniform(-1, 1, o.slots), lvl)
        prim[f"rotate1@{lvl}"] = digest(o.ct_export(o.rotate(ct, 1)))
        prim[f"rotate4096@{lvl}"] = digest(o.ct_export(o.rotate(ct, 4096)))
        prim[f"tensor_relin@{lvl}"] = digest(o.ct_export(o.relin(o.tensor(ct, ct))))
        prim[f"rescale@{lvl}"] = digest(o.ct_export(o.rescale(o.mul_pt_norescale(ct, pt))))
        c2 = o.ct_create(lvl, 2, 1)
        o.ct_import(c2, data)
        o.ntt(c2)
        prim[f"ntt@{lvl}"] = digest(o.ct_export(c2))
    out["primitives"] = prim
    # one 128x128 ct x ct product, operands uniform[-1,1], one tile per ciphertext
    H = pkg.Hemmer(o)
    exports, err = cases.sc_ccmm_single_tile(o, H, target=4)
    out["config1_ccmm_128"] = {"digest": digest(exports[0]), "first_residues": [int(v) for v in exports[0].reshape(-1)[:8]], "max_abs_err": err}
    return out


# Units of the encoder-layer workload (encryption-friendly_llm_architecture_b200/layer.py, seed 1234, the nonces of
# LayerWorkload.check) computed one at a time by the oracle at full size: one product of every kind the layer runs.
LAYER_CCMM = ["lora0_xa0",   # two-tile ct x ct, activations x zero-padded rank-8 LoRA factor
              "qk0",         # right operand transposed: Q K^T of two heads
              "bwd0_db0",    # left operand transposed: (X A)^T dY
              "sv0"]         # scores in [0, 1/128] x V
LAYER_PCMM = [("qkv", "wq", 0)]   # complexPacking + matMulPre + matMulReUse over both K-groups of the 768-wide input, N(0, 0.02^2) weights
LAYER_SEED, LAYER_NONCE0 = 1234, 20_000


def layer_units(schedule, only=None):
    """{unit name: digest} for one schedule variant (0: the reference's rotation sequence, 2: the benchmarked one)."""
    layer = importlib.import_module("encryption-friendly_llm_architecture_b200.layer")
    o = pkg.capi.Lib(ORACLE, "orc_", pkg.make_params())
    o.keygen()
    H = pkg.Hemmer(o)
    H.set_schedule(schedule)
    wl = layer.LayerWorkload(H, layer.synthetic(LAYER_SEED))
    out = {}
    for name in LAYER_CCMM:
        if only and name not in only:
            continue
        c = wl.ccmm_alone(wl.unit_index(name), LAYER_NONCE0)
        out[name] = digest(o.ct_export(c.ct)[0])
        print(schedule, name, out[name], flush=True)
    for key in LAYER_PCMM:
        name = "/".join(str(k) for k in key)
        if only and name not in only:
            continue
        c = wl.pcmm_tile_alone(key, LAYER_NONCE0)
        out[name] = digest(o.ct_export(c.ct)[0])
        print(schedule, name, out[name], flush=True)
    return out


if __name__ == "__main__":
    path = os.path.join(ROOT, "tests", "golden", "golden.json")
    if "--layer-units" in sys.argv:
        # python tests/golden/make_golden.py --layer-units SCHEDULE [unit ...]: about ten minutes per unit on eight cores;
        # merges into the existing file
        k = sys.argv.index("--layer-units")
        schedule, only = int(sys.argv[k + 1]), sys.argv[k + 2:]
        got = layer_units(schedule, only or None)
        data = json.load(open(path))
        data.setdefault("layer_units", {}).setdefault(f"schedule{schedule}", {}).update(got)
        data["layer_units"]["seed"], data["layer_units"]["nonce0"] = LAYER_SEED, LAYER_NONCE0
    else:
        data = json.load(open(path)) if os.path.exists(path) else {}
        data["small"] = small_cases()
        if "--small-only" not in sys.argv:
            data["full"] = full_cases()
    with open(path, "w") as f:
        json.dump(data, f, indent=1, sort_keys=True)
    print("wrote golden.json")
