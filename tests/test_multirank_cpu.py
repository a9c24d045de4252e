"""Host-side logic of the multi-GPU path on CPU.

* every rank count from 1 to 8 deals all units, gives every output tile exactly one owner among the ranks that hold
  partial products of it, and issues matching sends and receives;
* two gloo ranks run the layer driver's own K-split exchange (`LayerWorkload._exchange_partials`) on random partial
  products, with torch.distributed point-to-point calls standing where the NCCL ones stand on the GPU: the owner ends
  up with the exact modular sum and nobody else holds the tile;
* a rank-local pass in the oracle's dry mode walks the whole driver, exchange included.
"""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = "encryption-friendly_llm_architecture_b200"


class _NoLib:
    N = 65536


class _NoHemmer:
    lib = _NoLib()


def test_dealing_and_tile_ownership_for_every_rank_count():
    sys.path.insert(0, ROOT)
    layer = importlib.import_module(PKG + ".layer")
    data = layer.synthetic(1)
    for world in range(1, 9):
        wls = [layer.LayerWorkload(_NoHemmer(), data, rank=r, world=world) for r in range(world)]
        seen = sorted(i for w in wls for i in w.mine)
        assert seen == list(range(54)), f"world {world}: units dealt {seen}"
        loads = [sum(layer.unit_cost(w.units[i]) for i in w.mine) for w in wls]
        assert max(loads) <= 1.25 * (sum(loads) / world) + 1e-9, f"world {world}: unbalanced {loads}"
        w0 = wls[0]
        assert len(w0.tile_keys) == 54
        for key in w0.tile_keys:
            owners = {w.tile_owner[key] for w in wls}
            assert len(owners) == 1, "ranks disagree on the owner"
            own = owners.pop()
            assert own in w0.members[key[0]], "owner holds no partial product of its tile"
        # what each rank reads back after the exchange: every tile and every ct x ct unit by exactly one rank
        held = []
        for w in wls:
            fake = {"pcmm": {k: layer.CtxtTensor(None, 1, 1) for k in w.tile_keys if w.rank == w.tile_owner[k]},
                    "ccmm": {"all": ([i for i in w.mine if w.units[i][0] == "ccmm"], layer.CtxtTensor(None, 1, 1))}}
            held += [tag for tag, _, _ in w.held_outputs(fake)]
        assert len(held) == len(set(held)) == 54 + 42, f"world {world}: {len(held)} results read back"
        # sends and receives pair up, in the same order on both sides
        plan = w0.exchange_plan()
        assert all(w.exchange_plan() == plan for w in wls)
        for key, src, own in plan:
            assert src != own and src in w0.members[key[0]]


class _GlooExchange:
    """The oracle library with the exchange calls carried by torch.distributed (gloo)."""

    def __init__(self, lib):
        self._lib = lib
        self._pending = []

    def __getattr__(self, name):
        return getattr(self._lib, name)

    def nccl_group_start(self):
        self._pending = []

    def send(self, ct, peer, comm):
        t = torch.from_numpy(self._lib.ct_export(ct).view(np.int64).copy())
        self._pending.append(dist.isend(t, peer))
        self._pending.append(t)

    def recv(self, ct, peer, comm):
        level, npoly, batch, _ = self._lib.ct_meta(ct)
        t = torch.empty((batch, npoly, level + 1, self._lib.N), dtype=torch.int64)
        self._pending.append((dist.irecv(t, peer), t, ct))

    def nccl_group_end(self):
        for p in self._pending:
            if isinstance(p, tuple):
                req, t, ct = p
                req.wait()
                self._lib.ct_import(ct, t.numpy().view(np.uint64))
            elif not isinstance(p, torch.Tensor):
                p.wait()
        self._pending = []


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = importlib.import_module(PKG)
    layer = importlib.import_module(PKG + ".layer")
    orc = pkg.capi.Lib(os.path.join(ROOT, "oracle", "_build", "liboracle.so"), "orc_", pkg.make_params())
    H = pkg.Hemmer(orc)
    H.lib = _GlooExchange(orc)
    wl = layer.LayerWorkload(H, layer.synthetic(1), rank=rank, world=world)
    wl.comm = 0
    # a few tiles of every sublayer keep the test small; the plan and the ownership rule are the driver's own
    wl.tile_keys = [k for k in wl.tile_keys if k[2] < 2]
    level = wl.target + 1
    stable = lambda key: sum(ord(c) for c in key[0] + key[1]) * 31 + key[2]
    def part(key, member):
        rng = np.random.default_rng(stable(key) * 8 + member)
        out = np.empty((1, 2, level + 1, orc.N), dtype=np.uint64)
        for l in range(level + 1):
            out[0, :, l, :] = rng.integers(0, int(orc.primes[l]), size=(2, orc.N), dtype=np.uint64)
        return out
    partial = {}
    for key in wl.tile_keys:
        if rank in wl.members[key[0]]:
            ct = orc.ct_create(level, 2, 1, 2)
            orc.ct_import(ct, part(key, rank))
            partial[key] = layer.CtxtTensor(ct, 128, 128, 256)
    wl._exchange_partials(partial)
    ok = True
    for key in wl.tile_keys:
        if wl.tile_owner[key] != rank:
            ok &= key not in partial
            continue
        want = np.zeros((1, 2, level + 1, orc.N), dtype=np.uint64)
        for m in wl.members[key[0]]:
            want += part(key, m)          # at most a few residues below 2^60: no overflow
        for l in range(level + 1):
            want[0, :, l, :] %= orc.primes[l]
        ok &= key in partial and bool(np.array_equal(orc.ct_export(partial[key].ct), want))
    results = [None] * world
    dist.all_gather_object(results, (ok, sorted(k for k in partial)))
    if rank == 0:
        q.put((results, [wl.members[n] for n in ("qkv", "wo", "w1", "w2")], len(wl.tile_keys)))
    dist.destroy_process_group()


def test_two_ranks_run_the_ksplit_exchange_exactly():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results, members, ntiles = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for ok, _ in results)
    held = [k for _, keys in results for k in keys]
    assert len(held) == len(set(held)) == ntiles           # every tile ends up on exactly one rank
    assert any(len(m) == 2 for m in members), "no sublayer was split over the two ranks: the exchange was not exercised"


def test_rank_local_step_runs_the_ksplit_exchange(pkg, oracle_so):
    """Each rank's pass over its share of the layer, including the K-split exchange code path, on the oracle in dry mode
    (operation bookkeeping only): the operation counts of the two ranks add up to those of the single-rank pass."""
    import ctypes as C
    layer = importlib.import_module(PKG + ".layer")

    def counts(rank, world):
        o = pkg.capi.Lib(oracle_so, "orc_", pkg.make_params())
        o.dll.orc_set_dry(o.ctx, 1)
        wl = layer.LayerWorkload(pkg.Hemmer(o), layer.synthetic(3), rank=rank, world=world)
        wl.comm = 0
        wl.step()
        need = o.dll.orc_stats_dump(o.ctx, None, 0)
        buf = C.create_string_buffer(need)
        o.dll.orc_stats_dump(o.ctx, buf, need)
        out = {}
        for line in buf.value.decode().splitlines():
            op, lvl, n = line.split()
            if op in ("rotate", "tensor", "relin", "mul_pt"):
                out[(op, int(lvl))] = int(n)
        return out

    whole, parts = counts(0, 1), [counts(r, 2) for r in range(2)]
    for key, n in whole.items():
        assert sum(p.get(key, 0) for p in parts) == n, key
