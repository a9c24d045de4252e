"""Host-side logic of the multi-GPU path on CPU: two gloo ranks deal the layer's units, and the K-split exchange
(sum of residues across ranks, then reduction modulo the prime) reproduces the modular sum."""
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


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layer = importlib.import_module(PKG + ".layer")
    wl = layer.LayerWorkload(_NoHemmer(), layer.synthetic(1), rank=rank, world=world)
    names = [u[1] + ":" + str(u[4]) if u[0] == "pcmm" else u[1] for u in wl.mine]
    gathered = [None] * world
    dist.all_gather_object(gathered, names)
    # lazy sum of residues below 2^60 over the ranks, then one reduction: equals the modular sum
    prime = (1 << 60) - 93 * (1 << 17) + 1
    rng = np.random.default_rng(10 + rank)
    part = rng.integers(0, prime, size=1024, dtype=np.uint64)
    t = torch.from_numpy(part.astype(np.int64))
    dist.all_reduce(t)
    lazy = (t.numpy().astype(np.uint64) % np.uint64(prime))
    parts = [None] * world
    dist.all_gather_object(parts, part)
    exact = np.zeros(1024, dtype=object)
    for p in parts:
        exact = (exact + p.astype(object)) % prime
    if rank == 0:
        q.put((gathered, len(wl.units), bool(np.array_equal(lazy.astype(object), exact))))
    dist.destroy_process_group()


def test_two_ranks_cover_all_units_and_ksplit_sum_is_exact():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    gathered, total, ok = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    flat = [n for g in gathered for n in g]
    assert len(flat) == total == 54 and len(set(flat)) == total
    assert abs(len(gathered[0]) - len(gathered[1])) <= 1
    assert ok


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
