"""Further CUDA-vs-oracle parity: the benchmarked schedule on every scenario, primes near the top of the range the
FP64-assisted arithmetic accepts, worst-case residues at full size, and the collective entry points on a one-rank
communicator."""
import ctypes as C

import numpy as np
import pytest

import cases
from conftest import open_oracle, rand_ct_residues

pytestmark = pytest.mark.gpu
TOL = 2.0 ** -14


def _same(a, b, what=""):
    assert a.shape == b.shape, what
    if not np.array_equal(a, b):
        bad = np.argwhere(a != b)
        raise AssertionError(f"{what}: {len(bad)} of {a.size} residues differ, first at {bad[0].tolist()}")


@pytest.mark.parametrize("size", ["small", "mid"])
@pytest.mark.parametrize("name", ["packed", "packed_reuse", "cc_reuse", "transforms", "single_matmul", "lora_backward", "transpose_packing", "repack_lora_opti", "gaussian_kernel"])
def test_lazy_schedule_parity_remaining_scenarios(request, pkg, size, name):
    """Schedule 2 on the scenarios that test_gpu_parity.py runs in the other schedules only."""
    g, o = request.getfixturevalue(f"gpu_{size}"), request.getfixturevalue(f"orc_{size}")
    Hg, Ho = pkg.open_hemmer(g), pkg.Hemmer(o)
    Hg.set_schedule(2); Ho.set_schedule(2)
    eg, err_g = cases.SCENARIOS[name](g, Hg)
    eo, err_o = cases.SCENARIOS[name](o, Ho)
    assert len(eg) == len(eo)
    for k, (a, b) in enumerate(zip(eg, eo)):
        _same(a, b, f"lazy {name}[{k}]")
    assert err_g < TOL and err_g == err_o


Q44 = dict(log_n=10, max_level=8, dnum=3, num_special=3, hamming_weight=32, q_bits=44)


@pytest.mark.parametrize("schedule", [0, 2])
@pytest.mark.parametrize("name", ["ccmm_two_tiles", "pcmm_reuse", "batched", "transforms"])
def test_primes_of_44_bits(pkg, oracle_so, schedule, name):
    """Scaling primes just below 2^44: the lazy sums of FP64-assisted products sit closest to their 2^52 limit."""
    g = pkg.open_gpu(pkg.make_params(**Q44))
    o = open_oracle(pkg, oracle_so, **Q44)
    assert int(g.primes[1]) > 2 ** 43
    for lib in (g, o):
        lib.keygen()
    Hg, Ho = pkg.open_hemmer(g), pkg.Hemmer(o)
    Hg.set_schedule(schedule); Ho.set_schedule(schedule)
    eg, err_g = cases.SCENARIOS[name](g, Hg)
    eo, err_o = cases.SCENARIOS[name](o, Ho)
    for k, (a, b) in enumerate(zip(eg, eo)):
        _same(a, b, f"q44 {name}[{k}]")
    assert err_g < TOL and err_g == err_o


def test_matmul_acc_many_terms_with_44_bit_primes(pkg, oracle_so):
    """The open-ended lazy sum of the fused plaintext accumulate with every residue at q - 1: 512 copies x 1 group."""
    prm = dict(log_n=10, max_level=3, dnum=2, num_special=3, hamming_weight=32, q_bits=44)
    g = pkg.open_gpu(pkg.make_params(**prm))
    g.keygen()
    copies, lvl = 512, 2
    data = np.empty((copies, 2, lvl + 1, g.N), dtype=np.uint64)
    for l in range(lvl + 1):
        data[:, :, l, :] = np.uint64(int(g.primes[l]) - 1)
    pre = g.ct_create(lvl, 2, copies)
    g.ct_import(pre, data)
    z = np.random.default_rng(3).uniform(-1, 1, g.slots)
    pt = g.encode(z, lvl)
    out = C.c_void_p()
    g._chk(g.dll.hb_matmul_acc(g.ctx, pre.ptr, pt.ptr, C.c_int64(0), C.byref(out)))
    got = g.ct_export(pkg.capi.Handle(g, out, "ct"))
    w = g.pt_export(pt)
    for l in range(lvl + 1):
        q = int(g.primes[l])
        want = (np.array([(copies * (q - 1) * int(v)) % q for v in w[l]], dtype=np.uint64))
        assert np.array_equal(got[0, 0, l], want) and np.array_equal(got[0, 1, l], want), f"limb {l}"


@pytest.mark.parametrize("pattern", ["max", "zero", "alternate"])
def test_edge_residues_full_size(gpu_full, orc_full, pattern):
    """All residues q - 1, all 0, and alternating 0 / q - 1 at N = 2^16: the lazy value ranges inside the transforms
    and the inner products at their extremes.  Transform both ways, rotation, masked rotation pair, fused accumulate."""
    g, o = gpu_full, orc_full
    lvl, batch = 6, 2
    data = np.zeros((batch, 2, lvl + 1, g.N), dtype=np.uint64)
    for l in range(lvl + 1):
        top = np.uint64(int(g.primes[l]) - 1)
        if pattern == "max":
            data[:, :, l, :] = top
        elif pattern == "alternate":
            data[:, :, l, 0::2] = top
    for lib in (g, o):
        lib.gen_rot_keys([1, 3, -5])
    m1 = (np.random.default_rng(31).uniform(0, 1, g.slots) > 0.5).astype(np.float64)
    outs = []
    for lib in (g, o):
        res = []
        ct = lib.ct_create(lvl, 2, batch)
        lib.ct_import(ct, data)
        for inverse in (False, True):
            c2 = lib.ct_create(lvl, 2, batch)
            lib.ct_import(c2, data)
            lib.ntt(c2, inverse)
            res.append(lib.ct_export(c2))
        res.append(lib.ct_export(lib.rotate(ct, 1)))
        res.append(lib.ct_export(lib.assemble_rot(ct, 3, lib.encode_ext(m1, lvl), -5, lib.encode_ext(1.0 - m1, lvl))))
        res.append(lib.ct_export(lib.relin(lib.tensor(ct, ct))))
        outs.append(res)
    for k, (a, b) in enumerate(zip(*outs)):
        _same(a, b, f"{pattern}[{k}]")
    # fused plaintext accumulate over 8 copies with the same residues: against exact integer arithmetic
    pre = g.ct_create(lvl, 2, 8)
    g.ct_import(pre, np.concatenate([data] * 4))
    pt = g.encode(np.random.default_rng(4).uniform(-1, 1, g.slots), lvl)
    out = C.c_void_p()
    g._chk(g.dll.hb_matmul_acc(g.ctx, pre.ptr, pt.ptr, C.c_int64(0), C.byref(out)))
    from importlib import import_module
    got = g.ct_export(import_module("encryption-friendly_llm_architecture_b200.capi").Handle(g, out, "ct"))
    w = g.pt_export(pt)
    for l in (0, lvl):
        q = int(g.primes[l])
        want = np.array([(8 * int(a) * int(v)) % q for a, v in zip(data[0, 0, l, :4096], w[l, :4096])], dtype=np.uint64)
        assert np.array_equal(got[0, 0, l, :4096], want), f"matmul_acc limb {l}"


def test_collectives_on_a_one_rank_communicator(pkg, gpu_mid):
    """hb_mod_reduce, hb_sum_mod_reduce and the NCCL entry points with a communicator of one rank: the results must be
    the exact modular sums (numpy)."""
    g = gpu_mid
    lvl = 4
    rng = np.random.default_rng(12)
    parts = [rand_ct_residues(g, lvl, 2, 2, seed=200 + t) for t in range(5)]
    lazy = sum(p for p in parts)                       # five residues below 2^60: no 64-bit overflow
    want = lazy.copy()
    for l in range(lvl + 1):
        want[:, :, l, :] %= g.primes[l]
    ct = g.ct_create(lvl, 2, 2)
    g.ct_import(ct, lazy)
    g.mod_reduce(ct)
    _same(g.ct_export(ct), want, "mod_reduce")
    hs = []
    for p in parts:
        h = g.ct_create(lvl, 2, 2)
        g.ct_import(h, p)
        hs.append(h)
    _same(g.ct_export(g.sum_mod_reduce(hs)), want, "sum_mod_reduce")
    ident = (C.c_ubyte * 128)()
    assert g.dll.hb_nccl_unique_id(ident) == 0
    comm = C.c_void_p()
    g._chk(g.dll.hb_nccl_comm_init(g.ctx, C.c_int(1), C.c_int(0), ident, C.byref(comm)))
    try:
        g.ct_import(ct, lazy)
        g.allreduce_sum(ct, comm.value)
        _same(g.ct_export(ct), want, "allreduce_sum")
        g.ct_import(ct, lazy)
        g.reduce_sum(ct, 0, 0, comm.value)
        _same(g.ct_export(ct), want, "reduce_sum")
        both = g.ct_create(lvl, 2, 2)
        g.ct_zero(both)
        g.allgather(hs[0], both, comm.value)
        _same(g.ct_export(both), parts[0], "allgather")
    finally:
        g.dll.hb_nccl_comm_destroy(comm)
    other = pkg.open_gpu(pkg.make_params(log_n=10, max_level=8, dnum=3, num_special=3, hamming_weight=32))
    with pytest.raises(pkg.HBError):     # a handle of another context
        other.mod_reduce(ct)


def test_square_and_constant_product(gpu_mid):
    """hb_square = mult(a, a); hb_mul_const = product with the constant in every slot, one rescale."""
    g = gpu_mid
    rng = np.random.default_rng(21)
    z = rng.uniform(-1, 1, g.slots)
    ct = g.encrypt(g.encode(z, 5), 88)
    sq = g._op("square", ct.ptr)
    _same(g.ct_export(sq), g.ct_export(g.mul(ct, ct)), "square")
    assert np.abs(g.decrypt(sq).real - z * z).max() < 1e-6
    mc = g._op("mul_const", ct.ptr, C.c_double(0.25), C.c_double(-0.5))
    _same(g.ct_export(mc), g.ct_export(g.mul_pt(ct, g.encode(np.full(g.slots, 0.25 - 0.5j), 5))), "mul_const")
    assert np.abs(g.decrypt(mc) - z * (0.25 - 0.5j)).max() < 1e-6
