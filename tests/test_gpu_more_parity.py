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
@pytest.mark.parametrize("name", ["packed", "packed_reuse", "cc_reuse", "transforms", "single_matmul", "lora_backward", "transpose_packing", "repack_lora_opti", "gaussian_kernel", "tr_rot_sum", "masks_and_sums"])
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


@pytest.mark.parametrize("tiles", [1, 2, 5, 7])
def test_tile_batched_accumulate_equals_tile_by_tile(pkg, gpu_mid, tiles):
    """hb_matmul_acc_tiles (shifted copies read once per four output tiles, FP64 products, with the 60-bit limb on the
    integer path) against hb_matmul_acc_multi called per tile: identical residues."""
    g = gpu_mid
    rng = np.random.default_rng(60 + tiles)
    copies, groups, lvl = 16, 3, 3
    data = np.empty((copies * groups, 2, lvl + 1, g.N), dtype=np.uint64)
    for l in range(lvl + 1):
        data[:, :, l, :] = rng.integers(0, int(g.primes[l]), size=(copies * groups, 2, g.N), dtype=np.uint64)
    data[0, :, :, :] = np.array([int(q) - 1 for q in g.primes[: lvl + 1]], dtype=np.uint64)[None, :, None]   # worst-case words
    pre = g.ct_create(lvl, 2, copies * groups)
    g.ct_import(pre, data)
    pts = [[g.encode(rng.uniform(-1, 1, g.slots), lvl) for _ in range(2)] for _ in range(tiles)]
    arr = (C.c_void_p * (tiles * 2))(*[p.ptr.value for row in pts for p in row])
    outs = (C.c_void_p * tiles)()
    g._chk(g.dll.hb_matmul_acc_tiles(g.ctx, pre.ptr, C.c_int(groups), C.c_int(1), arr, C.c_int(2), C.c_int(tiles), C.c_int64(32), outs))
    for t in range(tiles):
        one = C.c_void_p()
        row = (C.c_void_p * 2)(*[p.ptr.value for p in pts[t]])
        g._chk(g.dll.hb_matmul_acc_multi(g.ctx, pre.ptr, C.c_int(groups), C.c_int(1), row, C.c_int(2), C.c_int64(32), C.byref(one)))
        _same(g.ct_export(pkg.capi.Handle(g, C.c_void_p(outs[t]), "ct")), g.ct_export(pkg.capi.Handle(g, one, "ct")), f"tile {t}")


def test_part_sums_and_grouped_rotate_sum_equal_the_term_by_term_calls(pkg, gpu_mid):
    """hb_mul_pt_sum_parts against hb_sum_mul_pt_rescale per part (parts with different term sets, one of a single term),
    then hb_rotate_sum_grouped on the part-major result against hb_rotate_sum on the separate parts."""
    g = gpu_mid
    rng = np.random.default_rng(77)
    lvl, terms, parts, batch = 4, 6, 5, 3
    cts = []
    for j in range(terms):
        data = rand_ct_residues(g, lvl, 2, batch, seed=300 + j)
        ct = g.ct_create(lvl, 2, batch)
        g.ct_import(ct, data)
        cts.append(ct)
    use = [[0], [1, 2, 3], [1, 2, 3, 4, 5], [2], [3, 4]]
    masks = [{j: g.encode(rng.uniform(-1, 1, g.slots), lvl) for j in use[p]} for p in range(parts)]
    a = (C.c_void_p * terms)(*[c.ptr.value for c in cts])
    pp = (C.c_void_p * (parts * terms))(*[masks[p][j].ptr.value if j in masks[p] else None for p in range(parts) for j in range(terms)])
    out = C.c_void_p()
    g._chk(g.dll.hb_mul_pt_sum_parts(g.ctx, a, pp, C.c_int(terms), C.c_int(parts), C.byref(out)))
    grouped = pkg.capi.Handle(g, out, "ct")
    got = g.ct_export(grouped)
    singles = []
    for p in range(parts):
        aa = (C.c_void_p * len(use[p]))(*[cts[j].ptr.value for j in use[p]])
        mm = (C.c_void_p * len(use[p]))(*[masks[p][j].ptr.value for j in use[p]])
        one = C.c_void_p()
        g._chk(g.dll.hb_sum_mul_pt_rescale(g.ctx, aa, mm, C.c_int(len(use[p])), C.byref(one)))
        singles.append(pkg.capi.Handle(g, one, "ct"))
        _same(got[p * batch:(p + 1) * batch], g.ct_export(singles[-1]), f"part {p}")
    steps = [0, 3, -5, 64, 7]
    g.gen_rot_keys([s for s in steps if s])
    st = (C.c_int64 * parts)(*steps)
    r1, r2 = C.c_void_p(), C.c_void_p()
    g._chk(g.dll.hb_rotate_sum_grouped(g.ctx, grouped.ptr, st, C.c_int(parts), C.byref(r1)))
    xs = (C.c_void_p * parts)(*[s.ptr.value for s in singles])
    g._chk(g.dll.hb_rotate_sum(g.ctx, xs, st, C.c_int(parts), C.byref(r2)))
    _same(g.ct_export(pkg.capi.Handle(g, r1, "ct")), g.ct_export(pkg.capi.Handle(g, r2, "ct")), "grouped rotate-sum")


def test_tile_batched_accumulate_many_terms_with_44_bit_primes(pkg):
    """The signed double sums of hb_matmul_acc_tiles at their fold limit: every residue q - 1 (each product is then as far
    from zero as it gets), 512 copies x 2 groups = 1024 terms per output, primes just below 2^44, ring degree 2^10 ... the
    tile kernel needs 512 coefficients per CTA, so N = 2^10 gives two CTAs per limb."""
    prm = dict(log_n=10, max_level=3, dnum=2, num_special=3, hamming_weight=32, q_bits=44)
    g = pkg.open_gpu(pkg.make_params(**prm))
    g.keygen()
    copies, groups, lvl, tiles = 512, 2, 2, 3
    data = np.empty((copies * groups, 2, lvl + 1, g.N), dtype=np.uint64)
    for l in range(lvl + 1):
        data[:, :, l, :] = np.uint64(int(g.primes[l]) - 1)
    pre = g.ct_create(lvl, 2, copies * groups)
    g.ct_import(pre, data)
    rng = np.random.default_rng(5)
    pts = [[g.encode(rng.uniform(-1, 1, g.slots), lvl) for _ in range(groups)] for _ in range(tiles)]
    arr = (C.c_void_p * (tiles * groups))(*[p.ptr.value for row in pts for p in row])
    outs = (C.c_void_p * tiles)()
    g._chk(g.dll.hb_matmul_acc_tiles(g.ctx, pre.ptr, C.c_int(groups), C.c_int(0), arr, C.c_int(groups), C.c_int(tiles), C.c_int64(0), outs))
    for t in range(tiles):
        got = g.ct_export(pkg.capi.Handle(g, C.c_void_p(outs[t]), "ct"))
        w = [g.pt_export(p) for p in pts[t]]
        for l in range(lvl + 1):
            q = int(g.primes[l])
            want = np.array([(copies * (q - 1) * (int(a) + int(b))) % q for a, b in zip(w[0][l], w[1][l])], dtype=np.uint64)
            assert np.array_equal(got[0, 0, l], want) and np.array_equal(got[0, 1, l], want), f"tile {t} limb {l}"
