"""CUDA library vs CPU oracle through the C ABI: ciphertext residues must be bit-identical."""
import numpy as np
import pytest

import cases
from conftest import rand_ct_residues

pytestmark = pytest.mark.gpu
TOL = 2.0 ** -14


def _same(a, b, what=""):
    assert a.shape == b.shape, what
    if not np.array_equal(a, b):
        bad = np.argwhere(a != b)
        raise AssertionError(f"{what}: {len(bad)} of {a.size} residues differ, first at {bad[0].tolist()}")


def _pairs(request, size):
    return request.getfixturevalue(f"gpu_{size}"), request.getfixturevalue(f"orc_{size}")


@pytest.mark.parametrize("size", ["small", "mid", "full"])
def test_context_tables(request, size):
    g, o = _pairs(request, size)
    assert np.array_equal(g.primes, o.primes)
    assert np.array_equal(g.scales, o.scales)


@pytest.mark.parametrize("size", ["small", "mid", "full"])
def test_ntt_roundtrip_and_parity(request, size):
    g, o = _pairs(request, size)
    lvl = g.L
    data = rand_ct_residues(g, lvl, 2, 3, seed=1)
    cg, co = g.ct_create(lvl, 2, 3), o.ct_create(lvl, 2, 3)
    g.ct_import(cg, data); o.ct_import(co, data)
    g.ntt(cg); o.ntt(co)
    _same(g.ct_export(cg), o.ct_export(co), "forward NTT")
    g.ntt(cg, inverse=True)
    _same(g.ct_export(cg), data, "inverse NTT round trip")
    g.ct_import(cg, data); g.ntt(cg, inverse=True); o.ct_import(co, data); o.ntt(co, inverse=True)
    _same(g.ct_export(cg), o.ct_export(co), "inverse NTT")


@pytest.mark.parametrize("size", ["small", "mid", "full"])
def test_keys_and_encryption(request, size):
    g, o = _pairs(request, size)
    for lib in (g, o):
        lib.gen_rot_keys([1, -3])
    for gal in (0, g.galois(1), g.galois(-3), 2 * g.N - 1):
        _same(g.evk_export(gal), o.evk_export(gal), f"switching key {gal}")
    rng = np.random.default_rng(2)
    z = rng.uniform(-1, 1, g.slots) + 1j * rng.uniform(-1, 1, g.slots)
    for lvl in (g.L, 2):
        pg, po = g.encode(z, lvl), o.encode(z, lvl)
        _same(g.pt_export(pg), o.pt_export(po), "encode")
        assert np.array_equal(g.decode(pg), o.decode(po))
        cg, co = g.encrypt(pg, 77), o.encrypt(po, 77)
        _same(g.ct_export(cg), o.ct_export(co), "encrypt")
        dg, do = g.decrypt(cg), o.decrypt(co)
        assert np.array_equal(dg, do) and np.abs(dg - z).max() < 1e-6


def _primitive_sweep(g, o, lvl, batch, seed):
    data = rand_ct_residues(g, lvl, 2, batch, seed)
    data2 = rand_ct_residues(g, lvl, 2, batch, seed + 1)
    cg, co = g.ct_create(lvl, 2, batch), o.ct_create(lvl, 2, batch)
    cg2, co2 = g.ct_create(lvl, 2, batch), o.ct_create(lvl, 2, batch)
    g.ct_import(cg, data); o.ct_import(co, data); g.ct_import(cg2, data2); o.ct_import(co2, data2)
    z = np.random.default_rng(seed).uniform(-1, 1, g.slots)
    pg, po = g.encode(z, lvl), o.encode(z, lvl)
    ops = [("add", lambda L, a, b, p: L.add(a, b)), ("sub", lambda L, a, b, p: L.sub(a, b)), ("negate", lambda L, a, b, p: L.negate(a)),
           ("mult_imag", lambda L, a, b, p: L.mult_imag(a)), ("mult_int", lambda L, a, b, p: L.mult_int(a, -12345)),
           ("mul_pt_norescale", lambda L, a, b, p: L.mul_pt_norescale(a, p)), ("tensor", lambda L, a, b, p: L.tensor(a, b)),
           ("conjugate", lambda L, a, b, p: L.conjugate(a))]
    for s in (1, 128 % g.slots, 4096 % g.slots):
        ops.append((f"rotate{s}", lambda L, a, b, p, s=s: L.rotate(a, s)))
    if lvl >= 1:
        ops += [("mul_pt", lambda L, a, b, p: L.mul_pt(a, p)), ("mul", lambda L, a, b, p: L.mul(a, b)),
                ("tensor+relin", lambda L, a, b, p: L.relin(L.tensor(a, b))), ("rescale", lambda L, a, b, p: L.rescale(L.mul_pt_norescale(a, p))),
                ("level_down", lambda L, a, b, p: L.level_down(a, max(lvl - 2, 0)))]
    for name, f in ops:
        rg, ro = f(g, cg, cg2, pg), f(o, co, co2, po)
        assert g.ct_meta(rg) == o.ct_meta(ro), name
        _same(g.ct_export(rg), o.ct_export(ro), f"{name} @ level {lvl}")


@pytest.mark.parametrize("size,levels,batch", [("small", (8, 5, 2, 1, 0), 2), ("mid", (8, 4, 1), 2), ("full", (12, 8, 4, 1), 2)])
def test_primitive_sweep(request, size, levels, batch):
    g, o = _pairs(request, size)
    for lib in (g, o):
        lib.gen_rot_keys([1, 128 % g.slots, 4096 % g.slots])
    for lvl in levels:
        _primitive_sweep(g, o, lvl, batch, seed=10 + lvl)


@pytest.mark.parametrize("size", ["small", "mid"])
@pytest.mark.parametrize("name", sorted(cases.SCENARIOS))
def test_schedule_parity(request, pkg, size, name):
    g, o = _pairs(request, size)
    Hg, Ho = pkg.open_hemmer(g), pkg.Hemmer(o)
    eg, err_g = cases.SCENARIOS[name](g, Hg)
    eo, err_o = cases.SCENARIOS[name](o, Ho)
    assert len(eg) == len(eo)
    for k, (a, b) in enumerate(zip(eg, eo)):
        _same(a, b, f"{name}[{k}]")
    assert err_g < TOL and err_g == err_o


@pytest.mark.parametrize("size", ["small", "mid"])
@pytest.mark.parametrize("name", ["transforms", "ccmm_two_tiles", "pcmm_reuse", "cc_reuse", "packed", "packed_reuse", "batched"])
def test_direct_schedule_parity(request, pkg, size, name):
    """Hoisted rotations on the GPU against plain direct rotations in the oracle: bit-identical."""
    g, o = _pairs(request, size)
    Hg, Ho = pkg.open_hemmer(g), pkg.Hemmer(o)
    Hg.set_schedule(1); Ho.set_schedule(1)
    eg, err_g = cases.SCENARIOS[name](g, Hg)
    eo, err_o = cases.SCENARIOS[name](o, Ho)
    for k, (a, b) in enumerate(zip(eg, eo)):
        _same(a, b, f"direct {name}[{k}]")
    assert err_g < TOL and err_g == err_o


@pytest.mark.parametrize("size", ["small", "mid"])
@pytest.mark.parametrize("name", ["ccmm_single_tile", "ccmm_two_tiles", "pcmm_reuse", "batched", "lora_forward"])
def test_lazy_schedule_parity(request, pkg, size, name):
    """Schedule 2 (one division by P * q_level per wrapped copy) on the GPU against the oracle's assemble_rot: bit-identical."""
    g, o = _pairs(request, size)
    Hg, Ho = pkg.open_hemmer(g), pkg.Hemmer(o)
    Hg.set_schedule(2); Ho.set_schedule(2)
    eg, err_g = cases.SCENARIOS[name](g, Hg)
    eo, err_o = cases.SCENARIOS[name](o, Ho)
    for k, (a, b) in enumerate(zip(eg, eo)):
        _same(a, b, f"lazy {name}[{k}]")
    assert err_g < TOL and err_g == err_o


@pytest.mark.parametrize("size", ["small", "mid", "full"])
def test_assemble_rot_parity(request, size):
    """The masked pair of rotations with one division, at every digit count, on random residues and a batch of 2."""
    g, o = _pairs(request, size)
    steps = (3, -5)
    for lib in (g, o):
        lib.gen_rot_keys(list(steps))
    rng = np.random.default_rng(31)
    m1 = (rng.uniform(0, 1, g.slots) > 0.5).astype(np.float64)
    levels = (g.L, 7, 4, 2, 1) if size != "full" else (g.L, 6, 1)
    for lvl in levels:
        data = rand_ct_residues(g, lvl, 2, 2, seed=40 + lvl)
        outs = []
        for lib in (g, o):
            ct = lib.ct_create(lvl, 2, 2)
            lib.ct_import(ct, data)
            r = lib.assemble_rot(ct, steps[0], lib.encode_ext(m1, lvl), steps[1], lib.encode_ext(1.0 - m1, lvl))
            assert lib.ct_meta(r) == (lvl - 1, 2, 2, 1)
            outs.append(lib.ct_export(r))
        _same(outs[0], outs[1], f"assemble_rot@{lvl}")


def test_assemble_rot_argument_errors(pkg, gpu_small):
    g = gpu_small
    g.gen_rot_keys([1, 2])
    ct = g.ct_create(3, 2, 1)
    g.ct_zero(ct)
    ones = np.ones(g.slots)
    with pytest.raises(pkg.HBError):  # plain (not extended) plaintext
        g.assemble_rot(ct, 1, g.encode(ones, 3), 2, g.encode_ext(ones, 3))
    with pytest.raises(pkg.HBError):  # plaintext of another level
        g.assemble_rot(ct, 1, g.encode_ext(ones, 4), 2, g.encode_ext(ones, 3))
    with pytest.raises(pkg.HBError):  # zero rotation
        g.assemble_rot(ct, 0, g.encode_ext(ones, 3), 2, g.encode_ext(ones, 3))


@pytest.mark.parametrize("size", ["mid", "full"])
def test_encrypt_many_equals_encrypt(request, size):
    """The batched encode + encrypt gives, member by member, the residues of hb_encode + hb_encrypt (and of the oracle)."""
    g, o = _pairs(request, size)
    rng = np.random.default_rng(56)
    msgs = rng.uniform(-1, 1, (3, g.slots))
    nonces = [901, 77, 4242]
    many = g.ct_export(g.encrypt_many(msgs, g.L, nonces))
    for i in range(3):
        _same(many[i:i + 1], g.ct_export(g.encrypt(g.encode(msgs[i], g.L), nonces[i])), f"encrypt_many[{i}]")
    _same(many[2:3], o.ct_export(o.encrypt(o.encode(msgs[2], o.L), nonces[2])), "encrypt_many vs oracle")
    cplx = msgs[:2] + 1j * msgs[1:3]
    many = g.ct_export(g.encrypt_many(cplx, 5, nonces[:2]))
    _same(many[1:2], g.ct_export(g.encrypt(g.encode(cplx[1], 5), nonces[1])), "encrypt_many complex, level 5")


def test_decrypt_many_equals_decrypt(gpu_mid):
    """One batched call gives, member by member, exactly the values of hb_decrypt (also with a level-0 member)."""
    g = gpu_mid
    rng = np.random.default_rng(55)
    zs = [rng.uniform(-1, 1, g.slots) + 1j * rng.uniform(-1, 1, g.slots) for _ in range(5)]
    cts = [g.encrypt(g.encode(z, g.L), 300 + i) for i, z in enumerate(zs)]
    cts[1] = g.level_down(cts[1], 3)
    cts[2] = g.mul_pt_norescale(cts[2], g.encode(np.ones(g.slots), g.L))   # scale Delta^2
    both = g.batch_concat([cts[3], cts[4]])
    items = [(cts[0], 0), (cts[1], 0), (cts[2], 0), (both, 1), (both, 0)]
    many = g.decrypt_many(items)
    for (ct, k), row in zip(items, many):
        assert np.array_equal(row, g.decrypt(ct, k))
    assert np.abs(many[3] - zs[4]).max() < 1e-6
    items.append((g.level_down(cts[0], 0), 0))
    many = g.decrypt_many(items)
    for (ct, k), row in zip(items, many):
        assert np.array_equal(row, g.decrypt(ct, k))


def test_hoisted_rotation_equals_rotation(gpu_mid):
    g = gpu_mid
    import ctypes as C
    g.gen_rot_keys([1, 7, -3])
    ct = g.ct_create(5, 2, 3)
    g.ct_import(ct, rand_ct_residues(g, 5, 2, 3, seed=77))
    dg = C.c_void_p()
    g._chk(g.dll.hb_decompose(g.ctx, ct.ptr, C.byref(dg)))
    try:
        for s in (1, 7, -3):
            out = C.c_void_p()
            g._chk(g.dll.hb_rotate_hoisted(g.ctx, ct.ptr, dg, C.c_int64(s), C.byref(out)))
            h = pkg_handle(g, out)
            _same(g.ct_export(h), g.ct_export(g.rotate(ct, s)), f"hoisted rotation by {s}")
    finally:
        g.dll.hb_digits_free.restype = None
        g.dll.hb_digits_free(dg)


def pkg_handle(lib, ptr):
    from importlib import import_module
    return import_module("encryption-friendly_llm_architecture_b200.capi").Handle(lib, ptr, "ct")


def test_full_size_golden_fixtures(pkg, gpu_full):
    """Full-size results against digests recorded from the oracle (no oracle run needed here):
    the primitive sweep cases and a single 128x128 ct x ct product with one tile per ciphertext."""
    import hashlib, json, os
    from conftest import ROOT
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "golden.json")))["full"]
    dg = lambda a: hashlib.sha256(np.ascontiguousarray(a, dtype=np.uint64).tobytes()).hexdigest()
    g = gpu_full
    assert [int(q) for q in g.primes] == gold["primes"]
    g.gen_rot_keys([1, 128, 4096])
    for lvl in (12, 4, 1):
        data = rand_ct_residues(g, lvl, 2, 1, seed=500 + lvl)
        ct = g.ct_create(lvl, 2, 1)
        g.ct_import(ct, data)
        pt = g.encode(np.random.default_rng(600 + lvl).uniform(-1, 1, g.slots), lvl)
        assert dg(g.ct_export(g.rotate(ct, 1))) == gold["primitives"][f"rotate1@{lvl}"]
        assert dg(g.ct_export(g.rotate(ct, 4096))) == gold["primitives"][f"rotate4096@{lvl}"]
        assert dg(g.ct_export(g.relin(g.tensor(ct, ct)))) == gold["primitives"][f"tensor_relin@{lvl}"]
        assert dg(g.ct_export(g.rescale(g.mul_pt_norescale(ct, pt)))) == gold["primitives"][f"rescale@{lvl}"]
        c2 = g.ct_create(lvl, 2, 1)
        g.ct_import(c2, data)
        g.ntt(c2)
        assert dg(g.ct_export(c2)) == gold["primitives"][f"ntt@{lvl}"]
    exports, err = cases.sc_ccmm_single_tile(g, pkg.open_hemmer(g), target=4)
    assert dg(exports[0]) == gold["config1_ccmm_128"]["digest"]
    assert err < TOL and err == gold["config1_ccmm_128"]["max_abs_err"]


def test_error_codes(pkg, gpu_small):
    g = gpu_small
    a = g.ct_create(3, 2, 1)
    b = g.ct_create(3, 3, 1)
    with pytest.raises(pkg.HBError) as e:
        g.sub(a, b)
    assert e.value.code == -3
    with pytest.raises(pkg.HBError) as e:
        g.rotate(a, 17)  # no key for this step
    assert e.value.code == -4
    with pytest.raises(pkg.HBError) as e:
        g.rescale(a)
    assert e.value.code == -3
    with pytest.raises(pkg.HBError) as e:
        g.mul_pt(a, g.encode(np.zeros(4), 5))
    assert e.value.code == -2


def test_masked_keys_give_the_residues_of_assemble_rot(gpu_mid):
    """hb_assemble_masked (masks folded into the keys) against hb_assemble_hoisted, two rotations and one."""
    import ctypes as C
    g = gpu_mid
    g.gen_rot_keys([3, -5])
    rng = np.random.default_rng(32)
    m1 = (rng.uniform(0, 1, g.slots) > 0.5).astype(np.float64)
    dll = g.dll
    dll.hb_digits_free.restype = None
    dll.hb_masked_key_free.restype = None
    for lvl in (g.L, 5, 1):
        ct = g.ct_create(lvl, 2, 2)
        g.ct_import(ct, rand_ct_residues(g, lvl, 2, 2, seed=60 + lvl))
        p1, p2 = g.encode_ext(m1, lvl), g.encode_ext(1.0 - m1, lvl)
        dg, k1, k2, k12 = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        g._chk(dll.hb_decompose(g.ctx, ct.ptr, C.byref(dg)))
        g._chk(dll.hb_masked_key_create(g.ctx, C.c_int64(3), p1.ptr, None, C.byref(k1)))
        g._chk(dll.hb_masked_key_create(g.ctx, C.c_int64(-5), p2.ptr, None, C.byref(k2)))
        g._chk(dll.hb_masked_key_create(g.ctx, C.c_int64(3), p1.ptr, p2.ptr, C.byref(k12)))
        try:
            out = C.c_void_p()
            g._chk(dll.hb_assemble_masked(g.ctx, ct.ptr, dg, k1, k2, C.byref(out)))
            _same(g.ct_export(pkg_handle(g, out)), g.ct_export(g.assemble_rot(ct, 3, p1, -5, p2)), f"masked pair@{lvl}")
            out = C.c_void_p()
            g._chk(dll.hb_assemble_masked(g.ctx, ct.ptr, dg, k12, None, C.byref(out)))
            _same(g.ct_export(pkg_handle(g, out)), g.ct_export(g.assemble_rot(ct, 3, p1, 3, p2)), f"masked single@{lvl}")
        finally:
            for k in (k1, k2, k12):
                dll.hb_masked_key_free(k)
            dll.hb_digits_free(dg)


@pytest.mark.parametrize("size", ["small", "mid", "full"])
def test_rotate_sum_parity(request, size):
    """Sum of rotations with one ModDown: rotated and unrotated terms, every digit count, batch of 2."""
    g, o = _pairs(request, size)
    steps = [0, 3, -5, 0, 17]
    for lib in (g, o):
        lib.gen_rot_keys(steps)
    levels = (g.L, 6, 3, 0) if size != "full" else (g.L, 5)
    for lvl in levels:
        outs = []
        for lib in (g, o):
            xs = []
            for t in range(len(steps)):
                ct = lib.ct_create(lvl, 2, 2)
                lib.ct_import(ct, rand_ct_residues(g, lvl, 2, 2, seed=70 + 10 * lvl + t))
                xs.append(ct)
            outs.append(lib.ct_export(lib.rotate_sum(xs, steps)))
            if lib is g and lvl == levels[0]:   # unrotated terms only: the plain sum
                _same(lib.ct_export(lib.rotate_sum([xs[0], xs[3]], [0, 0])), lib.ct_export(lib.add(xs[0], xs[3])), "rotate_sum of unrotated terms")
        _same(outs[0], outs[1], f"rotate_sum@{lvl}")
