"""The oracle's schedule restatement against float64 matrix products (reference tolerance 2^-14)."""
import pytest

import cases

TOL = 2.0 ** -14


@pytest.fixture(scope="module")
def H(pkg, orc_small):
    return pkg.Hemmer(orc_small)


@pytest.mark.parametrize("name", sorted(cases.SCENARIOS))
def test_scenario_semantics(name, orc_small, H):
    _, err = cases.SCENARIOS[name](orc_small, H)
    assert err < TOL, (name, err)


def test_shape_and_level_errors(pkg, orc_small, H):
    import numpy as np
    d = cases.tile_dim(orc_small)
    a = H.encrypt(np.zeros((d, d)), nonce=90)
    b = H.encrypt2(np.zeros((d, d)), np.zeros((d, d)), nonce=91)
    with pytest.raises(pkg.HBError):  # different block width (MatrixUtils.cpp:33-40)
        H.single_cc_matmul(a, b, 2)
    low = pkg.CtxtTensor(orc_small.level_down(a.ct, 3), d, d)
    with pytest.raises(pkg.HBError):  # level guard (MatrixUtils.cpp:1320-1324)
        H.single_cc_matmul(low, low, 2)


DIRECT = ["transforms", "ccmm_two_tiles", "pcmm_reuse", "cc_reuse", "packed", "packed_reuse"]


@pytest.mark.parametrize("name", DIRECT)
def test_direct_schedule_semantics(name, pkg, orc_small):
    """The direct-rotation variant (every shifted copy is one rotation of the transformed operand) computes the same products."""
    Hd = pkg.Hemmer(orc_small)
    Hd.set_schedule(1)
    exports_d, err = cases.SCENARIOS[name](orc_small, Hd)
    assert err < TOL, (name, err)
    Hf = pkg.Hemmer(orc_small)
    exports_f, _ = cases.SCENARIOS[name](orc_small, Hf)
    import numpy as np
    assert any(not np.array_equal(a, b) for a, b in zip(exports_d, exports_f)), "variants are expected to differ in bits"


@pytest.mark.parametrize("name", ["ccmm_single_tile", "ccmm_two_tiles", "pcmm_reuse", "batched"])
def test_lazy_schedule_semantics(name, pkg, orc_small):
    """Schedule 2: each wrapped copy is one assemble_rot (one division by P * q_level); same products, other bits."""
    Hl = pkg.Hemmer(orc_small)
    Hl.set_schedule(2)
    exports_l, err = cases.SCENARIOS[name](orc_small, Hl)
    assert err < TOL, (name, err)
    Hd = pkg.Hemmer(orc_small)
    Hd.set_schedule(1)
    exports_d, _ = cases.SCENARIOS[name](orc_small, Hd)
    import numpy as np
    assert any(not np.array_equal(a, b) for a, b in zip(exports_l, exports_d))


def test_assemble_rot_semantics(orc_small):
    """p1 (.) rot(x, s1) + p2 (.) rot(x, s2) at every level, against the slot arithmetic and the unfused sequence."""
    import numpy as np
    o = orc_small
    rng = np.random.default_rng(3)
    z = rng.uniform(-1, 1, o.slots) + 1j * rng.uniform(-1, 1, o.slots)
    m1 = (rng.uniform(0, 1, o.slots) > 0.5).astype(float)
    o.gen_rot_keys([3, -13])
    want = m1 * np.roll(z, -3) + (1 - m1) * np.roll(z, 13)
    for lvl in range(o.L, 0, -1):
        ct = o.encrypt(o.encode(z, o.L), 5)
        if lvl < o.L:
            ct = o.level_down(ct, lvl)
        a = o.assemble_rot(ct, 3, o.encode_ext(m1, lvl), -13, o.encode_ext(1 - m1, lvl))
        assert o.ct_meta(a) == (lvl - 1, 2, 1, 1)
        ref = o.rescale(o.add(o.mul_pt_norescale(o.rotate(ct, 3), o.encode(m1, lvl)), o.mul_pt_norescale(o.rotate(ct, -13), o.encode(1 - m1, lvl))))
        err, err_ref = np.abs(o.decrypt(a) - want).max(), np.abs(o.decrypt(ref) - want).max()
        assert err < 4 * err_ref + 1e-9, (lvl, err, err_ref)


def test_rotate_sum_semantics(orc_small):
    """sum_t rot(x_t, s_t) with one ModDown decrypts to the sum of the rotated messages."""
    import numpy as np
    o = orc_small
    rng = np.random.default_rng(4)
    steps = [0, 3, -13, 40]
    o.gen_rot_keys(steps)
    zs = [rng.uniform(-1, 1, o.slots) + 1j * rng.uniform(-1, 1, o.slots) for _ in steps]
    for lvl in (o.L, 4, 1):
        xs = [o.encrypt(o.encode(z, o.L), 50 + i) for i, z in enumerate(zs)]
        if lvl < o.L:
            xs = [o.level_down(x, lvl) for x in xs]
        want = sum(np.roll(z, -s) for z, s in zip(zs, steps))
        got = o.decrypt(o.rotate_sum(xs, steps))
        ref = o.decrypt(o.add(o.add(xs[0], o.rotate(xs[1], 3)), o.add(o.rotate(xs[2], -13), o.rotate(xs[3], 40))))
        assert np.abs(got - want).max() < 2 * np.abs(ref - want).max() + 1e-9
