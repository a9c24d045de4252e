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
