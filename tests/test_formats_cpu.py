"""The weight tilings of the reference's checkpoint converter (ciphertext/convert.py:34-53) as numpy."""
import importlib

import numpy as np
import pytest


def test_convert_matches_the_torch_expression():
    torch = pytest.importorskip("torch")
    fm = importlib.import_module("encryption-friendly_llm_architecture_b200.formats")
    rng = np.random.default_rng(0)
    for height, width in ((768, 768), (768, 3072), (3072, 768)):
        w = rng.normal(size=(width, height))                      # nn.Linear layout: [out, in]
        want = torch.from_numpy(w).transpose(0, 1).view(height // 128, 128, width // 128, 128).transpose(1, 2).numpy()
        got = fm.convert(w, height, width)
        assert got.shape == (height // 128, width // 128, 128, 128) and np.array_equal(got, want)
        # tile (i, j) is the block the layer multiplies input tile i with for output tile j
        assert np.array_equal(got[1, 2], w.T[128:256, 256:384])
    with pytest.raises(ValueError):
        fm.convert(np.zeros((10, 20)), 768, 768)


def test_convert_norm_repeats_the_vector_over_the_token_rows():
    fm = importlib.import_module("encryption-friendly_llm_architecture_b200.formats")
    v = np.arange(768, dtype=np.float64)
    t = fm.convert_norm(v)
    assert t.shape == (6, 128, 128)
    for k in range(6):
        assert np.array_equal(t[k], np.tile(v[128 * k:128 * (k + 1)], (128, 1)))
