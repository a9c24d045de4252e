"""Host-side data layouts of the reference's checkpoint converter, as plain numpy.

``convert`` is ciphertext/convert.py:34-45: a weight of shape [out, in] (PyTorch's nn.Linear layout) becomes
[in / 128, n / 128, 128, 128] -- tile (i, j) is rows 128 i .. of the TRANSPOSED weight (the input side) and columns
128 j .. (the output side), the tiles HEMMer::encodeDiagonalToRow4 packs four at a time.  ``convert_norm`` is
convert.py:48-53: a LayerNorm vector repeated over the 128 token rows and cut into [dim / 128, 128, 128].
Ciphertexts, plaintexts and keys use the library's own file container (hb_ct_save, hb_pt_save, hb_keys_save in
include/hemmer_b200.h); HEaaN's binary format is not published.
"""
from __future__ import annotations

import numpy as np

SUBMATRIX_DIM = 128
MAX_SEQ_LEN = 128


def convert(weight: np.ndarray, height: int, width: int) -> np.ndarray:
    """[width, height] weight (rows = outputs) -> [height / 128, width / 128, 128, 128] tiles of its transpose."""
    w = np.asarray(weight).T
    if w.shape != (height, width):
        raise ValueError(f"expected a [{width}, {height}] weight")
    t = w.reshape(height // SUBMATRIX_DIM, SUBMATRIX_DIM, width // SUBMATRIX_DIM, SUBMATRIX_DIM)
    return np.ascontiguousarray(t.transpose(0, 2, 1, 3))


def convert_norm(weight: np.ndarray) -> np.ndarray:
    """[dim] vector -> [dim / 128, 128 tokens, 128]: every token row carries the same slice."""
    w = np.asarray(weight)
    rep = np.tile(w, (MAX_SEQ_LEN, 1)).reshape(MAX_SEQ_LEN, w.size // SUBMATRIX_DIM, SUBMATRIX_DIM)
    return np.ascontiguousarray(rep.transpose(1, 0, 2))
