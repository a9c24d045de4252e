"""hb_rescale_noalloc: the rescale entry point for callers that cannot allocate device memory.

Some users of this library run under a device-memory budget that is handed out once, up front (or next to
another allocator they must leave alone) and so cannot let a call reach cudaMalloc.  For them the library
keeps the temporaries of one rescale in a buffer inside its own image.  The result must be the same as
hb_rescale's, also when the shared buffer still holds the previous call's data -- hence two calls in a row.
This file sorts last on purpose: a failure here must not hide the other tests under `pytest -x`.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import rand_ct_residues

pytestmark = pytest.mark.gpu


def _rescale_noalloc(g, src, level, n_poly=2, batch=1):
    out = g.ct_create(level - 1, n_poly, batch, 1)
    g._chk(g.dll.hb_rescale_noalloc(g.ctx, src.ptr, out.ptr))
    return out


@pytest.mark.parametrize("size", ["full", "small"])
def test_noalloc_rescale_matches_rescale_twice(request, size):
    g = request.getfixturevalue(f"gpu_{size}")
    for call, level in enumerate((g.L, 5)):
        src = g.ct_create(level, 2, 1, 2)
        g.ct_import(src, rand_ct_residues(g, level, 2, 1, seed=900 + call))
        want = g.ct_export(g.rescale(src))
        got = _rescale_noalloc(g, src, level)
        assert g.ct_meta(got) == (level - 1, 2, 1, 1)
        assert np.array_equal(g.ct_export(got), want), f"call {call} at level {level}"
        # the property the entry point exists for: with the output handle in place and the scratch address resolved,
        # a further call obtains no device memory, neither from the context's pool nor from the driver
        import torch
        pool, used = C.c_uint64(), C.c_uint64()
        g.dll.hb_mem_info(g.ctx, C.byref(pool), C.byref(used))
        before = (pool.value, used.value, torch.cuda.mem_get_info()[0])
        g._chk(g.dll.hb_rescale_noalloc(g.ctx, src.ptr, got.ptr))
        g.sync()
        g.dll.hb_mem_info(g.ctx, C.byref(pool), C.byref(used))
        assert (pool.value, used.value, torch.cuda.mem_get_info()[0]) == before, "hb_rescale_noalloc obtained device memory"
        assert np.array_equal(g.ct_export(got), want)


def test_noalloc_rejects_a_foreign_output_handle(pkg, gpu_full, gpu_small):
    src = gpu_small.ct_create(3, 2, 1, 2)
    gpu_small.ct_zero(src)
    out = gpu_full.ct_create(2, 2, 1, 1)
    assert gpu_small.dll.hb_rescale_noalloc(gpu_small.ctx, src.ptr, out.ptr) == -1


def test_noalloc_rejects_oversized_request(pkg, gpu_full):
    g = gpu_full
    src = g.ct_create(g.L, 2, 2, 2)  # two ciphertexts: twice the built-in scratch
    out = g.ct_create(g.L - 1, 2, 2, 1)
    rc = g.dll.hb_rescale_noalloc(g.ctx, src.ptr, out.ptr)
    assert rc == -9
    g.dll.hb_last_error.restype = C.c_char_p
    assert b"scratch" in g.dll.hb_last_error(g.ctx)
