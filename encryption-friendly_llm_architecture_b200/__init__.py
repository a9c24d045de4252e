"""B200-native HEMMer: CKKS homomorphic matrix multiplication behind the reference's call surface.

The package is a thin Python mirror over two native libraries built in-tree:
``libhemmer_b200.so`` (sm_100a kernels + C ABI) and ``libhellm_b200.so`` (C++ HEMMer schedules).
Importing it never computes anything on the CPU; opening a context without a CUDA device fails.
"""
from __future__ import annotations

import ctypes
import os

from . import capi
from .capi import HBError, Lib, Params, make_params
from .hemmer import CtxtTensor, Hemmer, PtxtTensor

_HERE = os.path.dirname(os.path.abspath(__file__))
CUDA_LIB = os.path.join(_HERE, "libhemmer_b200.so")
HELLM_LIB = os.path.join(_HERE, "libhellm_b200.so")


def open_gpu(params: Params | None = None, device: int = 0) -> Lib:
    """Create a context on ``device``.  Raises if the CUDA library is missing or no GPU answers."""
    if not os.path.exists(CUDA_LIB):
        raise HBError(-5, f"{CUDA_LIB} not built: run `python __graft_entry__.py` (needs nvcc, sm_100a)")
    return Lib(CUDA_LIB, "hb_", params if params is not None else make_params(), device)


def open_hemmer(lib: Lib) -> Hemmer:
    """HELLM::HEMMer over an open GPU context."""
    if not os.path.exists(HELLM_LIB):
        raise HBError(-5, f"{HELLM_LIB} not built")
    ctypes.CDLL(CUDA_LIB, mode=ctypes.RTLD_GLOBAL)
    return Hemmer(lib, ctypes.CDLL(HELLM_LIB), "hb_hemmer_")
