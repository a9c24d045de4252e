"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes
import os
import re

from conftest import ROOT


def _declared(header):
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_header_symbols(pkg):
    names = _declared(os.path.join(ROOT, "include", "hemmer_b200.h"))
    assert len(names) > 40
    dll = ctypes.CDLL(pkg.CUDA_LIB)
    missing = [n for n in names if not hasattr(dll, n)]
    assert not missing, missing


def test_hellm_layer_exports(pkg):
    names = [n for n in _declared(os.path.join(ROOT, "include", "hellm_b200.h")) if n.startswith("hb_hemmer_")]
    assert len(names) > 35
    ctypes.CDLL(pkg.CUDA_LIB, mode=ctypes.RTLD_GLOBAL)
    dll = ctypes.CDLL(pkg.HELLM_LIB)
    missing = [n for n in names if not hasattr(dll, n)]
    assert not missing, missing


def test_no_gpu_means_loud_failure(pkg):
    """Without a CUDA device the product path must refuse to run rather than fall back."""
    import torch
    if torch.cuda.is_available():
        return
    try:
        pkg.open_gpu()
    except pkg.HBError as e:
        assert e.code != 0
    else:
        raise AssertionError("context creation succeeded without a GPU")
