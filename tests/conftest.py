import importlib
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
PKG_NAME = "encryption-friendly_llm_architecture_b200"
ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "liboracle.so")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module(PKG_NAME)


@pytest.fixture(scope="session")
def oracle_so():
    if not os.path.exists(ORACLE_SO):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    return ORACLE_SO


SMALL = dict(log_n=10, max_level=8, dnum=3, num_special=3, hamming_weight=32)
MID = dict(log_n=12, max_level=8, dnum=3, num_special=3, hamming_weight=64)
FULL = dict()  # the benchmark parameter set: N=2^16, L=12, dnum=4, K=3


def open_oracle(pkg, oracle_so, **kw):
    return pkg.capi.Lib(oracle_so, "orc_", pkg.make_params(**kw))


@pytest.fixture(scope="session")
def orc_small(pkg, oracle_so):
    o = open_oracle(pkg, oracle_so, **SMALL)
    o.keygen()
    return o


@pytest.fixture(scope="session")
def gpu_small(pkg):
    g = pkg.open_gpu(pkg.make_params(**SMALL))
    g.keygen()
    return g


@pytest.fixture(scope="session")
def orc_mid(pkg, oracle_so):
    o = open_oracle(pkg, oracle_so, **MID)
    o.keygen()
    return o


@pytest.fixture(scope="session")
def gpu_mid(pkg):
    g = pkg.open_gpu(pkg.make_params(**MID))
    g.keygen()
    return g


@pytest.fixture(scope="session")
def orc_full(pkg, oracle_so):
    o = open_oracle(pkg, oracle_so, **FULL)
    o.keygen()
    return o


@pytest.fixture(scope="session")
def gpu_full(pkg):
    g = pkg.open_gpu(pkg.make_params(**FULL))
    g.keygen()
    return g


def rand_ct_residues(lib, level, n_poly, batch, seed):
    """Uniform residues below each prime, the inputs of the primitive sweep."""
    rng = np.random.default_rng(seed)
    out = np.empty((batch, n_poly, level + 1, lib.N), dtype=np.uint64)
    for l in range(level + 1):
        out[:, :, l, :] = rng.integers(0, int(lib.primes[l]), size=(batch, n_poly, lib.N), dtype=np.uint64)
    return out
