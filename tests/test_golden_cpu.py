"""The oracle against the committed fixtures (tests/golden/golden.json, produced by tests/golden/make_golden.py)."""
import hashlib
import json
import os

import numpy as np
import pytest

import cases
from conftest import ROOT

GOLDEN = os.path.join(ROOT, "tests", "golden", "golden.json")


def digest(arr):
    return hashlib.sha256(np.ascontiguousarray(arr, dtype=np.uint64).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def golden():
    return json.load(open(GOLDEN))


@pytest.mark.parametrize("name", sorted(cases.SCENARIOS))
def test_oracle_reproduces_small_fixtures(name, golden, pkg, orc_small):
    exports, err = cases.SCENARIOS[name](orc_small, pkg.Hemmer(orc_small))
    assert [digest(e) for e in exports] == golden["small"][name]["digests"]
    assert err < 2.0 ** -14


def test_full_size_fixture_is_within_tolerance(golden):
    """The full-size 128x128 ct x ct product recorded by the generator met the reference's 2^-14 tolerance."""
    assert golden["full"]["config1_ccmm_128"]["max_abs_err"] < 2.0 ** -14
    assert len(golden["full"]["primes"]) == 16 and golden["full"]["primes"][0] < 2 ** 60
