"""Shared pytest set-up: markers, import paths, fixtures."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (ROOT, os.path.join(ROOT, "tiga-lang_b200")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the unmodified reference on small seeded cases
    (tests/golden/make_golden.py wrote them)."""
    path = os.path.join(ROOT, "tests", "golden", "reference_cases.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as module
    module.build()
    return module


def assert_sum_close(got, ref, magnitude, *, rtol=1e-5, atol=1e-6, ulps=8, equal_nan=False):
    """float32 sums: rel 1e-5 / abs 1e-6, plus the rounding that a different
    summation order may legitimately introduce: `ulps` float32 ulps of the sum of
    absolute values of the terms (`magnitude`).  Rows whose terms are added in the
    reference's order are still checked bit for bit by the tests that call this."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    bound = rtol * np.abs(ref) + atol + ulps * np.finfo(np.float32).eps * np.asarray(magnitude, dtype=np.float64)
    error = np.abs(got - ref)
    if equal_nan:
        both_nan = np.isnan(got) & np.isnan(ref)
        error = np.where(both_nan, 0.0, error)
        bound = np.where(both_nan, 1.0, bound)
    bad = ~(error <= bound)
    assert not bad.any(), f"{bad.sum()} of {bad.size} elements differ; worst excess {np.nanmax(error - bound)}"
