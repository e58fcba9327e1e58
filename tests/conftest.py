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
