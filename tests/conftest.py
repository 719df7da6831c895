"""Shared pytest configuration: markers, import paths and golden-vector loading."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE = os.path.join(ROOT, "gptq-2d_b200")
for path in (PACKAGE, ROOT):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    return np.load(os.path.join(ROOT, "tests", "golden", name))


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), compiled on first use."""
    from oracle import oracle as module

    module.lib()
    return module
