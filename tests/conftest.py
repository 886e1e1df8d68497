import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
MEAN = (0.485, 0.456, 0.406)
STD = (0.229, 0.224, 0.225)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def fused_golden():
    return np.load(os.path.join(GOLDEN, "fused_cases.npz"))


@pytest.fixture(scope="session")
def functional_golden():
    return np.load(os.path.join(GOLDEN, "functional_cases.npz"))


@pytest.fixture(scope="session")
def class_golden():
    return np.load(os.path.join(GOLDEN, "class_cases.npz"))


def fused_case(z, name):
    """One record of fused_cases.npz as a dict."""
    pre = name + "|"
    return {k[len(pre):]: z[k] for k in z.files if k.startswith(pre)}
