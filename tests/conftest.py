import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def scmx():
    """The product package (directory name contains '-', so it is imported by name)."""
    return importlib.import_module("mxfp4-int8-m5_b200")


@pytest.fixture(scope="session")
def oracle():
    import scmx_oracle
    return scmx_oracle


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))


@pytest.fixture(scope="session")
def digests():
    out = {}
    with open(os.path.join(ROOT, "tests", "golden", "config1_digests.txt")) as fh:
        for line in fh:
            k, v = line.split()
            out[k] = v
    return out
