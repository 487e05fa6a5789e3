"""Shared pytest configuration: the ``gpu`` marker, repository imports and golden-fixture loaders."""

import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the sm_100a kernels through the C-ABI)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="CUDA device required")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def reference_tables():
    with open(os.path.join(GOLDEN, "reference_tables.json")) as handle:
        return json.load(handle)


@pytest.fixture(scope="session")
def golden_npz():
    def load(name):
        return np.load(os.path.join(GOLDEN, name))

    return load
