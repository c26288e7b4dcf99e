"""Shared test plumbing: the ``gpu`` marker, import paths, golden loaders."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


_FP8_KEYS = ("e0", "e1", "e2")


def load_golden(name: str, fp8_keys=()):
    """Load ``tests/golden/<name>.npz`` as a dict of torch tensors.  Arrays
    listed in ``fp8_keys`` were stored as raw bytes of float8_e5m2."""
    data = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for key in data.files:
        t = torch.from_numpy(data[key])
        if key in fp8_keys:
            t = t.view(torch.float8_e5m2)
        out[key] = t
    return out


@pytest.fixture(scope="session")
def golden():
    return load_golden


def reference_root():
    """Path of a carrykernel checkout if one is reachable, else None.  Only
    CPU tests use it, to re-check the oracle against the live reference."""
    for cand in (os.environ.get("CARRYKERNEL_REFERENCE"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "statequant", "kernel.py")):
            return cand
    return None
