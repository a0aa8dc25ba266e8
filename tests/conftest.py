"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on a
CPU-only machine (the native library still has to be built: it is cross-compiled
by nvcc and loads without a GPU)."""
import os
import sys
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
GOLDEN = REPO / "tests" / "golden"
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")
    # Test modules import the ctypes binding at import time, i.e. during collection: the native
    # library has to exist before that (a fresh checkout has none; it is not kept in version control).
    from att3ntion_b200 import build
    build.build()


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_files(prefix):
    return sorted(p.name for p in GOLDEN.glob(f"{prefix}*.pt"))


def load_golden(name):
    return torch.load(GOLDEN / name, map_location="cpu", weights_only=False)
