"""Shared test plumbing: the ``gpu`` marker, import path, seeded inputs."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    """Skip GPU tests when no device is visible and they were not deselected."""
    try:
        import torch

        available = torch.cuda.is_available()
    except Exception:  # pragma: no cover - torch is part of the image
        available = False
    if available:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def rng():
    return np.random.default_rng(705537)
