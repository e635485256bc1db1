"""Shared pytest configuration: the ``gpu`` marker, the golden fixtures, tolerance helpers."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box only)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    """Vectors produced by the reference's own CPU oracle (tests/golden/make_golden.py)."""
    return torch.load(os.path.join(ROOT, "tests", "golden", "golden.pt"), weights_only=True)


def max_rel(actual, expected):
    """Max abs error relative to the largest reference magnitude of the tensor (the
    per-tensor measure the reference's own kernel tests use, kernel/test_polar_kernel.py:108-111)."""
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    return ((a - e).abs().max() / e.abs().max().clamp_min(1e-12)).item()


def max_abs(actual, expected):
    return (actual.detach().float().cpu() - expected.detach().float().cpu()).abs().max().item()
