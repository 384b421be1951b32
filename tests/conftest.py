import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the sm_100a kernels)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    return torch.load(os.path.join(GOLDEN_DIR, name), weights_only=False)


def assert_same(a: torch.Tensor, b: torch.Tensor, what=""):
    """Bit-for-bit equality (NaNs in the same places count as equal; -0.0 == 0.0)."""
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} != {tuple(b.shape)}"
    assert a.dtype == b.dtype, f"{what}: dtype {a.dtype} != {b.dtype}"
    a, b = a.detach().cpu(), b.detach().cpu()
    same = (a == b) | (a.isnan() & b.isnan()) if a.is_floating_point() else (a == b)
    if not bool(same.all()):
        bad = (~same).nonzero()
        i = tuple(bad[0].tolist())
        raise AssertionError(
            f"{what}: {bad.shape[0]} of {a.numel()} elements differ; first at {i}: {a[i].item()!r} vs {b[i].item()!r}"
        )
