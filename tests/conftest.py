from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    """The shipped package, loaded under its importable alias."""
    return entry.load_package()


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "hotpath_golden.npz")


@pytest.fixture(scope="session")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().to("cpu", torch.float64)
    b = b.detach().to("cpu", torch.float64)
    denom = float(b.norm())
    return float((a - b).norm()) / (denom if denom > 0 else 1.0)
