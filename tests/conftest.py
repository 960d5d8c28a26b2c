import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def nrmse(ref, got):
    """Normalised RMSE = ||got-ref|| / ||ref|| in FP64 (the reference's relative-L2 metric,
    src/fast_delta_rule/validation.py:40-45)."""
    import torch
    ref = ref.detach().double().cpu()
    got = got.detach().double().cpu()
    return ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()
