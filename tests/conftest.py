import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN_DIR = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _library_is_built():
    """Build libkda_b200.so once if a fresh checkout has none (it is not part of the history)."""
    from kda_ascendc_b200 import build as kda_build
    if not kda_build.LIB_PATH.exists():
        kda_build.build()


def golden_cases():
    return sorted(p.stem for p in GOLDEN_DIR.glob("*.pt"))


def load_golden(name):
    return torch.load(GOLDEN_DIR / f"{name}.pt", weights_only=True)


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


def to_device(inp: dict, device):
    return {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in inp.items()}
