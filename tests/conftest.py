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
