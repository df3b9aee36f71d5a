import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "thor-fp4_b200", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="needs a CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)
    np.random.seed(0)


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN / "ref_fakequant.npz")


def rrms(a, b):
    a, b = a.float(), b.float()
    return ((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt().clamp_min(1e-30)).item()


def bits_to_f32(bits: np.ndarray, kind: str) -> np.ndarray:
    """uint16 bit patterns of f16 / bf16 values -> float32 (exact)."""
    if kind == "f16":
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def bits_to_torch(bits: np.ndarray, kind: str, device="cpu") -> torch.Tensor:
    t = torch.from_numpy(bits.view(np.int16).copy()).to(device)
    return t.view(torch.float16 if kind == "f16" else torch.bfloat16)
