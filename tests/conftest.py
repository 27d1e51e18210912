"""Shared pytest configuration: the ``gpu`` marker, import paths and fixture loading."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
for p in (REPO, REPO / "mega-moe-td_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"
GOLDEN_CASES = ["w1_e8_k2", "w2_e8_k3_drop", "w4_e16_k4_zipf", "w8_e16_k4"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _tensor(a: np.ndarray) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.view(torch.bfloat16) if t.dtype == torch.int16 else t


class Golden:
    """One fixture written by tests/golden/make_golden.py: per-rank inputs and reference outputs."""

    def __init__(self, name: str):
        with np.load(GOLDEN_DIR / f"{name}.npz") as z:
            self.raw = {k: z[k] for k in z.files}
        (self.world, self.tokens, self.hidden, self.ffn, self.experts,
         self.top_k) = (int(v) for v in self.raw["meta"])

    def get(self, rank: int, key: str) -> torch.Tensor:
        return _tensor(self.raw[f"r{rank}_{key}"])

    def per_rank(self, key: str):
        return [self.get(r, key) for r in range(self.world)]


@pytest.fixture(params=GOLDEN_CASES)
def golden(request):
    return Golden(request.param)
