"""Shared test helpers.  GPU tests are marked ``gpu``; everything else runs on CPU."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (Blackwell sm_100)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def from_bf16_bits(arr: np.ndarray) -> torch.Tensor:
    """int16 bit patterns -> bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(arr)).view(torch.bfloat16)


def load_golden(name: str) -> dict:
    data = np.load(GOLDEN_DIR / f"{name}.npz")
    return {key: data[key] for key in data.files}


def randn_bf16(gen: torch.Generator, *shape) -> torch.Tensor:
    """Seeded N(0,1) bf16 tensor on the CPU."""
    return torch.randn(*shape, generator=gen).to(torch.bfloat16)
