"""Shared test plumbing: the ``gpu`` marker, repo paths, fixture loading."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def load_golden(name: str) -> dict[str, torch.Tensor]:
    """Load ``tests/golden/<name>.npz``; ``__bf16`` entries come back as bfloat16."""
    out: dict[str, torch.Tensor] = {}
    with np.load(GOLDEN / f"{name}.npz") as data:
        for key in data.files:
            tensor = torch.from_numpy(data[key].copy())
            if key.endswith("__bf16"):
                out[key[: -len("__bf16")]] = tensor.view(torch.bfloat16)
            else:
                out[key] = tensor
    return out


def rel_l2(value: torch.Tensor, target: torch.Tensor) -> float:
    """``|value - target| / |target|`` in the Frobenius norm (0/0 counts as 0)."""
    value, target = value.double().cpu(), target.double().cpu()
    denom = float(target.norm())
    diff = float((value - target).norm())
    return diff if denom == 0.0 else diff / denom
