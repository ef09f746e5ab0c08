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
    value, target = value.detach().double().cpu(), target.detach().double().cpu()
    denom = float(target.norm())
    diff = float((value - target).norm())
    return diff if denom == 0.0 else diff / denom


# Rounding error of the Gram iteration on prescribed spectra (256 x 1024, as the reference's
# precision study does: bench/precision.py:31-117 there).  Its README lists, for an RTX 5090,
# 0.003 (Gaussian), 0.037 / 0.039 (geometric decay over 4 / 6 decades) and 0.030 / 0.052
# (rank 8 at 1, the rest at 1e-3 / 1e-4), other GPUs within 0.01.
PUBLISHED_ROUNDING = {"gaussian": 0.003, "geometric4": 0.037, "geometric6": 0.039, "lowrank3": 0.030,
                      "lowrank4": 0.052}


def spectrum_matrix(name: str) -> torch.Tensor:
    """A seeded ``[1, 256, 1024]`` fp32 matrix with the named singular values."""
    rows, cols = 256, 1024
    gen = torch.Generator().manual_seed(0)
    if name == "gaussian":
        return torch.randn(1, rows, cols, generator=gen)
    left, _ = torch.linalg.qr(torch.randn(rows, rows, dtype=torch.float64, generator=gen))
    right, _ = torch.linalg.qr(torch.randn(cols, rows, dtype=torch.float64, generator=gen))
    if name.startswith("geometric"):
        values = torch.logspace(0, -int(name[-1]), rows, dtype=torch.float64)
    else:
        values = torch.full((rows,), 10.0 ** -int(name[-1]), dtype=torch.float64)
        values[:8] = 1.0
    return ((left * values) @ right.mT).float()[None]
