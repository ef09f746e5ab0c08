"""Per-device scratch arena for the transient buffers of a run.

One byte tensor per device, grown when a run needs more and reused by every
later run and step: runs execute one after another on one stream, so they can
share it, and the caching allocator is not asked for gigabytes every step.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

_ALIGN = 256
_arenas: dict[torch.device, Tensor] = {}


def _round(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


def carve(device: torch.device, plan: dict[str, tuple[tuple[int, ...], torch.dtype]]) -> dict[str, Tensor]:
    """Return one tensor per ``name -> (shape, dtype)`` entry, all views of the device's arena.

    The contents are whatever the previous run left there.
    """
    sizes = {name: _round(math.prod(shape) * dtype.itemsize) for name, (shape, dtype) in plan.items()}
    total = sum(sizes.values())
    arena = _arenas.get(device)
    if arena is None or arena.numel() < total:
        _arenas.pop(device, None)
        arena = torch.empty(max(total, 1 << 20), dtype=torch.uint8, device=device)
        _arenas[device] = arena
    out: dict[str, Tensor] = {}
    offset = 0
    for name, (shape, dtype) in plan.items():
        nbytes = math.prod(shape) * dtype.itemsize
        out[name] = arena[offset : offset + nbytes].view(dtype).view(shape)
        offset += sizes[name]
    return out


def release() -> None:
    """Drop every arena (tests, or before a memory-hungry phase)."""
    _arenas.clear()
