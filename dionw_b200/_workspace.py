"""Per-device scratch arenas for the transient buffers of a run.

One byte tensor per (device, arena name), grown when a run needs more and
reused by every later run and step: runs execute one after another on one
stream, so they can share it, and the caching allocator is not asked for
gigabytes every step.  A plan is an ordered ``name -> (shape, dtype)`` mapping;
its entries are laid out in order, each starting on a 256-byte boundary, so two
processes that build the same plan agree on every offset.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

_ALIGN = 256
_arenas: dict[tuple[torch.device, str], Tensor] = {}
# Bumped whenever an arena is allocated, regrown or dropped: a recorded CUDA graph holds arena
# addresses and is only valid while this number stands.
generation = 0

Plan = dict[str, tuple[tuple[int, ...], torch.dtype]]


def _round(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


def layout(plan: Plan) -> tuple[dict[str, tuple[int, int]], int]:
    """``name -> (byte offset, byte size)`` of every entry, and the total bytes."""
    offsets: dict[str, tuple[int, int]] = {}
    cursor = 0
    for name, (shape, dtype) in plan.items():
        nbytes = math.prod(shape) * dtype.itemsize
        offsets[name] = (cursor, nbytes)
        cursor += _round(nbytes)
    return offsets, cursor


def views(buffer: Tensor, plan: Plan, base: int = 0) -> dict[str, Tensor]:
    """Typed views of ``buffer`` (a byte tensor) for every entry of ``plan``, laid out from ``base``."""
    offsets, _ = layout(plan)
    out: dict[str, Tensor] = {}
    for name, (shape, dtype) in plan.items():
        start, nbytes = offsets[name]
        out[name] = buffer[base + start : base + start + nbytes].view(dtype).view(shape)
    return out


def arena(device: torch.device, nbytes: int, name: str = "run") -> Tensor:
    """The named byte arena of ``device``, at least ``nbytes`` long (contents unspecified)."""
    key = (device, name)
    buffer = _arenas.get(key)
    if buffer is None or buffer.numel() < nbytes:
        global generation
        generation += 1
        _arenas.pop(key, None)
        buffer = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _arenas[key] = buffer
    return buffer


def carve(device: torch.device, plan: Plan, name: str = "run") -> dict[str, Tensor]:
    """One tensor per plan entry, all views of the device's arena ``name``."""
    _, total = layout(plan)
    return views(arena(device, total, name), plan)


def release() -> None:
    """Drop every arena (tests, or before a memory-hungry phase)."""
    global generation
    generation += 1
    _arenas.clear()
