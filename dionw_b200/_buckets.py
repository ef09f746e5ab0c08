"""Bucketed matrix state (layout of src/dionw/_buckets.py:43-191).

Same-shape blocks of one matrix group share one fp32 momentum buffer
``[N, rows, cols]`` and one fp32 variance buffer ``[N, rows, 1]``;
``optimizer.state[p]["momentum"]`` / ``["variance"]`` are views into them, so a
run of consecutive parameters is one contiguous slab for the kernels and
``torch.save`` keeps one storage per bucket.
"""

from __future__ import annotations

import math
from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor, nn

from dionw_b200._keys import (
    FRACTION_KEY, MOMENTUM_STATE, NEWTON_SCHULZ_KEY, NUM_HEADS_KEY, ROUTE_KEY, VARIANCE_STATE, ParamState,
)
from dionw_b200.newton_schulz import NewtonSchulz, Orthogonalize, newton_schulz_fn
from dionw_b200.param_groups import block_shape
from dionw_b200.routing import RouteKind

__all__ = ["Bucket", "block_shape", "build_buckets", "newton_schulz_fn"]


@dataclass
class Bucket:
    """Blocks of one shape in one matrix group.

    ``slices[i]`` is the block range of ``params[i]``; ``selected_rows`` is
    ``min(rows, ceil(fraction * rows))``; ``step_scale`` is the signed step size
    of the last run as a host float.  ``step_device`` and ``decay_device`` are
    one-element fp32 views of the optimizer's device table of step scalars
    (``-step_size`` of this bucket, ``1 - lr * weight_decay`` of its group), the
    counterpart of the 0-d ``step_scale`` tensor at src/dionw/_buckets.py:57-58:
    kernels read them from there, so a changed learning rate changes no launch.
    None (a bucket built by hand) makes the kernels take the host values.
    """

    group_index: int
    orthogonalize: Orthogonalize
    params: list[nn.Parameter]
    slices: list[slice]
    rows: int
    cols: int
    selected_rows: int
    momentum: Tensor
    variance: Tensor
    step_scale: float = 0.0
    step_device: Tensor | None = None
    decay_device: Tensor | None = None

    def run_blocks(self, positions: Sequence[int]) -> slice:
        """Block range covered by consecutive parameters ``positions``."""
        return slice(self.slices[positions[0]].start, self.slices[positions[-1]].stop)


def build_buckets(param_groups: list[dict[str, Any]], state: ParamState) -> list[Bucket]:
    """Pack every matrix group's state into per-shape buckets, in group order.

    Momentum and variance already present in ``state`` (a loaded checkpoint, or
    the buckets of an earlier layout) are copied into the new buffers first.
    """
    buckets: list[Bucket] = []
    for group_index, group in enumerate(param_groups):
        if RouteKind(group[ROUTE_KEY]) is not RouteKind.MATRIX:
            continue
        orthogonalize = newton_schulz_fn(NewtonSchulz(group[NEWTON_SCHULZ_KEY]))
        heads = group[NUM_HEADS_KEY]
        by_shape: dict[tuple[int, int, torch.device], list[nn.Parameter]] = {}
        for param in group["params"]:
            _, rows, cols = block_shape(param, heads)
            by_shape.setdefault((rows, cols, param.device), []).append(param)
        for (rows, cols, device), params in by_shape.items():
            slices, cursor = [], 0
            for param in params:
                count = block_shape(param, heads)[0]
                slices.append(slice(cursor, cursor + count))
                cursor += count
            bucket = Bucket(
                group_index=group_index, orthogonalize=orthogonalize, params=params, slices=slices,
                rows=rows, cols=cols,
                selected_rows=min(rows, math.ceil(float(group[FRACTION_KEY]) * rows)),
                momentum=torch.zeros(cursor, rows, cols, device=device),
                variance=torch.zeros(cursor, rows, 1, device=device),
            )
            for param, blocks in zip(params, slices):
                entry = state[param]
                momentum = bucket.momentum[blocks].view(param.shape)
                variance = bucket.variance[blocks].view(param.shape[0], 1)
                if MOMENTUM_STATE in entry:
                    momentum.copy_(entry[MOMENTUM_STATE])
                    variance.copy_(entry[VARIANCE_STATE])
                entry[MOMENTUM_STATE] = momentum
                entry[VARIANCE_STATE] = variance
            buckets.append(bucket)
    return buckets
