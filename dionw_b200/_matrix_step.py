"""One Dion step for a run of consecutive bucket parameters that have gradients.

Stages (the arithmetic is that of src/dionw/_matrix_step.py:104-311):

1. accumulate: ``M += G`` and, for row-selecting blocks, every row's l1 score
   and sum of squares -- one launch for the whole run;
2. select: the top-k rows of each block; those rows of ``M`` are decayed (error
   feedback) while being packed, normalised, into the fp16 operand;
   blocks that update every row decay all of ``M`` instead;
3. orthogonalize: the group's Newton-Schulz on the tensor cores;
4. finish: NorMuon row statistics (or none) reduced to one scale per row and
   one per block;
5. apply: decoupled weight decay on every row and the scaled update on the
   selected rows, in one pass over the weights.
"""

from __future__ import annotations

import math
import os
from collections.abc import Callable, Sequence
from contextlib import AbstractContextManager, contextmanager, nullcontext
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

from dionw_b200 import _native, _workspace
from dionw_b200._buckets import Bucket
from dionw_b200._keys import MOMENTUM_FORM_KEY, MOMENTUM_KEY, MUON_BETA2_KEY, ROW_NORMALIZATION_KEY, ParamState
from dionw_b200.matrix_update import MomentumForm, RowNormalization
from dionw_b200.newton_schulz import NativeOrthogonalizer, padded, run_iteration

__all__ = ["MAX_RUN_ELEMENTS", "apply_result", "apply_results", "open_run", "prepare_run", "run_core", "run_elements",
           "run_front", "step_run"]

ADAMW_UPDATE_RMS = 0.2        # update RMS of AdamW that matrix steps are matched to
NEWTON_SCHULZ_EPS = 1e-8      # added to the Frobenius norm; independent of AdamW's eps
NORMALIZATION_EPS = 1e-8      # NorMuon's epsilon
# Most update elements (blocks x selected rows x cols) one run orthogonalizes at
# once; bounds the transient memory of a step (src/dionw/_matrix_step.py:44-50).
MAX_RUN_ELEMENTS = 2**28


# Optional observer: ``STAGE_HOOK(name)`` must return a context manager; it is
# entered around each stage of a run ("accumulate", "select", "pack",
# "newton_schulz", "finish", "apply").  The benchmark uses it to bracket stages
# with CUDA events; None costs nothing.
STAGE_HOOK: Callable[[str], AbstractContextManager[object]] | None = None
# ``(blocks, rows, selected rows, cols)`` of the run whose stages are being entered, for an observer
# that wants its figures per shape.
CURRENT_RUN: tuple[int, int, int, int] | None = None


# DIONW_NVTX=1 wraps every stage (accumulate, select, pack, newton_schulz, finish, apply, adamw)
# in an NVTX range ``dionw/<stage>``, so a timeline profiler shows the kernel families of a step by
# name.  Read once at import; off by default (a push and a pop per stage cost host time).
_NVTX = os.environ.get("DIONW_NVTX", "0") not in ("", "0")


@contextmanager
def _nvtx_range(name: str, inner: AbstractContextManager[object]):
    torch.cuda.nvtx.range_push(f"dionw/{name}")
    try:
        with inner:
            yield
    finally:
        torch.cuda.nvtx.range_pop()


def _stage(name: str) -> AbstractContextManager[object]:
    inner = nullcontext() if STAGE_HOOK is None else STAGE_HOOK(name)
    return _nvtx_range(name, inner) if _NVTX else inner


def run_elements(bucket: Bucket, position: int) -> int:
    """Update elements of the parameter at ``position`` of ``bucket``."""
    blocks = bucket.slices[position]
    return (blocks.stop - blocks.start) * bucket.selected_rows * bucket.cols


def step_size(bucket: Bucket, lr: float) -> float:
    """``lr * 0.2 * sqrt(max(rows, cols)) * sqrt(min(rows, cols) / min(k, cols))``."""
    rows, cols, k = bucket.rows, bucket.cols, bucket.selected_rows
    return lr * ADAMW_UPDATE_RMS * math.sqrt(max(rows, cols)) * math.sqrt(min(rows, cols) / min(k, cols))


@dataclass
class RunResult:
    """What the first four stages of a run leave for the last one.

    ``orthogonal`` is the bf16 ``[count, k, ld]`` Newton-Schulz output, ``rowmap``
    the ``[count, rows]`` position of each weight row in it (-1: not selected;
    None: every row), ``denom`` the NorMuon divisor of each output row and
    ``scale`` the factor of each block (restored norm x signed step size).
    """

    params: list[Tensor]
    rows_per_tensor: list[int]
    count: int
    rows: int
    k: int
    cols: int
    orthogonal: Tensor
    rowmap: Tensor | None
    denom: Tensor
    scale: Tensor
    decay_device: Tensor | None = None   # 1 - lr * weight_decay in device memory (None: the host value is used)


def exchange_plan(count: int, rows: int, k: int, cols: int, selecting: bool) -> _workspace.Plan:
    """The buffers of a ``RunResult`` in the order they lie in the arena: everything another
    replica needs to apply the run (2-byte update rows, row map, row divisors, block scales)."""
    plan: _workspace.Plan = {"x": ((count, k, padded(cols)), torch.bfloat16)}
    if selecting:
        plan["rowmap"] = ((count, rows), torch.int32)
    plan["denom"] = ((count * k,), torch.float32)
    plan["scale"] = ((count,), torch.float32)
    return plan


def step_run(bucket: Bucket, positions: Sequence[int], group: dict[str, Any], state: ParamState) -> None:
    """Apply one Dion step to bucket parameters ``positions`` (consecutive, all with gradients).

    Raises:
        RuntimeError: If a parameter has no gradient.
    """
    del state  # momentum and variance are reached through the bucket's own buffers
    apply_result(prepare_run(bucket, positions, group), group)


@dataclass
class RunContext:
    """A run between its stages: the tensors it reads and the scratch it owns."""

    bucket: Bucket
    group: dict[str, Any]
    params: list[Tensor]
    grads: list[Tensor]
    rows_per_tensor: list[int]
    count: int
    momentum: Tensor
    variance: Tensor
    step: float
    buf: dict[str, Tensor]
    index: Tensor | None = None
    rowmap: Tensor | None = None
    source: Tensor | None = None

    @property
    def selecting(self) -> bool:
        return self.bucket.selected_rows < self.bucket.rows


def open_run(bucket: Bucket, positions: Sequence[int], group: dict[str, Any], arena: str = "run") -> RunContext:
    """Host-side set-up of a run: checks the gradients and carves the run's scratch from ``arena``.

    The scratch starts with the entries of ``exchange_plan`` in that order.

    Raises:
        RuntimeError: If a parameter has no gradient.
    """
    params = [bucket.params[i] for i in positions]
    grads: list[Tensor] = []
    for param in params:
        if param.grad is None:
            raise RuntimeError("a Dion run holds a parameter without a gradient")
        grads.append(param.grad)
    # The kernels walk row-major memory: a channels-last gradient is packed first.
    if len({g.dtype for g in grads}) > 1:
        grads = [g.float() for g in grads]
    grads = [g if g.is_contiguous() else g.contiguous() for g in grads]

    blocks = bucket.run_blocks(positions)
    count = blocks.stop - blocks.start
    rows, cols, k = bucket.rows, bucket.cols, bucket.selected_rows
    step = -step_size(bucket, float(group["lr"]))
    bucket.step_scale = step
    selecting = k < rows
    fn = bucket.orthogonalize
    native = isinstance(fn, NativeOrthogonalizer)
    dtype = fn.dtype if native else torch.float16

    plan = exchange_plan(count, rows, k, cols, selecting)
    plan["x"] = (plan["x"][0], dtype)  # the operand is iterated in place and ends as bf16
    plan.update({
        "scores": ((count, rows), torch.float32),
        "sumsq": ((count, rows), torch.float32),
        "index": ((count, k), torch.int32),
        "frob": ((count,), torch.float32),
    })
    # Row sums of squares of the orthogonalized rows: the last product's epilogue writes them as
    # partials per 128 columns when the block is iterated as it lies (wide or square); a tall block
    # is iterated transposed, and a foreign orthogonalizer knows nothing of this, so those take one
    # sum per row from a pass of their own.
    parts = _native.newton_schulz_rowsq_parts(cols) if native and k <= cols else 1
    plan["rowsq"] = ((count * k, parts), torch.float32)
    if not selecting:
        plan["u"] = ((count, rows, cols), torch.float32)
    if native:
        plan["ns"] = ((fn.workspace_bytes(count, k, cols),), torch.uint8)
        if k > cols:
            plan["xt"] = ((count, cols, padded(k)), dtype)
    momentum = bucket.momentum[blocks]
    return RunContext(
        bucket=bucket, group=group, params=params, grads=grads,
        rows_per_tensor=[(bucket.slices[i].stop - bucket.slices[i].start) * rows for i in positions],
        count=count, momentum=momentum, variance=bucket.variance[blocks].view(count, rows), step=step,
        buf=_workspace.carve(momentum.device, plan, arena))


def run_front(ctx: RunContext) -> None:
    """Stages 1-2 and the pack: the HBM-bound front of a run (reads G, updates M, writes the operand)."""
    global CURRENT_RUN
    bucket, group, buf = ctx.bucket, ctx.group, ctx.buf
    cols, k = bucket.cols, bucket.selected_rows
    CURRENT_RUN = (ctx.count, bucket.rows, k, cols)
    decay = float(group[MOMENTUM_KEY])
    if ctx.selecting:
        with _stage("accumulate"):
            _native.accumulate_row_l1_run(ctx.grads, ctx.rows_per_tensor, ctx.momentum, buf["scores"],
                                          buf["sumsq"], cols)
        with _stage("select"):
            _native.select_rows(buf["scores"], buf["sumsq"], k, buf["index"], buf["rowmap"], buf["frob"])
        ctx.index, ctx.rowmap, ctx.source = buf["index"], buf["rowmap"], ctx.momentum
    else:
        nesterov = MomentumForm(group[MOMENTUM_FORM_KEY]) is MomentumForm.NESTEROV
        with _stage("accumulate"):
            _native.accumulate_copy_decay_run(ctx.grads, ctx.rows_per_tensor, ctx.momentum, buf["u"],
                                              buf["sumsq"], cols, decay, nesterov)
            _native.block_norms(buf["sumsq"], buf["frob"])
        ctx.index, ctx.rowmap, ctx.source = None, None, buf["u"]
    fn = bucket.orthogonalize
    if isinstance(fn, NativeOrthogonalizer):
        with _stage("pack"):
            _native.pack_rows(ctx.source, ctx.index, buf["frob"], k, buf["x"], decay=decay,
                              decay_rows=ctx.selecting, eps=NEWTON_SCHULZ_EPS, norm_scale=fn.norm_scale)


def run_core(ctx: RunContext) -> RunResult:
    """Stages 3-4: the tensor-core part (Newton-Schulz) and the NorMuon scales."""
    global CURRENT_RUN
    bucket, group, buf = ctx.bucket, ctx.group, ctx.buf
    rows, cols, k = bucket.rows, bucket.cols, bucket.selected_rows
    CURRENT_RUN = (ctx.count, rows, k, cols)
    fn = bucket.orthogonalize
    normalize = RowNormalization(group[ROW_NORMALIZATION_KEY]) is RowNormalization.NORMUON
    parts = buf["rowsq"].shape[1]
    fused = normalize and parts > 1
    if isinstance(fn, NativeOrthogonalizer):
        with _stage("newton_schulz"):
            orthogonal = run_iteration(fn, buf["x"], k, cols, buf["ns"], buf.get("xt"),
                                       rowsq=buf["rowsq"] if fused else None)
    else:
        orthogonal = _foreign_orthogonalize(fn, ctx.source, ctx.index, float(group[MOMENTUM_KEY]), ctx.selecting,
                                            buf["x"])
    with _stage("finish"):
        if normalize and not fused:
            _native.row_sumsq_bf16(orthogonal, cols, buf["rowsq"])
        _native.normuon_rows(buf["rowsq"], ctx.variance, ctx.index, blocks=ctx.count, rows=rows, k=k, cols=cols,
                             weight=1.0 - float(group[MUON_BETA2_KEY]), eps=NORMALIZATION_EPS, step=ctx.step,
                             normalize=normalize, denom=buf["denom"], scale=buf["scale"],
                             parts=parts if fused else 1, step_device=bucket.step_device)
    return RunResult(params=ctx.params, rows_per_tensor=ctx.rows_per_tensor, count=ctx.count, rows=rows, k=k,
                     cols=cols, orthogonal=orthogonal, rowmap=ctx.rowmap, denom=buf["denom"], scale=buf["scale"],
                     decay_device=bucket.decay_device)


def prepare_run(bucket: Bucket, positions: Sequence[int], group: dict[str, Any],
                arena: str = "run") -> RunResult:
    """Stages 1-4 of a run, one after the other on the current stream."""
    ctx = open_run(bucket, positions, group, arena)
    run_front(ctx)
    return run_core(ctx)


def apply_result(result: RunResult, group: dict[str, Any]) -> None:
    """Stage 5: decoupled weight decay on every row, the scaled update on the selected rows."""
    apply_results([result], group)


def apply_results(results: Sequence[RunResult], group: dict[str, Any], warps: int = 0,
                  decay_job: Tensor | None = None) -> None:
    """Stage 5 for several results of one bucket shape (the contributions of every rank to a round
    of the sharded step) in ONE launch per 64 weights.  ``warps`` sets the CTA size (0: the default);
    ``decay_job``: the job the round's products carried (its cursor says which rows are decayed)."""
    global CURRENT_RUN
    first = results[0]
    CURRENT_RUN = (sum(r.count for r in results), first.rows, first.k, first.cols)
    lr, weight_decay = float(group["lr"]), float(group["weight_decay"])
    params: list[Tensor] = []
    targets: list[Tensor] = []
    rows_per_tensor: list[int] = []
    # device addresses of each tensor's first block within its result's buffers
    o: list[int] = []
    rowmap: list[int] = []
    denom: list[int] = []
    scale: list[int] = []
    for result in results:
        o_base, o_block = result.orthogonal.data_ptr(), result.k * result.orthogonal.stride(-2) * 2
        map_base = None if result.rowmap is None else result.rowmap.data_ptr()
        denom_base, scale_base = result.denom.data_ptr(), result.scale.data_ptr()
        block = 0
        for param, tensor_rows in zip(result.params, result.rows_per_tensor):
            params.append(param)
            # A channels-last weight is updated through a packed copy and written back.
            targets.append(param if param.is_contiguous() else param.detach().contiguous())
            rows_per_tensor.append(tensor_rows)
            o.append(o_base + block * o_block)
            if map_base is not None:
                rowmap.append(map_base + block * result.rows * 4)
            denom.append(denom_base + block * result.k * 4)
            scale.append(scale_base + block * 4)
            block += tensor_rows // result.rows
    with _stage("apply"):
        _native.apply_round(targets, rows_per_tensor, o, rowmap or None, denom, scale,
                            ldo=first.orthogonal.stride(-2), rows=first.rows, k=first.k, cols=first.cols,
                            decay_factor=1.0 - lr * weight_decay, has_decay=weight_decay > 0.0,
                            decay_device=first.decay_device, cta_warps=warps, decay_job=decay_job)
    for param, target in zip(params, targets):
        if target is not param:
            param.copy_(target)


def _foreign_orthogonalize(fn: Any, source: Tensor, index: Tensor | None, decay: float, selecting: bool,
                           out: Tensor) -> Tensor:
    """Orthogonalize with a caller-supplied function (``[N, k, cols]`` fp32 -> bf16).

    The built-in kinds never come here.  A test or a user that swaps
    ``_buckets.newton_schulz_fn`` for its own function gets the rows gathered
    in fp32 with torch indexing, its function called, and the bf16 result
    copied into the padded operand buffer the later kernels read.
    """
    if selecting:
        wide = index.long().unsqueeze(-1).expand(-1, -1, source.shape[-1])
        matrices = torch.gather(source, 1, wide)
        source.scatter_(1, wide, matrices * decay)
    else:
        matrices = source
    result = fn(matrices, NEWTON_SCHULZ_EPS)
    target = out.view(torch.bfloat16) if out.dtype is not torch.bfloat16 else out
    target[..., : matrices.shape[-1]].copy_(result)
    return target
