"""The orthogonalization of matrix updates (src/dionw/newton_schulz.py:33-68).

Every kind runs five quintic steps on a batch of matrices and returns bfloat16.
All of them run on this package's tcgen05 kernels: ``GRAM`` in float16 with the
Gram schedule of src/dionw/_gram.py:41-89, the Polar Express and Keller kinds in
bfloat16 with the schedule of src/dionw/_polar_express.py:74-104 (the ``_TRITON``
and plain names select the same device code here; the enum keeps both values
because they are part of the checkpoint's structural keys).
"""

from __future__ import annotations

import enum
from collections.abc import Callable
from dataclasses import dataclass

import torch
from torch import Tensor

from dionw_b200 import _native

# ([N, rows, cols] batch, epsilon added to the Frobenius norm) -> bf16 polar factors
Orthogonalize = Callable[[Tensor, float], Tensor]


class NewtonSchulz(enum.Enum):
    """Which iteration orthogonalizes matrix updates."""

    POLAR_EXPRESS = "polar_express"
    POLAR_EXPRESS_TRITON = "polar_express_triton"
    GRAM = "gram"
    KELLER = "keller"
    KELLER_TRITON = "keller_triton"


def padded(n: int) -> int:
    """Leading dimension used for 2-byte operands: a multiple of 8 elements (16 bytes)."""
    return (n + 7) // 8 * 8


@dataclass(frozen=True)
class NativeOrthogonalizer:
    """A built-in iteration.  ``Dion`` recognises it and feeds it from its fused
    pack kernel; called directly it orthogonalizes any ``[N, rows, cols]`` batch."""

    kind: NewtonSchulz
    code: int             # DIONW_NS_* of the C ABI
    dtype: torch.dtype    # element type of the iteration
    norm_scale: float     # factor on the Frobenius norm before normalising

    def __call__(self, matrix: Tensor, epsilon: float) -> Tensor:
        if matrix.ndim != 3:
            raise ValueError(f"expected a [N, rows, cols] batch, got shape {tuple(matrix.shape)}")
        if not matrix.is_cuda:
            raise ValueError("dionw_b200 orthogonalizes on CUDA devices only")
        blocks, rows, cols = matrix.shape
        src = matrix.float().contiguous()
        if self.dtype is torch.bfloat16:
            frob = src.bfloat16().norm(dim=(-2, -1)).float()
        else:
            frob = torch.linalg.vector_norm(src, dim=(-2, -1))
        x = torch.empty(blocks, rows, padded(cols), dtype=self.dtype, device=src.device)
        _native.pack_rows(src, None, frob, rows, x, decay=1.0, decay_rows=False, eps=epsilon,
                          norm_scale=self.norm_scale)
        scratch = torch.empty(self.workspace_bytes(blocks, rows, cols), dtype=torch.uint8, device=src.device)
        xt = None
        if rows > cols:
            xt = torch.empty(blocks, cols, padded(rows), dtype=self.dtype, device=src.device)
        out = run_iteration(self, x, rows, cols, scratch, xt)
        return out[..., :cols]

    def workspace_bytes(self, blocks: int, rows: int, cols: int) -> int:
        m, n = min(rows, cols), max(rows, cols)
        return _native.newton_schulz_workspace_bytes(blocks, m, n, self.code)


def run_iteration(fn: NativeOrthogonalizer, x: Tensor, rows: int, cols: int, scratch: Tensor,
                  xt: Tensor | None, rowsq: Tensor | None = None) -> Tensor:
    """Iterate on ``x`` ``[N, rows, ld]`` (normalised, in ``fn.dtype``); returns bf16 ``[N, rows, ld]``.

    Wide and square blocks are iterated in place.  Tall ones go through ``xt``, a
    ``[N, cols, padded(rows)]`` buffer of the same dtype.  ``scratch`` holds
    ``fn.workspace_bytes(...)`` bytes.  ``rowsq`` (wide and square blocks only):
    fp32 ``[N * rows, newton_schulz_rowsq_parts(cols)]``, filled with partial row
    sums of the squared result by the last product's epilogue.
    """
    m, n = min(rows, cols), max(rows, cols)
    out = x if x.dtype is torch.bfloat16 else x.view(torch.bfloat16)
    if rows <= cols:
        _native.newton_schulz(x, out, m, n, fn.code, scratch, rowsq)
        return out
    if rowsq is not None:
        raise ValueError("row sums come with wide and square blocks only: a tall block is iterated transposed")
    if xt is None:
        raise ValueError("tall blocks need the transposed buffer")
    _native.transpose_2byte(x[..., :cols], xt)
    xt_out = xt if xt.dtype is torch.bfloat16 else xt.view(torch.bfloat16)
    _native.newton_schulz(xt, xt_out, m, n, fn.code, scratch)
    _native.transpose_2byte(xt_out[..., :rows], out)
    return out


_NATIVE = {
    NewtonSchulz.GRAM: NativeOrthogonalizer(NewtonSchulz.GRAM, _native.NS_GRAM, torch.float16, 1.0),
    NewtonSchulz.POLAR_EXPRESS: NativeOrthogonalizer(
        NewtonSchulz.POLAR_EXPRESS, _native.NS_POLAR_EXPRESS, torch.bfloat16, 1.02),
    NewtonSchulz.POLAR_EXPRESS_TRITON: NativeOrthogonalizer(
        NewtonSchulz.POLAR_EXPRESS_TRITON, _native.NS_POLAR_EXPRESS, torch.bfloat16, 1.02),
    NewtonSchulz.KELLER: NativeOrthogonalizer(NewtonSchulz.KELLER, _native.NS_KELLER, torch.bfloat16, 1.0),
    NewtonSchulz.KELLER_TRITON: NativeOrthogonalizer(
        NewtonSchulz.KELLER_TRITON, _native.NS_KELLER, torch.bfloat16, 1.0),
}


def newton_schulz_fn(kind: NewtonSchulz) -> Orthogonalize:
    """The orthogonalization for ``kind``.

    Raises:
        RuntimeError: For an unhandled kind.
    """
    try:
        return _NATIVE[kind]
    except KeyError:
        raise RuntimeError(f"Unhandled NewtonSchulz: {kind}") from None


def gram_polar_express(matrix: Tensor, epsilon: float) -> Tensor:
    """Gram Newton-Schulz of a batch, bf16 (src/dionw/_gram.py:72-89)."""
    return _NATIVE[NewtonSchulz.GRAM](matrix, epsilon)
