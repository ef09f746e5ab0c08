"""CPU oracle for the dionw optimizer step.  TEST INFRASTRUCTURE ONLY.

A restatement, in plain torch-on-CPU arithmetic, of what the reference's
``optimizer.step()`` computes.  Only the test-suite, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import this
module; nothing under ``dionw_b200/`` does, and the product path raises when
its CUDA library is missing instead of coming here.

Parity pin: the functions below are checked against outputs of the reference
itself (imported from its source tree on CPU with its Triton launches swapped
for the reference's own torch forms) by ``tests/test_oracle_golden.py`` using
the fixtures ``tests/golden/make_golden.py`` wrote.

Each function cites the reference file:line it follows (paths are relative to
the reference project's root).

Two orders the reference leaves to its compiler are fixed here so that the CUDA
kernels can be compared bit for bit:

* row scores (``sum |M|`` per row): 1024 strided lanes accumulate sequentially
  (element ``j`` goes to lane ``j % 1024``, as in the reference's row kernel),
  then the lanes are folded by halving: ``lane[i] += lane[i + w]`` for
  ``w = 512, 256, ..., 1``;
* the selected row set is reported in ascending row order; among equal scores
  the lower row index wins.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Sequence

import torch
from torch import Tensor

LANES = 1024

# src/dionw/_gram.py:25-38 — Polar Express table divided by the safety factor
# 1.05, 1.05**3, 1.05**5.
_SAFETY = 1.05
_TABLE = (
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
)
GRAM_COEFFS = tuple((a / _SAFETY, b / _SAFETY**3, c / _SAFETY**5) for a, b, c in _TABLE)
RESTART_AT = 2  # src/dionw/_gram.py:38
NS_EPS = 1e-8  # src/dionw/_matrix_step.py:43
ROW_EPS = 1e-8  # src/dionw/_row_normalization.py:15
UPDATE_RMS = 0.2  # src/dionw/_matrix_step.py:41

# src/dionw/_polar_express.py:28-36 and src/dionw/_keller.py:20-22
POLAR_EXPRESS_COEFFS = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)
KELLER_COEFFS = ((3.4445, -4.7750, 2.0315),) * 5


# ----------------------------------------------------------------------------
# momentum passes
# ----------------------------------------------------------------------------
def row_scores(m: Tensor) -> Tensor:
    """l1 norm of each row of ``m`` ``[R, cols]`` in the fixed lane order.

    src/dionw/_momentum_kernels.py:40-55: lane ``j`` of 1024 adds elements
    ``j, j+1024, ...`` in turn, then the lanes are summed.
    """
    rows, cols = m.shape
    pad = (-cols) % LANES
    a = torch.nn.functional.pad(m.abs().float(), (0, pad)).view(rows, -1, LANES)
    lanes = torch.zeros(rows, LANES, dtype=torch.float32)
    for chunk in range(a.shape[1]):
        lanes = lanes + a[:, chunk]
    width = LANES
    while width > 1:
        width //= 2
        lanes = lanes[:, :width] + lanes[:, width : 2 * width]
    return lanes[:, 0]


def row_sumsq(m: Tensor) -> Tensor:
    """Sum of squares of each row in the same lane order as ``row_scores``."""
    rows, cols = m.shape
    pad = (-cols) % LANES
    sq = (m.float() * m.float())
    a = torch.nn.functional.pad(sq, (0, pad)).view(rows, -1, LANES)
    lanes = torch.zeros(rows, LANES, dtype=torch.float32)
    for chunk in range(a.shape[1]):
        lanes = lanes + a[:, chunk]
    width = LANES
    while width > 1:
        width //= 2
        lanes = lanes[:, :width] + lanes[:, width : 2 * width]
    return lanes[:, 0]


def accumulate_row_l1(grad: Tensor, momentum: Tensor, cols: int) -> Tensor:
    """``M += G`` in place; returns the row scores.

    src/dionw/_momentum_kernels.py:89-103 (kernel :40-55).
    """
    momentum.add_(grad.reshape(momentum.shape).float())
    return row_scores(momentum.view(-1, cols))


def accumulate_copy_decay(
    grad: Tensor, momentum: Tensor, decay: float, nesterov: bool
) -> Tensor:
    """``m = M + G``; ``M = decay * m``; returns ``m`` (or ``G + decay*m``).

    src/dionw/_momentum_kernels.py:58-77, :106-133.
    """
    g = grad.reshape(momentum.shape).float()
    m = momentum + g
    decayed = m * torch.tensor(decay, dtype=torch.float32)
    momentum.copy_(decayed)
    return g + decayed if nesterov else m


def select_rows(scores: Tensor, k: int) -> Tensor:
    """Top-``k`` rows of each block, ``scores`` ``[B, rows]`` -> int64 ``[B, k]``.

    src/dionw/_matrix_step.py:172-174 takes ``topk(sorted=False)``: the set is
    what matters.  Here the set is listed in ascending row order and equal
    scores go to the lower row.
    """
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices
    return torch.sort(order[:, :k], dim=-1).values


# ----------------------------------------------------------------------------
# Newton-Schulz
# ----------------------------------------------------------------------------
def _sym1(a: Tensor) -> Tensor:
    """``A A^T`` in A's dtype (src/dionw/_symmetric_kernels.py:252-277)."""
    return torch.bmm(a, a.mT)


def _sym2(a: Tensor, alpha: float, beta: float) -> Tensor:
    """``alpha A A^T + beta A`` (src/dionw/_symmetric_kernels.py:280-312)."""
    return torch.baddbmm(a, a, a.mT, beta=beta, alpha=alpha)


def _gram_wide(x: Tensor, eager_diagonal: bool = False) -> Tensor:
    """Gram iteration on wide fp16 ``[N, m, n]`` (src/dionw/_gram.py:50-69).

    ``Q = Z + a I`` (src/dionw/_gram.py:60-61): the reference's GPU step is compiled, and the fused
    expression adds the fp32 coefficient to fp32(Z) and rounds once (the default here).  Its eager
    run on the CPU evaluates ``a * eye`` in fp16 first, i.e. adds fp16(a): ``eager_diagonal=True``
    reproduces that bit for bit (the CPU-written fixtures pin it).
    """
    g = _sym1(x)
    eye = torch.eye(x.size(-2), dtype=x.dtype).expand_as(g)
    q = eye
    last = len(GRAM_COEFFS) - 1
    for i, (a, b, c) in enumerate(GRAM_COEFFS):
        if i == RESTART_AT:
            x = torch.bmm(q, x)
            g = _sym1(x)
        z = _sym2(g, alpha=c, beta=b)
        if i in (0, RESTART_AT):
            if eager_diagonal:
                q = z + a * eye
            else:
                q = (z.float() + torch.tensor(a, dtype=torch.float32) * eye.float()).to(z.dtype)
        else:
            q = torch.baddbmm(q, q, z, beta=a)
        if i < last and i + 1 != RESTART_AT:
            rz = torch.baddbmm(g, g, z, beta=a)
            g = torch.baddbmm(rz, z, rz, beta=a)
    return torch.bmm(q, x)


def _gram_square(x: Tensor) -> Tensor:
    """Standard iteration for square blocks (src/dionw/_gram.py:41-47)."""
    for a, b, c in GRAM_COEFFS:
        g = _sym1(x)
        p = _sym2(g, alpha=c, beta=b)
        x = torch.baddbmm(x, p, x, beta=a)
    return x


def gram_newton_schulz(matrix: Tensor, eps: float = NS_EPS, eager_diagonal: bool = False) -> Tensor:
    """Polar factor of each matrix of ``[N, rows, cols]``; bf16 result.

    src/dionw/_gram.py:72-89: transpose tall inputs, normalise by the Frobenius
    norm (+eps) in fp32, iterate in fp16, return bf16 in the input orientation.
    ``eager_diagonal``: see ``_gram_wide``.
    """
    tall = matrix.size(-2) > matrix.size(-1)
    x = (matrix.mT if tall else matrix).float()
    x = (x / (torch.linalg.vector_norm(x, dim=(-2, -1), keepdim=True) + eps)).half()
    x = x.contiguous()
    x = _gram_wide(x, eager_diagonal) if x.size(-1) > x.size(-2) else _gram_square(x)
    return (x.mT if tall else x).bfloat16()


def quintic_bf16(
    matrix: Tensor, eps: float, coeffs: Sequence[tuple[float, float, float]], safety: float
) -> Tensor:
    """bf16 quintic iteration (src/dionw/_polar_express.py:74-104)."""
    tall = matrix.size(-2) > matrix.size(-1)
    x = matrix.to(torch.bfloat16)
    if tall:
        x = x.mT
    x = x / (x.norm(dim=(-2, -1), keepdim=True) * safety + eps)
    x = x.contiguous()
    for a, b, c in coeffs:
        g = _sym1(x)
        p = _sym2(g, alpha=c, beta=b)
        x = torch.baddbmm(x, p, x, beta=a)
    return x.mT if tall else x


def polynomial_fp64(
    x: Tensor, coeffs: Sequence[tuple[float, float, float]] = GRAM_COEFFS,
    safety: float = 1.0, eps: float = 1e-7,
) -> Tensor:
    """The same polynomials in fp64: what an iteration computes without rounding.

    bench/precision.py:103-117.
    """
    x = x.double()
    x = x / (x.norm(dim=(-2, -1), keepdim=True) * safety + eps)
    for a, b, c in coeffs:
        g = x @ x.mT
        x = a * x + (b * g + c * g @ g) @ x
    return x


def exact_polar(x: Tensor) -> Tensor:
    """``U V^T`` of the thin SVD (tests/test_optimizer.py:74-87)."""
    u, _, vh = torch.linalg.svd(x.double(), full_matrices=False)
    return (u @ vh).float()


# ----------------------------------------------------------------------------
# NorMuon, step size, apply
# ----------------------------------------------------------------------------
def step_size(rows: int, cols: int, k: int, lr: float) -> float:
    """src/dionw/_matrix_step.py:147-159."""
    return lr * UPDATE_RMS * math.sqrt(max(rows, cols)) * math.sqrt(min(rows, cols) / min(k, cols))


def normalize_rows(o: Tensor, variance: Tensor, beta2: float, step: Tensor) -> tuple[Tensor, Tensor]:
    """NorMuon on ``[B, k, cols]`` (src/dionw/_row_normalization.py:41-60)."""
    u = o.float()
    n0 = torch.linalg.vector_norm(u, dim=(-2, -1), keepdim=True)
    variance = torch.lerp(variance, u.square().mean(-1, keepdim=True), 1 - beta2)
    normalized = u / (variance.sqrt() + ROW_EPS)
    n1 = torch.linalg.vector_norm(normalized, dim=(-2, -1), keepdim=True)
    restore = n0 / n1.clamp_min(ROW_EPS)
    return normalized * (restore * step), variance


# ----------------------------------------------------------------------------
# AdamW and EMA
# ----------------------------------------------------------------------------
def adamw_(
    p: Tensor, g: Tensor, m: Tensor, v: Tensor, step: Tensor, *,
    lr: float, beta1: float, beta2: float, weight_decay: float, eps: float,
) -> None:
    """Decoupled-decay AdamW with bias correction, fp32, in place.

    src/dionw/_adamw.py:25-61 hands this to torch's fused multi-tensor AdamW
    (``amsgrad=False, maximize=False``) after adding one to the fp32 step
    counter; the arithmetic below is that algorithm in float32.
    """
    f32 = torch.float32
    step.add_(1.0)
    t = float(step)
    b1, b2 = torch.tensor(beta1, dtype=f32), torch.tensor(beta2, dtype=f32)
    lr32, wd32, eps32 = (torch.tensor(x, dtype=f32) for x in (lr, weight_decay, eps))
    bc1 = 1 - torch.pow(b1, torch.tensor(t, dtype=f32))
    bc2_sqrt = torch.sqrt(1 - torch.pow(b2, torch.tensor(t, dtype=f32)))
    g = g.float()
    if weight_decay != 0:
        p.sub_((lr32 * wd32) * p)
    m.copy_(b1 * m + (g - b1 * g))
    gg = g * g
    v.copy_(b2 * v + (gg - b2 * gg))
    denom = v.sqrt() / bc2_sqrt + eps32
    p.sub_((lr32 / bc1) * m / denom)


def ema_lerp_(shadow: Tensor, source: Tensor, decay: float) -> None:
    """``shadow += (1-decay) * (source - shadow)`` (src/dionw/ema/_update.py:17-29)."""
    shadow.lerp_(source.float(), 1.0 - decay)


# ----------------------------------------------------------------------------
# one whole step over a parameter set
# ----------------------------------------------------------------------------
@dataclass
class MatrixBucket:
    """State of same-shape blocks (src/dionw/_buckets.py:43-74, :154-178)."""

    params: list[Tensor]
    rows: int
    cols: int
    k: int
    momentum: Tensor  # [N, rows, cols]
    variance: Tensor  # [N, rows, 1]
    last_index: Tensor | None = None


@dataclass
class AdamState:
    exp_avg: Tensor
    exp_avg_sq: Tensor
    step: Tensor


@dataclass
class OracleDion:
    """The reference step over plain tensors (no autograd, no torch.optim).

    ``matrix`` lists 2-D weights with their row fraction, ``adamw`` lists
    (tensor, weight_decay) pairs.  Mirrors src/dionw/optimizer.py:324-343 and
    src/dionw/_matrix_step.py:104-311 for contiguous fp32 inputs, one bucket
    per ``(rows, cols)`` and one run per bucket.
    """

    matrix: list[tuple[Tensor, float]]
    adamw: list[tuple[Tensor, float]]
    lr: float
    momentum: float = 0.95
    muon_beta2: float = 0.95
    betas: tuple[float, float] = (0.9, 0.95)
    weight_decay: float = 0.0
    eps: float = 1e-8
    orthogonalize: object = None
    buckets: list[MatrixBucket] = field(default_factory=list)
    adam_state: list[AdamState] = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.orthogonalize is None:
            self.orthogonalize = gram_newton_schulz
        by_shape: dict[tuple[int, int, float], list[Tensor]] = {}
        for w, fraction in self.matrix:
            by_shape.setdefault((w.shape[0], w[0].numel(), fraction), []).append(w)
        for (rows, cols, fraction), ws in by_shape.items():
            k = min(rows, math.ceil(fraction * rows))
            self.buckets.append(
                MatrixBucket(ws, rows, cols, k,
                             torch.zeros(len(ws), rows, cols), torch.zeros(len(ws), rows, 1))
            )
        for p, _ in self.adamw:
            self.adam_state.append(
                AdamState(torch.zeros_like(p), torch.zeros_like(p), torch.zeros((), dtype=torch.float32))
            )

    def step(self, matrix_grads: Sequence[Tensor], adamw_grads: Sequence[Tensor]) -> None:
        grads = {id(w): g for (w, _), g in zip(self.matrix, matrix_grads)}
        for b in self.buckets:
            self._step_bucket(b, [grads[id(w)] for w in b.params])
        for (p, wd), st, g in zip(self.adamw, self.adam_state, adamw_grads):
            adamw_(p, g, st.exp_avg, st.exp_avg_sq, st.step, lr=self.lr,
                   beta1=self.betas[0], beta2=self.betas[1],
                   weight_decay=self.weight_decay if wd is None else wd, eps=self.eps)

    def _step_bucket(self, b: MatrixBucket, grads: list[Tensor]) -> None:
        step = torch.tensor(-step_size(b.rows, b.cols, b.k, self.lr), dtype=torch.float32)
        n = len(b.params)
        if b.k < b.rows:
            # src/dionw/_matrix_step.py:162-185
            scores = torch.stack(
                [accumulate_row_l1(g, b.momentum[i], b.cols) for i, g in enumerate(grads)]
            )
            index = select_rows(scores, b.k).unsqueeze(-1)
            b.last_index = index
            wide = index.expand(-1, -1, b.cols)
            selected = torch.gather(b.momentum, 1, wide)
            b.momentum.scatter_(1, wide, selected * float(self.momentum))
            v_sel = torch.gather(b.variance, 1, index)
            o = self.orthogonalize(selected, NS_EPS)
            update, v_new = normalize_rows(o, v_sel, self.muon_beta2, step)
            b.variance.scatter_(1, index, v_new)
        else:
            # src/dionw/_matrix_step.py:202-214
            current = torch.stack(
                [accumulate_copy_decay(g, b.momentum[i], float(self.momentum), False)
                 for i, g in enumerate(grads)]
            )
            o = self.orthogonalize(current, NS_EPS)
            update, v_new = normalize_rows(o, b.variance, self.muon_beta2, step)
            b.variance.copy_(v_new)
            index = None
        # src/dionw/_matrix_step.py:274-304
        if self.weight_decay > 0.0:
            for w in b.params:
                w.mul_(1.0 - self.lr * self.weight_decay)
        for i in range(n):
            w = b.params[i].view(b.rows, b.cols)
            if index is None:
                w.add_(update[i])
            else:
                w.scatter_add_(0, index[i].expand(-1, b.cols), update[i])
