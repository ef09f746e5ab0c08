"""Size-independent properties at the full sizes of the Llama-3-8B- and 70B-shaped configurations.

The CPU oracle cannot run a bucket of 64 gate/up weights (3.76 G elements), so the largest
bucket of the 8B shapes, a 5.6 G-element bucket of the 70B shapes and the two AdamW tables are
held to properties that need no oracle: the decoupled decay is exact on every row the step did not select, the momentum of a
selected row is exactly its decayed sum, the selected rows are the top-k by l1 norm, and every
parameter of the bucket comes out bit-identical to the same parameter stepped alone, wherever it
lies in the slab (offsets beyond 2^32 elements, first and last position of every run).
"""

from __future__ import annotations

import math

import pytest
import torch
from torch import nn

import dionw_b200 as dionw
from dionw_b200 import _native, _workspace

pytestmark = pytest.mark.gpu
DEV = "cuda"
LR, WEIGHT_DECAY, MOMENTUM = 3e-4, 0.05, 0.95


def _need_free_gb(gb: float) -> None:
    torch.cuda.empty_cache()
    _workspace.release()
    free, _ = torch.cuda.mem_get_info()
    if free < gb * 2**30:
        pytest.skip(f"needs {gb:.0f} GB of free device memory, {free / 2**30:.0f} GB are free")


def _seeded(shape: tuple[int, ...], seed: int, std: float) -> torch.Tensor:
    gen = torch.Generator(device=DEV).manual_seed(seed)
    return torch.empty(shape, device=DEV).normal_(0.0, std, generator=gen)


@pytest.mark.parametrize(("rows", "cols", "count", "alone_at", "free_gb"), [
    # the 64 gate/up weights of the Llama-3-8B shapes: runs of 18, 18, 18 and 10 parameters
    (14336, 4096, 64, (0, 17, 18, 35, 36, 53, 54, 63), 70),
    # 24 gate/up weights of the Llama-3-70B shapes (5.6 G elements): runs of 4
    (28672, 8192, 24, (0, 3, 4, 19, 20, 23), 100),
])
@torch.no_grad()
def test_gate_up_bucket_holds_its_properties_at_full_size(rows, cols, count, alone_at, free_gb) -> None:
    k = math.ceil(0.25 * rows)
    _need_free_gb(free_gb)
    net = nn.Module()
    net.w = nn.ParameterList([nn.Parameter(_seeded((rows, cols), 1000 + i, 0.02)) for i in range(count)])
    groups, _ = dionw.param_groups(net)
    opt = dionw.Dion(groups, lr=LR, weight_decay=WEIGHT_DECAY, momentum=MOMENTUM)
    for i, p in enumerate(net.w):
        p.grad = _seeded((rows, cols), 2000 + i, 1e-3)
    opt.step()
    torch.cuda.synchronize()
    assert _native.device_status() == 0
    assert opt.state[net.w[0]]["momentum"].untyped_storage().nbytes() == count * rows * cols * 4

    step = LR * 0.2 * math.sqrt(max(rows, cols)) * math.sqrt(min(rows, cols) / min(k, cols))
    for i, p in enumerate(net.w):
        grad, state = p.grad, opt.state[p]
        momentum, variance = state["momentum"], state["variance"]
        picked = (momentum != grad).any(dim=1)
        assert int(picked.sum()) == k, i
        # error feedback: a selected row keeps momentum x (M + G), every other row M + G, exactly (M was 0)
        assert torch.equal(momentum[picked], grad[picked] * MOMENTUM), i
        # the selected rows are the top k by l1 norm (fp64 scores; rows within rounding of the cut may swap)
        scores = grad.abs().sum(dim=1, dtype=torch.float64)
        want = torch.zeros(rows, dtype=torch.bool, device=DEV)
        want[torch.topk(scores, k).indices] = True
        swapped = picked ^ want
        if bool(swapped.any()):
            cut = float(scores[want].min())
            assert int(swapped.sum()) <= 4 and float((scores[swapped] - cut).abs().max()) <= 1e-6 * cut, i
        # decoupled decay on every row, exact where no update was added
        decayed = _seeded((rows, cols), 1000 + i, 0.02) * (1 - LR * WEIGHT_DECAY)
        assert torch.equal(p[~picked], decayed[~picked]), i
        assert torch.equal(variance.view(-1) != 0, picked), i
        # NorMuon restores the block's norm: |U|_F = |O|_F x step, and O is close to k orthonormal rows
        update = (p[picked] - decayed[picked]).double().norm()
        assert 0.7 <= float(update) / (math.sqrt(k) * step) <= 1.1, (i, float(update))
        del decayed

    # a second step (momentum now carries), then parameters at the ends of every run against themselves alone
    opt.step()
    torch.cuda.synchronize()
    for i in alone_at:
        alone = nn.Module()
        alone.w = nn.ParameterList([nn.Parameter(_seeded((rows, cols), 1000 + i, 0.02))])
        single = dionw.Dion(dionw.param_groups(alone).groups, lr=LR, weight_decay=WEIGHT_DECAY, momentum=MOMENTUM)
        alone.w[0].grad = net.w[i].grad
        single.step()
        single.step()
        torch.cuda.synchronize()
        assert torch.equal(alone.w[0], net.w[i]), i
        for key in ("momentum", "variance"):
            assert torch.equal(single.state[alone.w[0]][key], opt.state[net.w[i]][key]), (i, key)
    assert _native.device_status() == 0


@torch.no_grad()
def test_adamw_tables_of_the_8b_shapes_equal_torch_fused_adamw_at_full_size() -> None:
    """Embedding and output table, 128256 x 4096 each, in one multi-tensor launch: bit-equal to
    ``torch.optim.AdamW(fused=True)``, which src/dionw/_adamw.py:45 calls into."""
    _need_free_gb(45)
    shape = (128256, 4096)
    net = nn.Module()
    net.embed = nn.Embedding(*shape, device=DEV)
    net.head = nn.Embedding(*shape, device=DEV)
    with torch.no_grad():
        for i, p in enumerate(net.parameters()):
            p.copy_(_seeded(shape, 10 + i, 0.02))
    theirs = [nn.Parameter(p.detach().clone()) for p in net.parameters()]
    stock = torch.optim.AdamW(theirs, lr=LR, betas=(0.9, 0.95), weight_decay=WEIGHT_DECAY, eps=1e-8, fused=True)
    opt = dionw.Dion(dionw.param_groups(net).groups, lr=LR, weight_decay=WEIGHT_DECAY)
    for step in range(2):
        for i, (p, q) in enumerate(zip(net.parameters(), theirs)):
            p.grad = _seeded(shape, 100 + 10 * step + i, 1e-3)
            q.grad = p.grad
        opt.step()
        stock.step()
    torch.cuda.synchronize()
    for p, q in zip(net.parameters(), theirs):
        assert torch.equal(p, q), "parameter"
        assert torch.equal(opt.state[p]["exp_avg"], stock.state[q]["exp_avg"])
        assert torch.equal(opt.state[p]["exp_avg_sq"], stock.state[q]["exp_avg_sq"])
        assert float(opt.state[p]["adamw_step"]) == 2.0
