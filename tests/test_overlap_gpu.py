"""The two-stream step gives the same bits as the one-stream step."""

from __future__ import annotations

import pytest
import torch
from torch import nn

import dionw_b200 as dionw

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _build(overlap: bool):
    torch.manual_seed(0)
    net = nn.Module()
    net.a = nn.ParameterList([nn.Parameter(torch.randn(256, 512) * 0.02) for _ in range(5)])
    net.b = nn.ParameterList([nn.Parameter(torch.randn(512, 128) * 0.02) for _ in range(3)])
    net.c = nn.Parameter(torch.randn(64, 64) * 0.02)
    net.table = nn.Embedding(300, 64)
    net.bias = nn.Parameter(torch.zeros(64))
    net = net.to(DEV)
    groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=128)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05, ema=dionw.EMAConfig(decay=0.9))
    opt.overlap_streams = overlap
    return net, opt


def test_overlapped_step_is_bit_identical(monkeypatch) -> None:
    import dionw_b200.optimizer as optimizer_module

    monkeypatch.setattr(optimizer_module, "MAX_RUN_ELEMENTS", 2 * 64 * 512)  # several runs per bucket
    (net_a, opt_a), (net_b, opt_b) = _build(True), _build(False)
    gen = torch.Generator(device=DEV).manual_seed(1)
    for step in range(4):
        for i, (pa, pb) in enumerate(zip(net_a.parameters(), net_b.parameters())):
            g = None if (step == 2 and i == 1) else torch.randn(pa.shape, device=DEV, generator=gen) * 1e-3
            pa.grad = g
            pb.grad = None if g is None else g.clone()
        opt_a.step()
        opt_b.step()
        torch.cuda.synchronize()
        for pa, pb in zip(net_a.parameters(), net_b.parameters()):
            assert torch.equal(pa, pb), step
    sa, sb = opt_a.state_dict(), opt_b.state_dict()
    for index, entry in sa["state"].items():
        for key, value in entry.items():
            if isinstance(value, torch.Tensor):
                assert torch.equal(value, sb["state"][index][key]), (index, key)
