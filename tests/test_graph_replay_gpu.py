"""A step replayed from a CUDA graph gives the same bits as the step run as launches."""

from __future__ import annotations

import pytest
import torch
from torch import nn

import dionw_b200 as dionw

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _build(replay: bool, ema: bool = True):
    torch.manual_seed(0)
    net = nn.Module()
    net.a = nn.ParameterList([nn.Parameter(torch.randn(256, 512) * 0.02) for _ in range(5)])
    net.b = nn.ParameterList([nn.Parameter(torch.randn(512, 128) * 0.02) for _ in range(3)])
    net.c = nn.Parameter(torch.randn(64, 64) * 0.02)
    net.table = nn.Embedding(300, 64)
    net.bias = nn.Parameter(torch.zeros(64))
    net = net.to(DEV)
    groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=128)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05, ema=dionw.EMAConfig(decay=0.9) if ema else None)
    opt.graph_replay = replay
    for p in net.parameters():
        p.grad = torch.zeros_like(p)
    return net, opt


def _same_state(opt_a, opt_b) -> None:
    sa, sb = opt_a.state_dict(), opt_b.state_dict()
    for index, entry in sa["state"].items():
        for key, value in entry.items():
            if isinstance(value, torch.Tensor):
                assert torch.equal(value, sb["state"][index][key]), (index, key)


def _fill_grads(net_a, net_b, gen) -> None:
    """New gradient values at the same addresses, as ``zero_grad(set_to_none=False)`` training does."""
    for pa, pb in zip(net_a.parameters(), net_b.parameters()):
        g = torch.randn(pa.shape, device=DEV, generator=gen) * 1e-3
        pa.grad.copy_(g)
        pb.grad.copy_(g)


def test_replayed_step_is_bit_identical(monkeypatch) -> None:
    import dionw_b200.optimizer as optimizer_module

    monkeypatch.setattr(optimizer_module, "MAX_RUN_ELEMENTS", 2 * 64 * 512)  # several runs per bucket
    (net_a, opt_a), (net_b, opt_b) = _build(True), _build(False)
    gen = torch.Generator(device=DEV).manual_seed(1)
    for step in range(6):
        _fill_grads(net_a, net_b, gen)
        opt_a.step()
        opt_b.step()
        torch.cuda.synchronize()
        for pa, pb in zip(net_a.parameters(), net_b.parameters()):
            assert torch.equal(pa, pb), step
        # step 0 runs as launches, step 1 records, the rest replay that one recording
        assert (opt_a._graph is not None) == (step >= 1), step
    assert opt_a._graph_recordings == 1
    assert opt_b._graph is None
    _same_state(opt_a, opt_b)


def test_a_scheduled_learning_rate_keeps_the_recording(monkeypatch) -> None:
    """The step scalars that follow the learning rate (-step_size, 1 - lr * wd, AdamW's lr and weight
    decay) are read from a device table, as the reference keeps -step_size in a 0-d device tensor
    (src/dionw/_buckets.py:57-58): twenty steps of a cosine schedule (lr and weight decay both
    moving) replay ONE recording and equal, bit for bit, the same steps run as launches -- with the
    scalars read from the device table and with them passed as kernel arguments."""
    import math

    (net_a, opt_a), (net_b, opt_b), (net_c, opt_c) = (_build(True, ema=False), _build(False, ema=False),
                                                      _build(False, ema=False))
    monkeypatch.setattr(opt_c, "_refresh_scalars", lambda: None)   # host scalars: the kernels' other source
    gen = torch.Generator(device=DEV).manual_seed(2)
    for step in range(20):
        lr = 3e-4 * 0.5 * (1.0 + math.cos(math.pi * step / 20))
        for opt in (opt_a, opt_b, opt_c):
            for group in opt.param_groups:
                group["lr"] = lr
                if group["weight_decay"] > 0.0:
                    group["weight_decay"] = 0.05 * (1.0 - 0.02 * step)
        for pa, pb, pc in zip(net_a.parameters(), net_b.parameters(), net_c.parameters()):
            g = torch.randn(pa.shape, device=DEV, generator=gen) * 1e-3
            pa.grad.copy_(g)
            pb.grad.copy_(g)
            pc.grad.copy_(g)
        opt_a.step()
        opt_b.step()
        opt_c.step()
        torch.cuda.synchronize()
        for pa, pb, pc in zip(net_a.parameters(), net_b.parameters(), net_c.parameters()):
            assert torch.equal(pa, pb), step
            assert torch.equal(pb, pc), step
    assert opt_a._graph_recordings == 1 and opt_a.graph_replays == 19
    assert all(b.step_device is None for b in opt_c._buckets)
    _same_state(opt_a, opt_b)
    _same_state(opt_b, opt_c)


def test_a_weight_decay_switched_off_is_recorded_anew() -> None:
    """Whether a group decays at all selects code in the weight update, so that IS part of a
    recording's key: switching it off costs one step as launches and one new recording."""
    (net_a, opt_a), (net_b, opt_b) = _build(True, ema=False), _build(False, ema=False)
    gen = torch.Generator(device=DEV).manual_seed(2)
    for step in range(7):
        if step == 3:
            for opt in (opt_a, opt_b):
                for group in opt.param_groups:
                    group["weight_decay"] = 0.0
        _fill_grads(net_a, net_b, gen)
        opt_a.step()
        opt_b.step()
        torch.cuda.synchronize()
        for pa, pb in zip(net_a.parameters(), net_b.parameters()):
            assert torch.equal(pa, pb), step
    assert opt_a._graph_recordings == 2
    _same_state(opt_a, opt_b)


def test_gradients_that_move_fall_back_to_launches() -> None:
    """Reallocated gradients change the recording's key: those steps run as launches, and after
    ``GRAPH_RECORDINGS_MAX`` recordings the optimizer stops recording.  Results never differ."""
    (net_a, opt_a), (net_b, opt_b) = _build(True, ema=False), _build(False, ema=False)
    opt_a.GRAPH_RECORDINGS_MAX = 1
    gen = torch.Generator(device=DEV).manual_seed(3)
    keep = []
    for step in range(5):
        for pa, pb in zip(net_a.parameters(), net_b.parameters()):
            g = torch.randn(pa.shape, device=DEV, generator=gen) * 1e-3
            if step == 3:
                keep.append(pa.grad)  # hold the old storage so that the new one lies elsewhere
                pa.grad = g.clone()
            else:
                pa.grad.copy_(g)
            pb.grad.copy_(g)
        opt_a.step()
        opt_b.step()
        torch.cuda.synchronize()
        for pa, pb in zip(net_a.parameters(), net_b.parameters()):
            assert torch.equal(pa, pb), step
    assert opt_a._graph_recordings == 1 and opt_a._graph is None
    _same_state(opt_a, opt_b)


def test_a_loaded_checkpoint_drops_the_recording() -> None:
    """``load_state_dict`` replaces the state tensors a recording points at: the recording goes,
    the next steps run as launches, are recorded anew and keep matching the unrecorded optimizer."""
    import io

    (net_a, opt_a), (net_b, opt_b) = _build(True, ema=False), _build(False, ema=False)
    gen = torch.Generator(device=DEV).manual_seed(4)
    for _ in range(3):
        _fill_grads(net_a, net_b, gen)
        opt_a.step()
        opt_b.step()
    assert opt_a._graph is not None
    buffer = io.BytesIO()
    torch.save(opt_b.state_dict(), buffer)
    for opt in (opt_a, opt_b):
        buffer.seek(0)
        opt.load_state_dict(torch.load(buffer, weights_only=False))
    assert opt_a._graph is None
    for step in range(4):
        _fill_grads(net_a, net_b, gen)
        opt_a.step()
        opt_b.step()
        torch.cuda.synchronize()
        for pa, pb in zip(net_a.parameters(), net_b.parameters()):
            assert torch.equal(pa, pb), step
    assert opt_a._graph is not None and opt_a._graph_recordings == 2
    _same_state(opt_a, opt_b)
