"""The AdamW route: one fused multi-tensor launch per group (src/dionw/_adamw.py:18-61)."""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch
from torch import Tensor

from dionw_b200 import _native
from dionw_b200._keys import ADAMW_STEP_STATE, EXP_AVG_SQ_STATE, EXP_AVG_STATE, ParamState


def init_adamw_state(param: Tensor, state: dict[str, Any]) -> None:
    """Fresh moments and an fp32 step counter on the parameter's device."""
    state[EXP_AVG_STATE] = torch.zeros_like(param)
    state[EXP_AVG_SQ_STATE] = torch.zeros_like(param)
    state[ADAMW_STEP_STATE] = torch.zeros((), dtype=torch.float32, device=param.device)


def adamw_step(group: dict[str, Any], state: ParamState,
               hyper: Callable[[torch.device], Tensor | None] | None = None) -> None:
    """One decoupled-decay AdamW step for the group's parameters that have gradients.

    ``hyper(device)`` gives the two-element fp32 device tensor ``{lr, weight_decay}`` the kernel reads
    instead of the host values (so a scheduled learning rate changes no launch), or None."""
    params = [p for p in group["params"] if p.grad is not None]
    if not params:
        return
    devices = {p.device for p in params}
    if len(devices) > 1:   # one launch per device, each with that device current
        for device in sorted(devices, key=lambda d: d.index or 0):
            adamw_step({**group, "params": [p for p in params if p.device == device]}, state, hyper)
        return
    device = params[0].device
    fixups: list[tuple[Tensor, Tensor]] = []
    p_list, g_list, m_list, v_list, s_list = [], [], [], [], []
    for param in params:
        entry = state[param]
        if EXP_AVG_STATE not in entry:
            init_adamw_state(param, entry)
        grad = param.grad
        if grad is None:
            raise RuntimeError("an AdamW update holds a parameter without a gradient")
        if grad.dtype is not torch.float32 or not grad.is_contiguous():
            grad = grad.float().contiguous()
        target = param
        if not param.is_contiguous():
            # The kernel walks flat memory: update a packed copy and write it back.
            target = param.detach().contiguous()
            fixups.append((param, target))
        p_list.append(target)
        g_list.append(grad)
        m_list.append(entry[EXP_AVG_STATE])
        v_list.append(entry[EXP_AVG_SQ_STATE])
        s_list.append(entry[ADAMW_STEP_STATE])
    beta1, beta2 = group["betas"]
    with torch.cuda.device(device):
        _native.adamw_multi(
            p_list, g_list, m_list, v_list, s_list, lr=float(group["lr"]), beta1=float(beta1), beta2=float(beta2),
            weight_decay=float(group["weight_decay"]), eps=float(group["eps"]),
            hyper_device=None if hyper is None else hyper(device),
        )
    for param, packed in fixups:
        param.copy_(packed)
