"""The AdamW route: one fused multi-tensor launch per group (src/dionw/_adamw.py:18-61)."""

from __future__ import annotations

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


def adamw_step(group: dict[str, Any], state: ParamState) -> None:
    """One decoupled-decay AdamW step for the group's parameters that have gradients."""
    params = [p for p in group["params"] if p.grad is not None]
    if not params:
        return
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
    _native.adamw_multi(
        p_list, g_list, m_list, v_list, s_list, lr=float(group["lr"]), beta1=float(beta1), beta2=float(beta2),
        weight_decay=float(group["weight_decay"]), eps=float(group["eps"]),
    )
    for param, packed in fixups:
        param.copy_(packed)
