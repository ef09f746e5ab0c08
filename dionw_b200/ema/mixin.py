"""``IntegratedEMAOptimizer``: an optimizer mixin that steps, saves, loads and swaps an EMA.

Behaviour follows src/dionw/ema/mixin.py:77-308 and src/dionw/ema/_swap.py:31-101.
List it before the concrete optimizer and call ``_init_integrated_ema`` at the end
of ``__init__``::

    class AdamWWithEMA(IntegratedEMAOptimizer, torch.optim.AdamW): ...
"""

from __future__ import annotations

from collections.abc import Callable, Mapping
from typing import Any

import torch
from torch import Tensor
from torch.optim import Optimizer

from dionw_b200._keys import (
    EMA_INITIALIZED, EMA_KEY_PREFIX, EMA_PENDING, EMA_SCRATCH_KEYS, EMA_SHADOW, EMA_STEP_COUNT_KEY,
)
from dionw_b200.ema.config import EMAConfig, ProfileRegion
from dionw_b200.ema.tracker import FP32, OptimizerIntegratedEMA


class IntegratedEMAOptimizer(Optimizer):
    """Updates an ``OptimizerIntegratedEMA`` after each step of the concrete optimizer.

    Shadows and the schedule position travel in the optimizer's ``state_dict``;
    the CPU EMA's working buffers do not.  The concrete optimizer must create a
    parameter's state no later than its first step.
    """

    _ema_helper: OptimizerIntegratedEMA | None
    _stored_params: dict[int, Tensor]

    def _init_integrated_ema(self, ema: EMAConfig | None, profile_region: ProfileRegion) -> None:
        """Attach the EMA (``None`` disables it).

        Raises:
            ValueError: If the optimizer holds no trainable parameter.
        """
        if not self._iter_trainable_params():
            raise ValueError(f"{type(self).__name__} requires at least one trainable parameter")
        self._ema_helper = None if ema is None else OptimizerIntegratedEMA(self, ema, profile_region)
        self._stored_params = {}

    def _iter_trainable_params(self) -> list[torch.nn.Parameter]:
        return [p for group in self.param_groups for p in group["params"] if p.requires_grad]

    @property
    def ema(self) -> OptimizerIntegratedEMA | None:
        """The EMA, or None when disabled."""
        return self._ema_helper

    @property
    def ema_weights_swapped(self) -> bool:
        """Whether ``swap_ema_weights`` currently holds EMA weights in the parameters."""
        return bool(self._stored_params)

    # ---- stepping ----------------------------------------------------------
    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:
        """The concrete optimizer's step, then the due EMA update.

        Parameters without a gradient keep their value; their shadow still
        advances on the global cadence.

        Raises:
            RuntimeError: While EMA weights are swapped in.
        """
        if self._stored_params:
            raise RuntimeError(
                "step() while EMA weights are swapped in: call restore_non_ema_weights() first")
        helper = self._ema_helper
        due = False
        if helper is not None:
            helper.begin_step()
            due = helper.should_update_this_step()
        loss = super().step(closure)
        if helper is not None and due:
            for param in self._iter_trainable_params():
                helper.update_param(param)
            helper.finalize_updates()
        return loss

    # ---- device status -------------------------------------------------------
    def check_device(self) -> None:
        """Synchronise the parameters' devices and raise if a kernel of an earlier step gave up a wait.

        The tensor-core kernels bound every wait on a barrier; one that runs out stores a
        code in a device status word and returns instead of hanging.  ``step()`` never
        synchronises, so the word is read where the optimizer synchronises anyway:
        ``state_dict()`` and ``swap_ema_weights()`` call this first, and a training loop may
        call it as often as it likes.  Fail fast, never swallow
        (src/dionw/ema/_cpu_job.py:108-137 is the reference's form of the same rule).

        Raises:
            dionw_b200._native.DeviceWaitError: The weights and state written since the last
                check are not to be trusted.
        """
        from dionw_b200 import _native

        devices = {p.device for group in self.param_groups for p in group["params"] if p.is_cuda}
        for device in sorted(devices, key=lambda d: d.index or 0):
            with torch.cuda.device(device):
                _native.check_device()

    # ---- saving and loading ------------------------------------------------
    def state_dict(self) -> dict[str, Any]:
        """The optimizer state plus the shadows and ``_ema_step_count`` (pending work finished first).

        Raises:
            dionw_b200._native.DeviceWaitError: See ``check_device``.
        """
        self.check_device()
        helper = self._ema_helper
        if helper is None:
            return super().state_dict()
        helper.flush_pending_updates()
        saved = super().state_dict()
        saved["state"] = {
            index: {k: v for k, v in entry.items() if k not in EMA_SCRATCH_KEYS}
            for index, entry in saved["state"].items()
        }
        saved[EMA_STEP_COUNT_KEY] = helper.step_count
        return saved

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        """Restore the state, the shadows (on the configured EMA device) and the step count.

        Raises:
            ValueError: If the checkpoint carries EMA state but this optimizer has
                no EMA, or carries no valid EMA step count while this one has.
        """
        helper = self._ema_helper
        name = type(self).__name__
        if helper is None:
            carries = EMA_STEP_COUNT_KEY in state_dict or any(
                key.startswith(EMA_KEY_PREFIX) for entry in state_dict["state"].values() for key in entry)
            if carries:
                raise ValueError(
                    f"Checkpoint {name} state carries EMA shadows but the optimizer was built without EMA "
                    "(ema=None). Build it with the saved EMAConfig to continue the EMA, or load a fresh "
                    "optimizer state without the EMA.")
            super().load_state_dict(state_dict)
            return
        helper.flush_pending_updates()
        count = state_dict.get(EMA_STEP_COUNT_KEY)
        if type(count) is not int or count < 0:
            raise ValueError(
                f"{name} state has no valid EMA step count ({EMA_STEP_COUNT_KEY}={count!r}): "
                "it was not saved with an EMA")
        plain = {k: v for k, v in state_dict.items() if k != EMA_STEP_COUNT_KEY}
        plain["state"] = {
            index: {k: v for k, v in entry.items() if not k.startswith(EMA_KEY_PREFIX)}
            for index, entry in state_dict["state"].items()
        }
        super().load_state_dict(plain)
        # torch's loader would cast a shadow to its parameter's device: place them here instead.
        on_gpu = helper.uses_gpu_shadow
        pin = helper.config.pin_memory and not on_gpu
        for saved_group, group in zip(state_dict["param_groups"], self.param_groups, strict=True):
            for index, param in zip(saved_group["params"], group["params"], strict=True):
                source = state_dict["state"].get(index, {})
                if EMA_SHADOW not in source:
                    continue
                shadow = source[EMA_SHADOW]
                if not isinstance(shadow, Tensor):
                    raise TypeError(f"{name} EMA shadow must be a tensor")
                entry = self.state[param]
                shadow = self._loaded_shadow_share(param, shadow)
                entry[EMA_SHADOW] = torch.empty_like(
                    shadow, device=param.device if on_gpu else torch.device("cpu"), dtype=FP32,
                    pin_memory=pin).copy_(shadow)
                entry[EMA_INITIALIZED] = source[EMA_INITIALIZED]
                entry[EMA_PENDING] = False
        helper.step_count = count

    def _loaded_shadow_share(self, param: Tensor, shadow: Tensor) -> Tensor:
        """The part of a checkpoint's shadow this optimizer keeps (all of it, unless sharded)."""
        return shadow

    # ---- evaluation with EMA weights ----------------------------------------
    @torch.no_grad()
    def swap_ema_weights(self, model: torch.nn.Module | None = None) -> bool:
        """Put the shadows into the parameters (undo with ``restore_non_ema_weights``).

        ``model`` scopes the swap to that module's parameters.  Returns whether
        EMA weights were applied (False without EMA or before the first update).

        Raises:
            RuntimeError: If already swapped, or only some parameters have shadows.
            ValueError: If nothing can be swapped, or ``model`` shares no parameter
                with the optimizer or has trainable parameters outside it.
        """
        helper = self._ema_helper
        if helper is None:
            return False
        if self._stored_params:
            raise RuntimeError("EMA weights are already swapped in")
        self.check_device()
        helper.flush_pending_updates()
        context = type(self).__name__
        params = self._iter_trainable_params()
        if not params:
            raise ValueError("No parameters available to swap with EMA weights")
        if model is not None:
            managed = {id(p) for p in params}
            inside = [p for p in model.parameters() if id(p) in managed]
            outside = sum(1 for p in model.parameters() if id(p) not in managed and p.requires_grad)
            if outside:
                raise ValueError(
                    f"{context} EMA swap received a model with {outside} trainable parameters "
                    "outside the optimizer.")
            if not inside:
                raise ValueError(
                    f"{context} EMA swap received a model with no optimizer-managed parameters.")
            params = inside
        pairs: list[tuple[torch.nn.Parameter, Tensor]] = []
        for param in params:
            entry = self.state.get(param)
            shadow = entry.get(EMA_SHADOW) if isinstance(entry, Mapping) else None
            if shadow is None:
                continue
            if not isinstance(shadow, Tensor):
                raise TypeError(f"{context} EMA shadow must be a torch.Tensor")
            pairs.append((param, shadow))
        if not pairs:
            return False
        if len(pairs) != len(params):
            raise RuntimeError(
                f"{context} EMA swap found {len(pairs)} initialized shadows for {len(params)} parameters. "
                "Refusing to mix live and EMA weights.")
        for param, shadow in pairs:
            self._stored_params[id(param)] = self._swap_in(param, shadow)
        return True

    def _swap_in(self, param: Tensor, shadow: Tensor) -> Tensor:
        """Write ``shadow`` into ``param``; returns what ``_swap_out`` needs to undo it."""
        kept = param.data.clone()
        param.data.copy_(shadow.to(device=param.device, dtype=param.dtype))
        return kept

    def _swap_out(self, param: Tensor, kept: Tensor) -> None:
        param.data.copy_(kept)

    @torch.no_grad()
    def restore_non_ema_weights(self) -> bool:
        """Undo ``swap_ema_weights``.  False without EMA, True otherwise."""
        if self._ema_helper is None:
            return False
        for param in self._iter_trainable_params():
            kept = self._stored_params.get(id(param))
            if kept is not None:
                self._swap_out(param, kept)
        self._stored_params.clear()
        return True
