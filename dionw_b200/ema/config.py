"""EMA schedule and placement (src/dionw/ema/config.py:12-144)."""

from __future__ import annotations

import enum
from collections.abc import Callable
from contextlib import AbstractContextManager, nullcontext
from dataclasses import dataclass

# ``profile_region("name")`` returns a context manager entered around EMA work.
ProfileRegion = Callable[[str], AbstractContextManager[object]]


def no_profile(name: str) -> AbstractContextManager[object]:
    """The default ``ProfileRegion``: does nothing."""
    return nullcontext()


class EMADevice(enum.Enum):
    """Where the shadows live."""

    GPU = "gpu"
    CPU = "cpu"


class EMASchedule(enum.Enum):
    """How the per-step decay evolves."""

    CONSTANT = "constant"        # ``decay`` at every step
    LINEAR_RAMP = "linear_ramp"  # from ``decay`` to ``decay_final`` over ``decay_ramp_steps``
    POWER = "power"              # Karras et al. (EDM2): (1 - 1/n)^(gamma + 1), capped at ``decay``


@dataclass(frozen=True)
class EMAConfig:
    """EMA schedule and placement.

    ``decay`` is the per-step decay in [0, 1) (the cap of the power schedule);
    the shadows update every ``update_every_n_steps`` optimizer steps with the
    decay raised to that power; ``start_step`` > 0 copies the live weights into
    the shadows at that step and leaves the EMA untouched before it;
    ``decay_final`` with ``decay_ramp_steps`` selects the linear ramp,
    ``power_gamma`` (> 0) the power schedule; ``pin_memory`` pins the CPU
    shadows and staging buffers.

    Raises:
        ValueError: On out-of-range values, a half-specified ramp, or a ramp
            together with ``power_gamma``.
    """

    decay: float = 0.9999
    device: EMADevice = EMADevice.GPU
    pin_memory: bool = True
    update_every_n_steps: int = 1
    start_step: int = 0
    decay_final: float | None = None
    decay_ramp_steps: int | None = None
    power_gamma: float | None = None

    def __post_init__(self) -> None:
        if self.update_every_n_steps <= 0:
            raise ValueError("EMAConfig.update_every_n_steps must be positive")
        if self.start_step < 0:
            raise ValueError("EMAConfig.start_step must be non-negative")
        if not 0.0 <= self.decay < 1.0:
            raise ValueError("EMAConfig.decay must be in [0, 1)")
        ramp_given = (self.decay_final is not None, self.decay_ramp_steps is not None)
        if ramp_given[0] != ramp_given[1]:
            raise ValueError("EMAConfig.decay_final and decay_ramp_steps must be set together")
        if self.decay_final is not None and not 0.0 <= self.decay_final < 1.0:
            raise ValueError("EMAConfig.decay_final must be in [0, 1)")
        if self.decay_ramp_steps is not None and self.decay_ramp_steps <= 0:
            raise ValueError("EMAConfig.decay_ramp_steps must be positive")
        if self.power_gamma is not None:
            if self.decay_final is not None:
                raise ValueError("EMAConfig.power_gamma and the decay_final ramp are exclusive")
            if not self.power_gamma > 0.0:
                raise ValueError("EMAConfig.power_gamma must be positive")

    @property
    def schedule(self) -> EMASchedule:
        """The schedule the set fields select."""
        if self.power_gamma is not None:
            return EMASchedule.POWER
        return EMASchedule.CONSTANT if self.decay_final is None else EMASchedule.LINEAR_RAMP

    def decay_at_step(self, step_count: int) -> float:
        """Per-step decay at an EMA step count.

        Raises:
            ValueError: If ``step_count`` is negative.
        """
        if step_count < 0:
            raise ValueError("step_count must be non-negative")
        schedule = self.schedule
        if schedule is EMASchedule.CONSTANT:
            return self.decay
        if schedule is EMASchedule.LINEAR_RAMP:
            progress = min(1.0, step_count / self.decay_ramp_steps)
            return self.decay + (self.decay_final - self.decay) * progress
        if step_count == 0:
            return 0.0
        return min(self.decay, (1.0 - 1.0 / step_count) ** (self.power_gamma + 1.0))
