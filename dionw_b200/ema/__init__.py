"""EMA of the parameters, integrated in the optimizer, on the GPU or in pinned host memory.

Shadows live in ``optimizer.state[p]["ema_shadow"]`` (fp32) and are saved, loaded
and moved with the optimizer state; ``_ema_step_count`` is the schedule position.
The shadows update after each optimizer step, every ``update_every_n_steps``
steps, with ``decay ** n`` so the half-life in steps does not depend on ``n``.
Each update is ``shadow += (1 - decay) * (param - shadow)``: a constant parameter
keeps a bit-exact shadow.
"""

from dionw_b200._keys import EMA_STEP_COUNT_KEY
from dionw_b200.ema.config import EMAConfig, EMADevice, EMASchedule, ProfileRegion, no_profile
from dionw_b200.ema.mixin import IntegratedEMAOptimizer
from dionw_b200.ema.tracker import OptimizerIntegratedEMA

__all__ = [
    "EMA_STEP_COUNT_KEY", "EMAConfig", "EMADevice", "EMASchedule", "IntegratedEMAOptimizer",
    "OptimizerIntegratedEMA", "ProfileRegion", "no_profile",
]
