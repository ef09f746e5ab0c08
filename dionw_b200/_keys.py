"""String keys of Dion's param groups and per-parameter state.

The values are part of the checkpoint format and equal the reference's
(src/dionw/_keys.py:36-68, src/dionw/ema/_keys.py:18-33): a ``state_dict``
written by either implementation loads in the other.
"""

from __future__ import annotations

from collections.abc import MutableMapping
from typing import Any

from torch import Tensor

ParamState = MutableMapping[Tensor, dict[str, Any]]

# ---- group entries ----
ROUTE_KEY = "dion_route"                # RouteKind value of the group
NEWTON_SCHULZ_KEY = "newton_schulz"     # NewtonSchulz value
FRACTION_KEY = "fraction"               # share of rows updated per step
NUM_HEADS_KEY = "num_heads"             # row split of each parameter into blocks, or None
MOMENTUM_KEY = "momentum"               # matrix momentum / error-feedback decay
MUON_BETA2_KEY = "muon_beta2"           # NorMuon EMA decay of squared rows
ROW_NORMALIZATION_KEY = "row_normalization"
MOMENTUM_FORM_KEY = "momentum_form"
# A checkpoint is refused when one of these differs from the optimizer's groups.
STRUCTURAL_KEYS = (
    ROUTE_KEY, FRACTION_KEY, NUM_HEADS_KEY, NEWTON_SCHULZ_KEY, ROW_NORMALIZATION_KEY, MOMENTUM_FORM_KEY,
)

# ---- per-parameter state entries ----
MOMENTUM_STATE = "momentum"
VARIANCE_STATE = "variance"
EXP_AVG_STATE = "exp_avg"
EXP_AVG_SQ_STATE = "exp_avg_sq"
# torch's load_state_dict moves an entry called "step" to the CPU; this name keeps it on the device.
ADAMW_STEP_STATE = "adamw_step"

# ---- EMA entries ----
EMA_STEP_COUNT_KEY = "_ema_step_count"  # top-level state_dict entry
EMA_KEY_PREFIX = "ema_"
EMA_SHADOW = "ema_shadow"
EMA_INITIALIZED = "ema_initialized"
EMA_PENDING = "ema_pending"
EMA_TMP_CPU = "ema_tmp_cpu"
EMA_EVENT = "ema_event"
EMA_SCRATCH_KEYS = (EMA_PENDING, EMA_TMP_CPU, EMA_EVENT)  # rebuilt on load, never saved
