"""dionw_b200: the dionw optimizer step on B200 (sm_100a).

The same Python surface as the reference's ``dionw`` package
(src/dionw/__init__.py:16-65)::

    import dionw_b200 as dionw

    groups, report = dionw.param_groups(model)
    optimizer = dionw.Dion(groups, lr=3e-4, weight_decay=0.05)

Importing the package does not need a GPU; building an optimizer and stepping
it does, and needs ``dionw_b200/lib/libdionw_b200.so``
(``python -m dionw_b200.build_ext``).
"""

from dionw_b200._keys import (
    FRACTION_KEY, MOMENTUM_FORM_KEY, NEWTON_SCHULZ_KEY, NUM_HEADS_KEY, ROUTE_KEY, ROW_NORMALIZATION_KEY,
)
from dionw_b200.ema import EMAConfig, EMADevice, EMASchedule, IntegratedEMAOptimizer
from dionw_b200.matrix_update import DION3_UPDATE, MUON_UPDATE, MatrixUpdate, MomentumForm, RowNormalization
from dionw_b200.newton_schulz import NewtonSchulz
from dionw_b200.optimizer import Dion
from dionw_b200.param_groups import ParamGroups, param_groups
from dionw_b200.report import RoutedParameter, RouteReason, RoutingReport
from dionw_b200.routing import Route, RouteKind, RouteProvider

__version__ = "0.1.0"

__all__ = [
    "DION3_UPDATE", "FRACTION_KEY", "MOMENTUM_FORM_KEY", "MUON_UPDATE", "NEWTON_SCHULZ_KEY", "NUM_HEADS_KEY",
    "ROUTE_KEY", "ROW_NORMALIZATION_KEY", "Dion", "EMAConfig", "EMADevice", "EMASchedule",
    "IntegratedEMAOptimizer", "MatrixUpdate", "MomentumForm", "NewtonSchulz", "ParamGroups", "Route",
    "RouteKind", "RouteProvider", "RouteReason", "RoutedParameter", "RoutingReport", "RowNormalization",
    "__version__", "param_groups",
]
