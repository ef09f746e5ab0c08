"""Options of the matrix update (src/dionw/matrix_update.py:26-73)."""

from __future__ import annotations

import enum
from dataclasses import dataclass

from dionw_b200.newton_schulz import NewtonSchulz


class RowNormalization(enum.Enum):
    """What happens to the orthogonalized rows before they are applied."""

    NORMUON = "normuon"  # divide rows by the root of an EMA of their mean square, keep the block norm
    NONE = "none"        # plain Muon: use the orthogonalized rows as they are


class MomentumForm(enum.Enum):
    """Which momentum is orthogonalized; both keep ``B = momentum * B + G``."""

    HEAVY_BALL = "heavy_ball"  # orthogonalize B
    NESTEROV = "nesterov"      # orthogonalize G + momentum * B (needs every row each step)


@dataclass(frozen=True)
class MatrixUpdate:
    """Orthogonalization, row normalization and momentum form of matrix steps."""

    newton_schulz: NewtonSchulz
    row_normalization: RowNormalization
    momentum_form: MomentumForm


DION3_UPDATE = MatrixUpdate(NewtonSchulz.GRAM, RowNormalization.NORMUON, MomentumForm.HEAVY_BALL)
MUON_UPDATE = MatrixUpdate(NewtonSchulz.KELLER_TRITON, RowNormalization.NONE, MomentumForm.NESTEROV)
