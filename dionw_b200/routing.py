"""Routes: which update each parameter receives (src/dionw/routing.py:22-83).

``param_groups`` routes every parameter by its default rule; a module overrides
the rule for its own parameters with a ``dion_routes`` method, and the caller
with the ``routes`` argument.
"""

from __future__ import annotations

import enum
from collections.abc import Iterable
from dataclasses import dataclass
from typing import Protocol, runtime_checkable

from torch import Tensor


class RouteKind(enum.Enum):
    """The update family of a parameter."""

    ADAMW = "adamw"    # element-wise AdamW (vectors, embeddings, declared layers)
    MATRIX = "matrix"  # orthogonalized, row-selected NorMuon update


@dataclass(frozen=True)
class Route:
    """One parameter's route.

    ``num_heads`` (MATRIX only) splits the rows into that many equal blocks
    orthogonalized on their own; ``fraction`` (MATRIX only) overrides the row
    fraction ``param_groups`` would choose.

    Raises:
        ValueError: For matrix options on an ADAMW route or values out of range.
    """

    kind: RouteKind
    num_heads: int | None = None
    fraction: float | None = None

    def __post_init__(self) -> None:
        if self.kind is RouteKind.ADAMW:
            if self.num_heads is not None or self.fraction is not None:
                raise ValueError("Route num_heads and fraction apply only to MATRIX routes")
            return
        if self.kind is not RouteKind.MATRIX:
            raise RuntimeError(f"Unhandled RouteKind: {self.kind}")
        if self.num_heads is not None and self.num_heads <= 0:
            raise ValueError(f"Route num_heads must be positive, got {self.num_heads}")
        if self.fraction is not None and not 0.0 < self.fraction <= 1.0:
            raise ValueError(f"Route fraction must be in (0, 1], got {self.fraction}")


@runtime_checkable
class RouteProvider(Protocol):
    """Any module with a ``dion_routes`` method declares routes for its parameters."""

    def dion_routes(self) -> Iterable[tuple[Tensor, Route]]:
        """(parameter, route) pairs that override the default rule."""
        ...
