"""What ``param_groups`` decided for each parameter (src/dionw/report.py:14-82)."""

from __future__ import annotations

import enum
import math
from collections import OrderedDict
from dataclasses import dataclass

from dionw_b200.routing import RouteKind


class RouteReason(enum.Enum):
    """The rule that routed a parameter."""

    DECLARED = "declared"
    EMBEDDING = "embedding"
    GROUPED_CONVOLUTION = "grouped convolution"
    LEARNED_TOKENS = "learned tokens"
    EMBEDDING_NAME = "embedding-like name"
    VECTOR = "vector"
    NARROW = "narrow"
    MATRIX = "matrix"


@dataclass(frozen=True)
class RoutedParameter:
    """Name, shape, route, row fraction (1.0 for AdamW), head split, decay flag and reason."""

    name: str
    shape: tuple[int, ...]
    kind: RouteKind
    fraction: float
    num_heads: int | None
    decayed: bool
    reason: RouteReason


@dataclass(frozen=True)
class RoutingReport:
    """All routed parameters in group order."""

    parameters: tuple[RoutedParameter, ...]

    def lines(self) -> list[str]:
        """A header, one line per group, then every >= 2-D tensor that went to AdamW."""
        totals: OrderedDict[tuple, list[int]] = OrderedDict()
        for entry in self.parameters:
            key = (entry.kind, entry.fraction, entry.num_heads, entry.decayed)
            totals.setdefault(key, []).append(math.prod(entry.shape))
        text = ["dionw parameter routing:"]
        for (kind, fraction, heads, decayed), sizes in totals.items():
            text.append(
                f"  {kind.value} fraction={fraction} heads={heads} decay={'yes' if decayed else 'no'} "
                f"tensors={len(sizes)} params={sum(sizes) / 1e6:.2f}M"
            )
        for entry in self.parameters:
            if entry.kind is RouteKind.ADAMW and len(entry.shape) >= 2:
                text.append(f"    adamw ({entry.reason.value}): {entry.name} {entry.shape}")
        return text
