"""``param_groups(model)``: route every trainable parameter and build Dion's groups.

Behaviour follows src/dionw/param_groups.py:89-270 and the default rule of
src/dionw/_default_rule.py:52-127.  First matching rule wins:

1. weights of ``nn.Embedding`` / ``nn.EmbeddingBag`` -> AdamW;
2. weights of grouped (incl. depthwise) convolutions -> AdamW;
3. parameters whose own name ends in ``token``/``tokens`` -> AdamW;
4. own names containing ``pos_embed``, ``position_embedding`` or
   ``relative_position_bias`` -> AdamW;
5. fewer than two dimensions -> AdamW;
6. smaller side (after flattening to ``(shape[0], rest)``) below ``min_matrix_dim`` -> AdamW;
7. everything else -> MATRIX.

A declared route (a module's ``dion_routes`` or the ``routes`` argument) beats
the rule.  Matrix blocks whose smaller side reaches ``selection_min_dim`` update
``fraction`` of their rows per step, smaller blocks every row.  Groups of
decayed parameters carry no ``weight_decay`` key (they take the optimizer's),
exempt groups carry ``weight_decay = 0.0``; vectors, learned tokens and
embedding-like names are exempt unless ``no_weight_decay`` names the exempt set.
"""

from __future__ import annotations

import logging
import math
from collections import OrderedDict
from collections.abc import Collection, Iterable, Mapping
from typing import Any, NamedTuple

from torch import Tensor, nn

from dionw_b200._keys import FRACTION_KEY, NUM_HEADS_KEY, ROUTE_KEY
from dionw_b200.report import RoutedParameter, RouteReason, RoutingReport
from dionw_b200.routing import Route, RouteKind, RouteProvider

_LOGGER = logging.getLogger("dionw")

LEARNED_TOKEN_NAME_SUFFIXES = ("token", "tokens")
EMBEDDING_NAME_SUBSTRINGS = ("pos_embed", "position_embedding", "relative_position_bias")
_CONVOLUTIONS = (
    nn.Conv1d, nn.Conv2d, nn.Conv3d, nn.ConvTranspose1d, nn.ConvTranspose2d, nn.ConvTranspose3d,
)


class ParamGroups(NamedTuple):
    """``groups, report = param_groups(model)``."""

    groups: list[dict[str, Any]]
    report: RoutingReport


class _Home(NamedTuple):
    """Where a parameter is registered: qualified name, owning module, name on it."""

    name: str
    module: nn.Module
    local: str


def block_shape(param: Tensor, num_heads: int | None) -> tuple[int, int, int]:
    """``(blocks, rows, cols)`` of a matrix parameter (src/dionw/_buckets.py:77-90).

    Trailing dimensions flatten into the columns; a head split divides the rows.

    Raises:
        ValueError: If ``num_heads`` does not divide the rows.
    """
    rows = int(param.shape[0])
    cols = math.prod(int(d) for d in param.shape[1:])
    if num_heads is None:
        return 1, rows, cols
    if rows % num_heads:
        raise ValueError(f"num_heads={num_heads} does not divide {rows} rows")
    return num_heads, rows // num_heads, cols


def _homes(model: nn.Module) -> dict[int, _Home]:
    homes: dict[int, _Home] = {}
    for prefix, module in model.named_modules():
        for local, param in module.named_parameters(recurse=False):
            if id(param) not in homes:  # the first registration names a shared parameter
                homes[id(param)] = _Home(f"{prefix}.{local}" if prefix else local, module, local)
    return homes


def _looks_like_tokens(local: str) -> bool:
    return local.endswith(LEARNED_TOKEN_NAME_SUFFIXES)


def _looks_like_embedding(local: str) -> bool:
    return any(piece in local for piece in EMBEDDING_NAME_SUBSTRINGS)


def _default_route(home: _Home, param: Tensor, min_matrix_dim: int) -> tuple[Route, RouteReason]:
    adamw = Route(RouteKind.ADAMW)
    if home.local == "weight":
        if isinstance(home.module, (nn.Embedding, nn.EmbeddingBag)):
            return adamw, RouteReason.EMBEDDING
        if isinstance(home.module, _CONVOLUTIONS) and int(home.module.groups) > 1:
            return adamw, RouteReason.GROUPED_CONVOLUTION
    if _looks_like_tokens(home.local):
        return adamw, RouteReason.LEARNED_TOKENS
    if _looks_like_embedding(home.local):
        return adamw, RouteReason.EMBEDDING_NAME
    if param.ndim < 2:
        return adamw, RouteReason.VECTOR
    rows, cols = int(param.shape[0]), math.prod(int(d) for d in param.shape[1:])
    if min(rows, cols) < min_matrix_dim:
        return adamw, RouteReason.NARROW
    return Route(RouteKind.MATRIX), RouteReason.MATRIX


def _exempt_by_default(home: _Home, param: Tensor) -> bool:
    return param.ndim < 2 or _looks_like_tokens(home.local) or _looks_like_embedding(home.local)


def _collect_declarations(model: nn.Module, routes: Mapping[Tensor, Route] | None) -> dict[int, Route]:
    declared_by: list[tuple[str, Tensor, Route]] = [
        ("the routes argument", param, route) for param, route in (routes or {}).items()
    ]
    for module in model.modules():
        if isinstance(module, RouteProvider):
            declared_by.extend((type(module).__name__, p, r) for p, r in module.dion_routes())
    on_model = {id(p) for p in model.parameters()}
    result: dict[int, Route] = {}
    for source, param, route in declared_by:
        if id(param) not in on_model:
            raise ValueError(
                f"{source} declares a route for a parameter (shape {tuple(param.shape)}) "
                "that is not registered on the model"
            )
        earlier = result.setdefault(id(param), route)
        if earlier != route:
            raise ValueError(
                f"Conflicting routes for a parameter of shape {tuple(param.shape)}: "
                f"{earlier} vs {route} ({source})"
            )
    return result


def param_groups(
    model: nn.Module,
    *,
    params: Iterable[Tensor] | None = None,
    fraction: float = 0.25,
    selection_min_dim: int = 1024,
    min_matrix_dim: int = 8,
    routes: Mapping[Tensor, Route] | None = None,
    no_weight_decay: Collection[Tensor] | None = None,
) -> ParamGroups:
    """Route each trainable parameter and build ``Dion`` param groups.

    Returns ``(groups, report)``: AdamW groups first, then matrix groups, each in
    parameter order.  The report is logged at INFO on the ``dionw`` logger.

    Raises:
        ValueError: On out-of-range settings, invalid or conflicting routes, a
            parameter not registered on ``model``, or no trainable parameter.
    """
    if not 0.0 < fraction <= 1.0:
        raise ValueError(f"fraction must be in (0, 1], got {fraction}")
    if selection_min_dim <= 0 or min_matrix_dim <= 0:
        raise ValueError("selection_min_dim and min_matrix_dim must be positive")
    homes = _homes(model)
    chosen: OrderedDict[int, Tensor] = OrderedDict()
    for param in (model.parameters() if params is None else params):
        if param.requires_grad and id(param) not in chosen:
            chosen[id(param)] = param
    if not chosen:
        raise ValueError("No parameters require gradients")
    strangers = [tuple(p.shape) for key, p in chosen.items() if key not in homes]
    if strangers:
        raise ValueError(f"Parameters not registered on the model: {strangers[:8]}")
    if no_weight_decay is None:
        exempt = {key for key, p in chosen.items() if _exempt_by_default(homes[key], p)}
    else:
        exempt = {id(p) for p in no_weight_decay}
    declared = _collect_declarations(model, routes)

    buckets: OrderedDict[tuple, list[tuple[Tensor, RoutedParameter]]] = OrderedDict()
    for key, param in chosen.items():
        home = homes[key]
        if key in declared:
            route, reason = declared[key], RouteReason.DECLARED
        else:
            route, reason = _default_route(home, param, min_matrix_dim)
        if route.kind is RouteKind.MATRIX:
            if param.ndim < 2:
                raise ValueError(f"MATRIX route on {home.name} needs >= 2 dims, got {tuple(param.shape)}")
            _, rows, cols = block_shape(param, route.num_heads)
            if route.fraction is not None:
                row_fraction = float(route.fraction)
            else:
                row_fraction = fraction if min(rows, cols) >= selection_min_dim else 1.0
        elif route.kind is RouteKind.ADAMW:
            row_fraction = 1.0
        else:
            raise RuntimeError(f"Unhandled RouteKind: {route.kind}")
        entry = RoutedParameter(
            name=home.name, shape=tuple(int(d) for d in param.shape), kind=route.kind,
            fraction=row_fraction, num_heads=route.num_heads, decayed=key not in exempt, reason=reason,
        )
        group_key = (entry.kind, entry.num_heads, entry.fraction, entry.decayed)
        buckets.setdefault(group_key, []).append((param, entry))

    ordered = sorted(buckets.items(), key=lambda item: item[0][0] is RouteKind.MATRIX)  # stable: AdamW first
    groups: list[dict[str, Any]] = []
    for (kind, heads, row_fraction, decayed), members in ordered:
        group: dict[str, Any] = {"params": [p for p, _ in members], ROUTE_KEY: kind.value}
        if kind is RouteKind.MATRIX:
            group[FRACTION_KEY] = row_fraction
            group[NUM_HEADS_KEY] = heads
        if not decayed:
            group["weight_decay"] = 0.0
        groups.append(group)
    report = RoutingReport(tuple(entry for _, members in ordered for _, entry in members))
    _LOGGER.info("\n".join(report.lines()))
    return ParamGroups(groups=groups, report=report)
