"""``param_groups`` against the reference's own routing of the same modules
(tests/golden/routing.json) and against the behaviours its test-suite pins
(tests/test_routing.py of the reference)."""

from __future__ import annotations

import json
import sys

import pytest
import torch
from torch import nn

from conftest import GOLDEN

import dionw_b200 as dionw
from dionw_b200 import Route, RouteKind, RouteReason, param_groups

sys.path.insert(0, str(GOLDEN))
import routing_models  # noqa: E402

GOLD = json.loads((GOLDEN / "routing.json").read_text())


def _same(case: str, model: nn.Module, result) -> None:
    ours = json.loads(json.dumps(routing_models.describe(model, *result)))
    assert ours["parameters"] == GOLD[case]["parameters"]
    assert ours["groups"] == GOLD[case]["groups"]
    assert ours["lines"] == GOLD[case]["lines"]


def test_default_rule_matches_reference() -> None:
    shapes = routing_models.Shapes()
    _same("shapes_default", shapes, param_groups(shapes, fraction=0.5, selection_min_dim=1024, min_matrix_dim=8))
    _same("shapes_select", shapes, param_groups(shapes, fraction=0.25, selection_min_dim=32, min_matrix_dim=8))
    _same("shapes_no_decay", shapes, param_groups(shapes, no_weight_decay=[shapes.bare, shapes.norm.weight]))


def test_declared_routes_match_reference() -> None:
    attention = routing_models.Attention(Route, RouteKind)
    _same("attention", attention, param_groups(attention, fraction=0.5, selection_min_dim=16))
    routes = {attention.proj.weight: Route(RouteKind.MATRIX, fraction=1.0)}
    _same("attention_routes", attention,
          param_groups(attention, fraction=0.25, selection_min_dim=16, routes=routes))


def test_default_rule_outcomes() -> None:
    _, report = param_groups(routing_models.Shapes(), fraction=0.5)
    got = {p.name: (p.kind, p.reason) for p in report.parameters}
    assert got["bare"] == (RouteKind.MATRIX, RouteReason.MATRIX)
    assert got["mha.in_proj_weight"] == (RouteKind.MATRIX, RouteReason.MATRIX)
    assert got["grouped.weight"] == (RouteKind.ADAMW, RouteReason.GROUPED_CONVOLUTION)
    assert got["embed.weight"] == (RouteKind.ADAMW, RouteReason.EMBEDDING)
    assert got["pos_embed"] == (RouteKind.ADAMW, RouteReason.EMBEDDING_NAME)
    assert got["register_tokens"] == (RouteKind.ADAMW, RouteReason.LEARNED_TOKENS)
    assert got["narrow.weight"] == (RouteKind.ADAMW, RouteReason.NARROW)
    assert got["norm.bias"] == (RouteKind.ADAMW, RouteReason.VECTOR)
    # name rules read the parameter's own name, not its module path
    assert got["pos_embedder.weight"] == (RouteKind.MATRIX, RouteReason.MATRIX)


def test_conflicting_and_foreign_declarations_raise() -> None:
    attention = routing_models.Attention(Route, RouteKind)
    with pytest.raises(ValueError, match="Conflicting routes"):
        param_groups(attention, routes={attention.qkv.weight: Route(RouteKind.ADAMW)})
    stranger = nn.Parameter(torch.zeros(8, 8))
    with pytest.raises(ValueError, match="not registered"):
        param_groups(attention, routes={stranger: Route(RouteKind.ADAMW)})
    with pytest.raises(ValueError, match="not registered"):
        param_groups(attention, params=[stranger])


def test_groups_are_adamw_first_and_frozen_parameters_are_skipped() -> None:
    shapes = routing_models.Shapes()
    shapes.conv.requires_grad_(False)
    groups, report = param_groups(shapes, fraction=0.5)
    kinds = [RouteKind(g[dionw.ROUTE_KEY]) for g in groups]
    first = kinds.index(RouteKind.MATRIX)
    assert set(kinds[:first]) == {RouteKind.ADAMW} and set(kinds[first:]) == {RouteKind.MATRIX}
    assert not any(p.name.startswith("conv.") for p in report.parameters)
    for group in groups:
        if "weight_decay" in group:
            assert group["weight_decay"] == 0.0
    assert "    adamw (learned tokens): register_tokens (16, 32)" in report.lines()


def test_invalid_settings_raise() -> None:
    shapes = routing_models.Shapes()
    with pytest.raises(ValueError, match="fraction"):
        param_groups(shapes, fraction=0.0)
    with pytest.raises(ValueError, match="must be positive"):
        param_groups(shapes, selection_min_dim=0)
    with pytest.raises(ValueError, match="MATRIX routes"):
        Route(RouteKind.ADAMW, num_heads=2)
    with pytest.raises(ValueError, match="num_heads must be positive"):
        Route(RouteKind.MATRIX, num_heads=0)
    with pytest.raises(ValueError, match=r"fraction must be in \(0, 1\]"):
        Route(RouteKind.MATRIX, fraction=1.5)
    with pytest.raises(ValueError, match="does not divide"):
        param_groups(shapes, routes={shapes.big.weight: Route(RouteKind.MATRIX, num_heads=7)})
    with pytest.raises(ValueError, match=">= 2 dims"):
        param_groups(shapes, routes={shapes.norm.weight: Route(RouteKind.MATRIX)})
    shapes.requires_grad_(False)
    with pytest.raises(ValueError, match="No parameters require gradients"):
        param_groups(shapes)
