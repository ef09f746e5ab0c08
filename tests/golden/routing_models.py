"""Small modules whose parameters hit every routing rule; shared by the fixture
generator (which routes them with the reference) and the tests."""

from __future__ import annotations

import torch
from torch import nn


class Shapes(nn.Module):
    """One parameter per outcome of the default rule."""

    def __init__(self) -> None:
        super().__init__()
        self.bare = nn.Parameter(torch.zeros(32, 48))
        self.mha = nn.MultiheadAttention(32, 4, batch_first=True)
        self.up = nn.ConvTranspose2d(32, 16, 2, stride=2)
        self.conv = nn.Conv2d(32, 16, 3)
        self.grouped = nn.Conv2d(32, 32, 3, groups=4)
        self.embed = nn.Embedding(64, 32)
        self.bag = nn.EmbeddingBag(10, 16)
        self.pos_embed = nn.Parameter(torch.zeros(16, 32))
        self.register_tokens = nn.Parameter(torch.zeros(16, 32))
        self.cls_token = nn.Parameter(torch.zeros(1, 32))
        self.relative_position_bias_table = nn.Parameter(torch.zeros(9, 4))
        self.narrow = nn.Linear(32, 4)
        self.norm = nn.LayerNorm(32)
        self.pos_embedder = nn.Linear(32, 32, bias=False)
        self.big = nn.Linear(96, 64, bias=False)


class Attention(nn.Module):
    """Declares routes through ``dion_routes``; ``route_cls``/``kind_cls`` are the
    ``Route`` and ``RouteKind`` of whichever implementation routes the model."""

    def __init__(self, route_cls, kind_cls) -> None:
        super().__init__()
        self._route, self._kind = route_cls, kind_cls
        self.qkv = nn.Linear(64, 192, bias=False)
        self.patch = nn.Linear(48, 64, bias=False)
        self.proj = nn.Linear(64, 64)

    def dion_routes(self):
        return (
            (self.qkv.weight, self._route(self._kind.MATRIX, num_heads=6, fraction=None)),
            (self.patch.weight, self._route(self._kind.ADAMW, num_heads=None, fraction=None)),
        )


def describe(model: nn.Module, groups, report) -> dict:
    """A JSON-able record of a routing result."""
    names = {id(p): n for n, p in model.named_parameters()}
    return {
        "groups": [
            {**{k: v for k, v in g.items() if k != "params"}, "params": [names[id(p)] for p in g["params"]]}
            for g in groups
        ],
        "parameters": [
            {"name": p.name, "shape": list(p.shape), "kind": p.kind.value, "fraction": p.fraction,
             "num_heads": p.num_heads, "decayed": p.decayed, "reason": p.reason.value}
            for p in report.parameters
        ],
        "lines": report.lines(),
    }


class StepNet(nn.Module):
    """The parameter set of the ``step_*.npz`` fixtures: matrices ``mats.<i>``, a
    48-element ``bias`` and an 11 x 48 embedding ``table``."""

    def __init__(self, shapes: list[tuple[int, int]], vec: int = 48) -> None:
        super().__init__()
        self.mats = nn.ParameterList([nn.Parameter(torch.empty(r, c)) for r, c in shapes])
        self.bias = nn.Parameter(torch.empty(vec))
        self.table = nn.Embedding(11, vec)
