"""Write the golden fixtures in this folder by running the reference itself.

Run once, in a container that has the reference's source tree (it is not
shipped with this repository and is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/reference

The reference is imported from ``<reference>/src`` on the CPU.  It needs a GPU
only for its Triton launches, so those are replaced by the torch forms the
reference itself falls back to for non-contiguous gradients
(``src/dionw/_matrix_step.py:190-192, :240-251``) and by ``bmm``/``baddbmm`` for
the two symmetric products; its ``torch.compile`` wrappers are removed with
``inspect.unwrap`` as ``bench/static_vs_dynamic.py:40-41`` does; the CUDA-only
parameter check is switched off.  Nothing else is touched: the optimizer, the
bucket packing, the Newton-Schulz schedule, NorMuon, the AdamW call and the EMA
are the reference's own code.

Outputs (``*.npz``; bfloat16 tensors are stored as their int16 bit pattern
under a ``__bf16`` suffix).
"""

from __future__ import annotations

import importlib.metadata
import inspect
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _import_reference(root: str):
    sys.path.insert(0, str(Path(root) / "src"))
    real_version = importlib.metadata.version
    importlib.metadata.version = lambda name: "0.0.0" if name == "dionw" else real_version(name)
    import dionw  # noqa: PLC0415
    import dionw._buckets as buckets  # noqa: PLC0415
    import dionw._gram as gram  # noqa: PLC0415
    import dionw._matrix_step as matrix_step  # noqa: PLC0415
    import dionw._polar_express as polar  # noqa: PLC0415
    import dionw._row_normalization as row_norm  # noqa: PLC0415
    import dionw.optimizer as optimizer  # noqa: PLC0415

    importlib.metadata.version = real_version
    optimizer._check_param = lambda param: None
    gram.ns_line_1 = lambda a: a @ a.mT
    gram.ns_line_2 = lambda a, alpha, beta: torch.baddbmm(a, a, a.mT, beta=beta, alpha=alpha)

    def line_1(a, *, out=None):
        return torch.matmul(a, a.mT, out=out)

    def line_2(a, alpha, beta, *, out=None):
        fused = torch.baddbmm if a.ndim == 3 else torch.addmm
        return fused(a, a, a.mT, beta=beta, alpha=alpha, out=out)

    polar.ns_line_1, polar.ns_line_2 = line_1, line_2

    def row_l1(grad, momentum, scores, cols):
        momentum.add_(grad.view(momentum.shape))
        scores.copy_(torch.linalg.vector_norm(momentum.view(-1, cols), ord=1, dim=-1))

    def copy_decay(grad, momentum, out, decay, *, nesterov):
        momentum.add_(grad.view(momentum.shape))
        if nesterov:
            momentum.mul_(decay)
            out.copy_((momentum + grad.view(momentum.shape)).view(out.shape))
        else:
            out.copy_(momentum.view(out.shape))
            momentum.mul_(decay)

    matrix_step.accumulate_row_l1 = row_l1
    matrix_step.accumulate_copy_decay = copy_decay
    row_norm.normalize_rows = inspect.unwrap(row_norm.normalize_rows)
    plain = {kind: inspect.unwrap(dionw.newton_schulz.newton_schulz_fn(kind)) for kind in dionw.NewtonSchulz}
    buckets.newton_schulz_fn = lambda kind: plain[kind]
    return dionw, matrix_step, plain


def _np(t: torch.Tensor) -> tuple[str, np.ndarray]:
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return "__bf16", t.contiguous().view(torch.int16).numpy()
    return "", t.contiguous().numpy()


def _save(name: str, tensors: dict[str, torch.Tensor]) -> None:
    out = {}
    for key, value in tensors.items():
        suffix, array = _np(value)
        out[key + suffix] = array
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(f"{name}.npz: {len(out)} arrays, {(HERE / f'{name}.npz').stat().st_size / 1e3:.0f} kB")


class _Net(torch.nn.Module):
    def __init__(self, shapes: list[tuple[int, int]], vec: int) -> None:
        super().__init__()
        self.mats = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.empty(r, c)) for r, c in shapes]
        )
        self.bias = torch.nn.Parameter(torch.empty(vec))
        self.table = torch.nn.Embedding(11, vec)


def _step_case(dionw, matrix_step, name: str, shapes, *, fraction, min_dim, steps=3, ema=None) -> None:
    """Seeded weights and grads through ``steps`` reference steps; every state saved."""
    gen = torch.Generator().manual_seed(0)
    net = _Net(shapes, 48)
    with torch.no_grad():
        for p in net.parameters():
            p.copy_(torch.randn(p.shape, generator=gen) * 0.02)
    groups, _ = dionw.param_groups(net, fraction=fraction, selection_min_dim=min_dim)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05, ema=ema)
    record: dict[str, torch.Tensor] = {f"init.{n}": p.detach().clone() for n, p in net.named_parameters()}
    picked: list[torch.Tensor] = []
    original = matrix_step._selected_update

    def spy(run, group, step):
        update, index = original(run, group, step)
        picked.append(index.squeeze(-1).sort(dim=-1).values.clone())
        return update, index

    matrix_step._selected_update = spy
    try:
        for s in range(steps):
            picked.clear()
            for n, p in net.named_parameters():
                p.grad = torch.randn(p.shape, generator=gen) * 1e-3
                record[f"grad{s}.{n}"] = p.grad.clone()
            opt.step()
            if opt.ema is not None:
                opt.ema.flush_pending_updates()
            for n, p in net.named_parameters():
                record[f"w{s}.{n}"] = p.detach().clone()
                for key, value in opt.state[p].items():
                    if isinstance(value, torch.Tensor):
                        record[f"state{s}.{n}.{key}"] = value.detach().clone()
            for i, idx in enumerate(picked):
                record[f"index{s}.{i}"] = idx
    finally:
        matrix_step._selected_update = original
    _save(name, record)


def _newton_schulz_case(dionw, plain) -> None:
    gen = torch.Generator().manual_seed(0)
    record = {}
    for tag, shape in (("wide", (3, 64, 256)), ("tall", (3, 256, 64)),
                       ("square", (3, 128, 128)), ("odd", (1, 96, 160))):
        x = torch.randn(shape, generator=gen)
        record[f"{tag}.x"] = x
        for kind in dionw.NewtonSchulz:
            record[f"{tag}.{kind.value}"] = plain[kind](x, 1e-8)
    _save("newton_schulz", record)


def _adamw_case() -> None:
    """``torch._fused_adamw_`` on CPU as src/dionw/_adamw.py:45-61 calls it."""
    gen = torch.Generator().manual_seed(0)
    p = torch.randn(1000, generator=gen) * 0.02
    m, v, step = torch.zeros_like(p), torch.zeros_like(p), torch.zeros(())
    record = {"p0": p.clone()}
    for s in range(4):
        g = torch.randn(1000, generator=gen) * 1e-3
        record[f"g{s}"] = g.clone()
        torch._foreach_add_([step], 1)
        torch._fused_adamw_([p], [g], [m], [v], [], [step], amsgrad=False, lr=3e-4, beta1=0.9,
                            beta2=0.95, weight_decay=0.05, eps=1e-8, maximize=False,
                            grad_scale=None, found_inf=None)
        record[f"p{s + 1}"], record[f"m{s + 1}"], record[f"v{s + 1}"] = p.clone(), m.clone(), v.clone()
    _save("adamw", record)


def _routing_case(dionw) -> None:
    """``param_groups`` of the reference on the modules of routing_models.py."""
    sys.path.insert(0, str(HERE))
    import routing_models  # noqa: PLC0415

    out = {}
    shapes = routing_models.Shapes()
    out["shapes_default"] = routing_models.describe(
        shapes, *dionw.param_groups(shapes, fraction=0.5, selection_min_dim=1024, min_matrix_dim=8))
    out["shapes_select"] = routing_models.describe(
        shapes, *dionw.param_groups(shapes, fraction=0.25, selection_min_dim=32, min_matrix_dim=8))
    out["shapes_no_decay"] = routing_models.describe(
        shapes, *dionw.param_groups(shapes, no_weight_decay=[shapes.bare, shapes.norm.weight]))
    attention = routing_models.Attention(dionw.Route, dionw.RouteKind)
    out["attention"] = routing_models.describe(
        attention, *dionw.param_groups(attention, fraction=0.5, selection_min_dim=16))
    routes = {attention.proj.weight: dionw.Route(dionw.RouteKind.MATRIX, fraction=1.0)}
    out["attention_routes"] = routing_models.describe(
        attention, *dionw.param_groups(attention, fraction=0.25, selection_min_dim=16, routes=routes))
    (HERE / "routing.json").write_text(json.dumps(out, indent=1))
    print("routing.json:", len(out), "cases")


def main() -> None:
    torch.set_num_threads(1)  # one summation order for every run of this script
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    dionw, matrix_step, plain = _import_reference(sys.argv[1])
    _step_case(dionw, matrix_step, "step_selected", [(64, 192), (64, 192), (128, 64)],
               fraction=0.25, min_dim=32)
    _step_case(dionw, matrix_step, "step_full_rows", [(96, 160), (160, 96), (64, 64)],
               fraction=0.25, min_dim=1024)
    _step_case(dionw, matrix_step, "step_ema", [(64, 96)], fraction=0.25, min_dim=1024,
               steps=4, ema=dionw.EMAConfig(decay=0.9, device=dionw.EMADevice.CPU, pin_memory=False))
    _newton_schulz_case(dionw, plain)
    _adamw_case()
    _routing_case(dionw)


if __name__ == "__main__":
    main()
