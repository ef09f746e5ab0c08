"""Writes ``reference_gpu.npz``: outputs of the UNMODIFIED reference package running on a CUDA GPU.

    python tests/golden/make_golden_gpu.py <dir holding the reference's ``dionw`` package> <output.npz>

The reference's GPU step is compiled (torch.compile + Triton + cuBLAS) and differs in rounding from
its eager CPU run (``Q = Z + a I`` adds the fp32 coefficient there).  These vectors pin that path.
Inputs are regenerated from CPU generators with fixed seeds, so only compact outputs are stored:
for every orthogonalized matrix its row sums of squares and two seeded projections, for every
optimizer step the selected rows and per-row summaries of weights and state.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch
from torch import nn

NS_SHAPES = ((2, 256, 4096), (1, 1024, 4096), (2, 512, 512), (1, 2304, 768), (1, 896, 1024))
STEPS = 3


def ns_input(index: int, shape: tuple[int, int, int]) -> torch.Tensor:
    return torch.randn(*shape, generator=torch.Generator().manual_seed(100 + index))


def projections(y: torch.Tensor, seed: int) -> dict[str, torch.Tensor]:
    """Compact, sensitive summaries of a ``[N, rows, cols]`` result (computed in fp64 on the CPU)."""
    y = y.detach().double().cpu()
    gen = torch.Generator().manual_seed(seed)
    v = torch.randn(y.shape[-1], generator=gen, dtype=torch.float64)
    u = torch.randn(y.shape[-2], generator=gen, dtype=torch.float64)
    return {"rowsq": (y * y).sum(-1).float(), "right": (y @ v).float(), "left": (u @ y).float()}


class StepNet(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        gen = torch.Generator().manual_seed(0)
        mk = lambda *shape: nn.Parameter(torch.randn(*shape, generator=gen) * 0.02)  # noqa: E731
        self.wide = mk(1024, 4096)     # k = 256: the 256 x 4096 operand of config 1
        self.tall = mk(4096, 1024)     # k = 1024, transposed iteration
        self.small = mk(768, 2304)     # every row (min dim < 1024)
        self.bias = mk(4096)
        self.table = nn.Embedding(512, 256)
        with torch.no_grad():
            self.table.weight.copy_(torch.randn(512, 256, generator=gen) * 0.02)


def step_grads(step: int, net: nn.Module) -> list[torch.Tensor]:
    gen = torch.Generator().manual_seed(1000 + step)
    return [torch.randn(p.shape, generator=gen) * 1e-3 for p in net.parameters()]


def selected_rows(before: torch.Tensor, grad: torch.Tensor, after: torch.Tensor) -> torch.Tensor:
    return torch.nonzero((after != before + grad).any(dim=1)).flatten().to(torch.int32)


def main() -> None:
    sys.path.insert(0, sys.argv[1])
    import dionw

    device = "cuda"
    out: dict[str, np.ndarray] = {}
    fn = dionw.newton_schulz.newton_schulz_fn(dionw.NewtonSchulz.GRAM)
    for index, shape in enumerate(NS_SHAPES):
        y = fn(ns_input(index, shape).to(device), 1e-8)
        for key, value in projections(y, 7 + index).items():
            out[f"ns{index}.{key}"] = value.numpy()
    net = StepNet().to(device)
    groups, _ = dionw.param_groups(net)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05, ema=dionw.EMAConfig(decay=0.99, device=dionw.EMADevice.GPU))
    names = [n for n, _ in net.named_parameters()]
    for step in range(STEPS):
        grads = step_grads(step, net)
        before = {}
        for (name, p), g in zip(net.named_parameters(), grads):
            p.grad = g.to(device)
            m = opt.state[p].get("momentum") if p in opt.state else None
            before[name] = torch.zeros_like(p) if m is None else m.detach().clone()
        opt.step()
        torch.cuda.synchronize()
        for (name, p), g in zip(net.named_parameters(), grads):
            state = opt.state[p]
            tag = f"step{step}.{name}"
            value = p.detach().reshape(p.shape[0], -1)[None]
            for key, summary in projections(value, 50).items():
                out[f"{tag}.w.{key}"] = summary.numpy()
            for key, summary in projections(state["ema_shadow"].reshape(p.shape[0], -1)[None], 51).items():
                out[f"{tag}.ema.{key}"] = summary.numpy()
            if "momentum" in state:
                if name in ("wide", "tall"):
                    out[f"{tag}.rows"] = selected_rows(before[name], g.to(device), state["momentum"]).cpu().numpy()
                for key, summary in projections(state["momentum"][None], 52).items():
                    out[f"{tag}.momentum.{key}"] = summary.numpy()
                out[f"{tag}.variance"] = state["variance"].detach().float().cpu().numpy()
            else:
                for key in ("exp_avg", "exp_avg_sq"):
                    for k2, summary in projections(state[key].reshape(p.shape[0], -1)[None], 53).items():
                        out[f"{tag}.{key}.{k2}"] = summary.numpy()
    out["names"] = np.array(names)
    out["torch_version"] = np.array(torch.__version__)
    out["gpu"] = np.array(torch.cuda.get_device_name())
    Path(sys.argv[2]).parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(sys.argv[2], **out)
    print("wrote", sys.argv[2], len(out), "arrays")


if __name__ == "__main__":
    main()
