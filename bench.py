"""Optimizer-step benchmark: ``python bench.py --gpus N --steps K --warmup W``.

Workload (N = 1 and up): the Llama-3-8B-shaped parameter set — 32 layers of
q/o 4096x4096, k/v 1024x4096, gate/up 14336x4096, down 4096x14336 (Dion3,
fraction 0.25), 65 RMSNorm[4096] and embed + lm_head 128256x4096 (AdamW); fp32
masters, synthetic weights ~N(0, 0.02^2) and gradients ~N(0, 1e-3^2), lr 3e-4,
weight decay 0.05.  A "step" is one ``optimizer.step()`` over the whole set; the
gradients stay the same tensors across timed steps, as in the reference's own
benchmark (bench/optimizer_step.py:91-96 there).  Working set (~100 GB) is far
larger than L2, so nothing is flushed between steps.

Prints ONE JSON line (rank 0).  ``value`` is the device time of K steps; the
``stages`` come from K further steps run right after them with every stage
bracketed by CUDA events; ``e2e`` copies every gradient from pinned host memory
each step.  ``--impl reference`` times the CPU oracle
(``oracle/dion_oracle.py``, the restatement of the reference's step pinned by
its fixtures) on the host cores instead, on a bounded sample of the same
workload (one whole layer, scaled by the layer count).

Other workloads: ``--config gpt2-small`` (config 2), ``--config single-1024x4096``
(config 1), ``--config llama3-70b-20layers`` (config 5, 8 GPUs), ``--config gram-ns``
(config 4, the Newton-Schulz microbenchmark), ``--config gemm-sustained`` (the GEMM
against cuBLAS under the power cap); ``--ema cpu|gpu``, ``--graph-replay``.
"""

from __future__ import annotations

import argparse
import contextlib
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch
from torch import nn

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LR, WEIGHT_DECAY = 3e-4, 0.05
CONFIGS = {
    # name: (layers, d_model, d_kv, d_ff, vocab)
    "llama3-8b": (32, 4096, 1024, 14336, 128256),
    "llama3-8b-2layers": (2, 4096, 1024, 14336, 16032),
    # the matrix blocks one rank of eight owns at the full configuration (8 gate/up, 8 q/o, 8 k/v, 4 down)
    "llama3-8b-4layers": (4, 4096, 1024, 14336, 16032),
    "tiny": (2, 1024, 256, 3584, 4096),
    # 20-layer slice of the Llama-3-70B shapes, embedding only, GPU EMA (decay 0.9999): 8 GPUs
    "llama3-70b-20layers": (20, 8192, 1024, 28672, 128256),
    "llama3-70b-1layer": (1, 8192, 1024, 28672, 16032),
    # GPT-2-small (12 layers, d = 768, ~124 M parameters): the shapes are fixed in Gpt2Shaped
    "gpt2-small": (12, 768, 768, 3072, 50257),
    # one fp32 weight 1024 x 4096 (Dion3, k = 256) and a bias[4096] (AdamW): small enough for the
    # CPU arm to run the whole workload, unscaled; the shapes are fixed in SingleMatrix
    "single-1024x4096": (1, 4096, 1024, 0, 0),
}
EMBED_ONLY_WITH_EMA = {"llama3-70b-20layers", "llama3-70b-1layer"}
# Above this many bytes of fp32 weights + gradients per GPU the gradients are one tensor per
# shape, shared by all layers (the step reads them, never writes them).
SHARED_GRADS_ABOVE = 120e9


# ---------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------
class Layer(nn.Module):
    def __init__(self, d: int, dkv: int, dff: int, device) -> None:
        super().__init__()
        mk = lambda r, c: nn.Parameter(torch.empty(r, c, device=device))  # noqa: E731
        self.q, self.k, self.v, self.o = mk(d, d), mk(dkv, d), mk(dkv, d), mk(d, d)
        self.gate, self.up, self.down = mk(dff, d), mk(dff, d), mk(d, dff)
        self.norm1 = nn.Parameter(torch.empty(d, device=device))
        self.norm2 = nn.Parameter(torch.empty(d, device=device))


class LlamaShaped(nn.Module):
    """Only the parameters: nothing here is ever run forward."""

    def __init__(self, name: str, device) -> None:
        super().__init__()
        layers, d, dkv, dff, vocab = CONFIGS[name]
        self.embed = nn.Embedding(vocab, d, device=device)
        self.layers = nn.ModuleList(Layer(d, dkv, dff, device) for _ in range(layers))
        self.norm = nn.Parameter(torch.empty(d, device=device))
        self.lm_head = None if name in EMBED_ONLY_WITH_EMA else nn.Linear(d, vocab, bias=False, device=device)

    @torch.no_grad()
    def init_(self, seed: int) -> None:
        gen = torch.Generator(device=self.norm.device).manual_seed(seed)
        for p in self.parameters():
            p.normal_(0.0, 0.02, generator=gen)


class Gpt2Block(nn.Module):
    def __init__(self, d: int, device) -> None:
        super().__init__()
        mk = lambda *shape: nn.Parameter(torch.empty(*shape, device=device))  # noqa: E731
        self.ln1_w, self.ln1_b, self.ln2_w, self.ln2_b = mk(d), mk(d), mk(d), mk(d)
        self.c_attn, self.c_proj = mk(d, 3 * d), mk(d, d)
        self.fc, self.proj = mk(d, 4 * d), mk(4 * d, d)


class Gpt2Shaped(nn.Module):
    """GPT-2-small's parameter shapes (12 layers, d = 768): every matrix has a dimension below 1024,
    so all rows are updated (no selection); wte and wpe go through AdamW."""

    def __init__(self, device) -> None:
        super().__init__()
        self.wte = nn.Embedding(50257, 768, device=device)
        self.wpe = nn.Embedding(1024, 768, device=device)
        self.layers = nn.ModuleList(Gpt2Block(768, device) for _ in range(12))
        self.norm = nn.Parameter(torch.empty(768, device=device))
        self.ln_f_b = nn.Parameter(torch.empty(768, device=device))
        self.lm_head = None

    init_ = LlamaShaped.init_


class SingleMatrix(nn.Module):
    """One weight 1024 x 4096 and one bias[4096]."""

    def __init__(self, device) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(1024, 4096, device=device))
        self.norm = nn.Parameter(torch.empty(4096, device=device))   # the bias: AdamW, no decay
        self.lm_head = None

    init_ = LlamaShaped.init_


def build_model(config: str, device) -> nn.Module:
    if config == "gpt2-small":
        return Gpt2Shaped(device)
    if config == "single-1024x4096":
        return SingleMatrix(device)
    return LlamaShaped(config, device)


def flops_newton_schulz(m: int, n: int) -> float:
    """Algorithmic FLOPs of one orthogonalization of an m x n operand (m <= n): the Gram
    schedule's product census, symmetric products counted as half."""
    if m == n:
        return 2.0 * 10.0 * m**3
    return 2.0 * (3.0 * m * m * n + 11.5 * m**3)


# DRAM bytes the products of one Gram Newton-Schulz move for an m x n operand: the operand census
# 2 B x (6 m n + 40 m^2) (every product reads its operands and writes its result once) times 1.06,
# the ratio an ncu capture of the 18 products of four 3584 x 4096 blocks measured against it
# (1.278 GB per block; dram__bytes_read.sum + dram__bytes_write.sum).
NS_TRAFFIC_CALIBRATION = 1.06


def traffic_newton_schulz(m: int, n: int) -> float:
    return NS_TRAFFIC_CALIBRATION * 2.0 * (6.0 * m * n + 40.0 * m * m)


def flops_newton_schulz_executed(m: int, n: int) -> float:
    """FLOPs the kernels execute for the same orthogonalization: the products Q Z, G Z and Z RZ are
    symmetric too and run on the lower-triangle schedule (7 m^3 instead of 11.5 m^3)."""
    if m == n:
        return 2.0 * 10.0 * m**3
    return 2.0 * (3.0 * m * m * n + 7.0 * m**3)


def census(groups: list[dict]) -> dict[str, float]:
    """Algorithmic work of one step, from the optimizer's groups: elements, bytes per pass,
    Newton-Schulz FLOPs.  Blocks that update every row (fraction 1) take the full-row path:
    accumulate, copy and decay in one pass (16 B/element: read G and M, write M and the fp32 copy),
    then norm + pack (6 B/element)."""
    from dionw_b200._keys import FRACTION_KEY, ROUTE_KEY
    from dionw_b200.routing import RouteKind

    e = es = ns = adam = ns_traffic = ns_exec = full = 0.0
    for group in groups:
        if RouteKind(group[ROUTE_KEY]) is not RouteKind.MATRIX:
            adam += sum(p.numel() for p in group["params"])
            continue
        fraction = float(group[FRACTION_KEY])
        for w in group["params"]:
            rows, cols = w.shape[0], w[0].numel()
            k = min(rows, max(1, math.ceil(fraction * rows)))
            e += rows * cols
            es += k * cols
            if k == rows:
                full += rows * cols
            m, n = min(k, cols), max(k, cols)
            ns += flops_newton_schulz(m, n)
            ns_traffic += traffic_newton_schulz(m, n)
            ns_exec += flops_newton_schulz_executed(m, n)
    selecting = e - full
    return {
        "matrix_elements": e, "selected_elements": es, "adamw_elements": adam, "ns_flops": ns,
        "ns_traffic": ns_traffic, "ns_flops_executed": ns_exec,
        "bytes_accumulate": 12 * selecting + 16 * full, "bytes_pack": 10 * (es - full) + 10 * full,
        "bytes_finish": 2 * es, "bytes_apply": 8 * e + 2 * es, "bytes_adamw": 28 * adam, "bytes_ema": 12 * (e + adam),
    }


# ---------------------------------------------------------------------------
# timing helpers
# ---------------------------------------------------------------------------
class StageTimer:
    """Brackets the stages of every run (and the AdamW groups) with CUDA events on the
    current stream; ``collect()`` sums milliseconds per stage after a synchronize."""

    def __init__(self) -> None:
        self.events: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self.blocks: dict[str, int] = {}
        self.enabled = False

    @contextlib.contextmanager
    def __call__(self, name: str):
        if not self.enabled:
            yield
            return
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        yield
        end.record()
        self.events.append((name, start, end))
        if name == "newton_schulz":   # also per operand shape: blocks x selected rows x cols of the run
            from dionw_b200 import _matrix_step

            count, _, k, cols = _matrix_step.CURRENT_RUN or (0, 0, 0, 0)
            self.events.append((f"ns:{k}x{cols}", start, end))
            self.blocks[f"ns:{k}x{cols}"] = self.blocks.get(f"ns:{k}x{cols}", 0) + count

    def collect(self) -> dict[str, float]:
        torch.cuda.synchronize()
        totals: dict[str, float] = {}
        for name, start, end in self.events:
            totals[name] = totals.get(name, 0.0) + start.elapsed_time(end)
        self.events.clear()
        return totals


class ClockSampler:
    """``nvidia-smi`` sampling of SM clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc, self.file = index, None, None

    def start(self) -> None:
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def samples(self) -> int:
        if self.proc is None or self.file is None:
            return 1 << 30
        try:
            return Path(self.file.name).read_text().count("\n")
        except OSError:
            return 1 << 30

    def stop(self) -> dict | None:
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 6]
        os.unlink(self.file.name)
        if not rows:
            return None
        sm = [float(r[0]) for r in rows if r[0].strip().replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any("Active" == r[3 + i].strip() for r in rows)]
        loaded = [v for v in sm if v > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": float(rows[0][1]), "samples": len(rows),
                "power_w_max": max(float(r[2]) for r in rows), "reasons": reasons}


def split_ns_shapes(stages: dict[str, float], blocks: dict[str, int], steps: int) -> list[dict]:
    """Takes the per-shape Newton-Schulz entries (``ns:<m>x<n>``) out of ``stages`` and returns them as
    rows: operand shape, blocks and milliseconds per step on this rank, executed TFLOP/s."""
    rows = []
    for key in sorted(k for k in stages if k.startswith("ns:")):
        ms = stages.pop(key)
        k, cols = (int(v) for v in key[3:].split("x"))
        m, n = min(k, cols), max(k, cols)
        count = blocks.get(key, 0) / max(1, steps)
        rows.append({"operand": [m, n], "blocks": count, "ms": ms,
                     "executed_TFLOP/s": count * flops_newton_schulz_executed(m, n) / ms / 1e9 if ms else None,
                     "algorithmic_TFLOP/s": count * flops_newton_schulz(m, n) / ms / 1e9 if ms else None})
    blocks.clear()
    return rows


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ---------------------------------------------------------------------------
# the CPU arm (oracle) — also the cpu_baseline of the GPU arm
# ---------------------------------------------------------------------------
_REFERENCE_CPU: tuple[object | None, str] | None = None


def reference_on_cpu() -> tuple[object | None, str]:
    """The UNMODIFIED reference package from ``baseline/_ref`` (git-ignored; it travels with the
    repository's working copy), made to step on CPU tensors: its Triton launches are replaced by the
    torch forms the reference itself uses for non-contiguous gradients
    (src/dionw/_matrix_step.py:190-192, :240-251) and by ``bmm``/``baddbmm`` for the two symmetric
    products, ``torch.compile`` wrappers are taken off with ``inspect.unwrap`` (as its own
    bench/static_vs_dynamic.py:40-41 does) and the CUDA-only parameter check is switched off.  The
    optimizer, bucket packing, Newton-Schulz schedule, NorMuon, AdamW call and EMA stay its own code.
    Returns ``(module, "")`` or ``(None, why)``."""
    global _REFERENCE_CPU
    if _REFERENCE_CPU is not None:
        return _REFERENCE_CPU
    import inspect

    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "dionw" / "__init__.py").exists():
        _REFERENCE_CPU = (None, "no reference package under baseline/_ref")
        return _REFERENCE_CPU
    sys.path.insert(0, str(ref_root))
    try:
        import dionw as ref
        import dionw._buckets as buckets
        import dionw._gram as gram
        import dionw._matrix_step as matrix_step
        import dionw._polar_express as polar
        import dionw._row_normalization as row_norm
        import dionw.optimizer as ref_optimizer

        ref_optimizer._check_param = lambda param: None
        gram.ns_line_1 = lambda a: a @ a.mT
        gram.ns_line_2 = lambda a, alpha, beta: torch.baddbmm(a, a, a.mT, beta=beta, alpha=alpha)
        polar.ns_line_1 = lambda a, *, out=None: torch.matmul(a, a.mT, out=out)
        polar.ns_line_2 = lambda a, alpha, beta, *, out=None: (torch.baddbmm if a.ndim == 3 else torch.addmm)(
            a, a, a.mT, beta=beta, alpha=alpha, out=out)

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

        matrix_step.accumulate_row_l1, matrix_step.accumulate_copy_decay = row_l1, copy_decay
        row_norm.normalize_rows = inspect.unwrap(row_norm.normalize_rows)
        plain = {kind: inspect.unwrap(ref.newton_schulz.newton_schulz_fn(kind)) for kind in ref.NewtonSchulz}
        buckets.newton_schulz_fn = lambda kind: plain[kind]
        _REFERENCE_CPU = (ref, "")
    except Exception as exc:  # noqa: BLE001 - the reason is reported in the JSON line
        _REFERENCE_CPU = (None, f"the reference does not import on this host: {exc!r}")
    finally:
        sys.path.remove(str(ref_root))
    return _REFERENCE_CPU


def cpu_sample_step(config: str, steps: int, warmup: int) -> dict:
    """Times the reference's step on the host cores, on a bounded sample of the workload scaled to
    the whole set.  The reference itself (``reference_on_cpu``, ``kind: "reference"``) when its
    package is there, else the oracle port (``kind: "port"``).

    Matrix part: one whole layer's blocks, multiplied by the layer count, where a layer is
    affordable (d_model <= 4096: about 3 s per sample step on 16 threads at the Llama-3-8B shapes);
    for wider models the attention blocks alone, scaled by Newton-Schulz FLOPs.  AdamW part: a
    slice of the embedding table (at most 2^24 elements), scaled by elements.  The single-matrix
    configuration is run whole."""
    layers, d, dkv, dff, vocab = CONFIGS[config]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(0)
    if config == "gpt2-small":
        per_layer = [(d, 3 * d), (d, d), (d, 4 * d), (4 * d, d)]
        shapes, what = per_layer, "one layer's c_attn, c_proj, fc, proj blocks"
        adam_total = (vocab + 1024) * d + (4 * layers + 2) * d
    elif config == "single-1024x4096":
        per_layer = shapes = [(1024, 4096)]
        what = "the whole workload: the 1024x4096 weight"
        adam_total = 4096
    else:
        per_layer = [(d, d)] * 2 + [(dkv, d)] * 2 + [(dff, d)] * 2 + [(d, dff)]
        tables = 1 if config in EMBED_ONLY_WITH_EMA else 2
        adam_total = tables * vocab * d + (2 * layers + 1) * d
        if d <= 4096:
            shapes, what = per_layer, f"one whole layer (q, o, k, v, gate, up, down at d = {d})"
        else:
            shapes = [(d, d), (d, d), (dkv, d), (dkv, d)]
            what = f"one layer's q, o ({d}x{d}) and k, v ({dkv}x{d}) blocks"

    def block_flops(r: int, c: int) -> float:
        k = -(-r // 4) if min(r, c) >= 1024 else r
        return flops_newton_schulz(min(k, c), max(k, c))

    def median_ms(step) -> float:
        times = []
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            step()
            if i >= warmup:
                times.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(times)

    adam_sample = min(adam_total, 1 << 24)
    reference, why_not = reference_on_cpu()
    if reference is not None:
        kind = "reference"
        who = "the reference package itself (torch eager on CPU tensors, its Triton launches replaced by its own torch forms)"

        class Sample(nn.Module):
            def __init__(self, sizes) -> None:
                super().__init__()
                self.mats = nn.ParameterList([nn.Parameter(torch.randn(size, generator=gen) * 0.02) for size in sizes])

        def stepper(module: nn.Module, routes=None):
            groups, _ = reference.param_groups(module, routes=routes)
            optimizer = reference.Dion(groups, lr=LR, weight_decay=WEIGHT_DECAY)
            for p in module.parameters():
                p.grad = torch.randn(p.shape, generator=gen) * 1e-3
            return optimizer.step

        matrix_step = stepper(Sample(shapes))
        table = nn.Embedding(1, adam_sample)   # an embedding goes to AdamW, with weight decay, like the model's tables
        with torch.no_grad():
            table.weight.normal_(0.0, 0.02, generator=gen)
        adam_step = stepper(table)
    else:
        from oracle import dion_oracle as oracle

        kind = "port"
        who = f"CPU oracle port ({why_not})"
        weights = [torch.randn(size, generator=gen) * 0.02 for size in shapes]
        grads = [torch.randn(size, generator=gen) * 1e-3 for size in shapes]
        matrices = oracle.OracleDion(matrix=[(w, 0.25 if min(w.shape) >= 1024 else 1.0) for w in weights],
                                     adamw=[], lr=LR, weight_decay=WEIGHT_DECAY)
        matrix_step = lambda: matrices.step(grads, [])  # noqa: E731
        table = torch.randn(adam_sample, generator=gen) * 0.02
        table_grad = torch.randn(adam_sample, generator=gen) * 1e-3
        vectors = oracle.OracleDion(matrix=[], adamw=[(table, None)], lr=LR, weight_decay=WEIGHT_DECAY)
        adam_step = lambda: vectors.step([], [table_grad])  # noqa: E731

    matrix_ms = median_ms(matrix_step)
    sample_flops = sum(block_flops(r, c) for r, c in shapes)
    model_flops = layers * sum(block_flops(r, c) for r, c in per_layer)
    matrix_scale = model_flops / sample_flops
    adam_ms = median_ms(adam_step)
    adam_scale = adam_total / adam_sample
    scaled = matrix_ms * matrix_scale + adam_ms * adam_scale
    whole = matrix_scale == 1.0 and adam_scale == 1.0
    return {
        "value": scaled, "unit": "ms", "cores": cores, "kind": kind,
        "sample": (f"{who}, {cores} threads, median of {steps} steps after {warmup}: "
                   f"{what}: {matrix_ms:.1f} ms x{matrix_scale:.0f} (Newton-Schulz FLOPs of the whole set / of the "
                   f"sample); AdamW on {adam_sample} elements: {adam_ms:.2f} ms x{adam_scale:.1f} (elements)"),
        "sample_ms": matrix_ms + adam_ms, "extrapolated": not whole,
        "scale": {"matrix": matrix_scale, "adamw": adam_scale},
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_sample_step(args.config, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": "optimizer_step_ms", "value": base["value"], "unit": "ms",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["value"],
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32 state, fp16 Newton-Schulz", "data": "synthetic",
        "config": {"workload": f"{args.config}-shaped parameter set, fp32 masters, Dion3 fraction 0.25 + AdamW",
                   "lr": LR, "weight_decay": WEIGHT_DECAY,
                   "arm": ("the reference package on host CPU cores" if base["kind"] == "reference"
                           else "reference's algorithm on host CPU cores (oracle port)")},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# the reference's own GPU step (``--impl reference-gpu``; ``--impl reference`` is the CPU arm)
# ---------------------------------------------------------------------------
def run_reference_gpu_arm(args) -> None:
    """The UNMODIFIED reference package, if a copy sits under ``baseline/_ref`` (git-ignored), on the
    same workload through its own public API: ``dionw.param_groups`` + ``dionw.Dion(...).step()``
    (torch.compile + Triton + cuBLAS inside).  Timed like the B200 arm.  Prints an ``unavailable``
    line when the package is not there or does not run under this torch."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    ref_root = ROOT / "baseline" / "_ref"

    def unavailable(why: str) -> None:
        print(json.dumps({"impl": "reference-gpu", "unavailable": why[:400]}), flush=True)

    if not (ref_root / "dionw" / "__init__.py").exists():
        unavailable("no reference package under baseline/_ref (its build backend, hatchling, is not installable offline)")
        return
    sys.path.insert(0, str(ref_root))
    try:
        import dionw as reference
    except Exception as exc:  # noqa: BLE001 - the reason is the result
        unavailable(f"import failed: {exc!r}")
        return
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    try:
        model = build_model(args.config, device)
        model.init_(seed=0)
        routes = {} if model.lm_head is None else {model.lm_head.weight: reference.Route(reference.RouteKind.ADAMW)}
        groups, _ = reference.param_groups(model, routes=routes)
        optimizer = reference.Dion(groups, lr=LR, weight_decay=WEIGHT_DECAY)
        gen = torch.Generator(device=device).manual_seed(1)
        for p in model.parameters():
            p.grad = torch.empty_like(p).normal_(0.0, 1e-3, generator=gen)
        t0 = time.time()
        for _ in range(max(3, args.warmup)):
            optimizer.step()
        torch.cuda.synchronize()
        warm_s = time.time() - t0
        sampler = ClockSampler(0)
        sampler.start()
        times = []
        for _ in range(args.steps):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            optimizer.step()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        clocks = sampler.stop()
    except Exception as exc:  # noqa: BLE001
        import traceback
        unavailable(f"the reference's step failed under torch {torch.__version__}: {exc!r} | {traceback.format_exc()[-300:]}")
        return
    total = sum(times)
    line = {
        "impl": "reference-gpu", "metric": "optimizer_step_ms", "value": total / len(times), "unit": "ms", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": total / len(times),
        "median_ms": statistics.median(times), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32 state, fp16 Newton-Schulz", "data": "synthetic",
        "config": {"workload": f"{args.config}-shaped parameter set, fp32 masters, Dion3 fraction 0.25 + AdamW",
                   "arm": f"unmodified reference package (torch {torch.__version__}, its Triton + cuBLAS step), "
                          f"warm-up incl. compilation {warm_s:.1f} s"},
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_reference_gpu_ns(args) -> None:
    """The reference's own Gram Newton-Schulz entry on the microbenchmark's batches (same inputs as
    ``--config gram-ns``), whole-call device time, median."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "dionw" / "__init__.py").exists():
        print(json.dumps({"impl": "reference-gpu", "unavailable": "no reference package under baseline/_ref"}))
        return
    sys.path.insert(0, str(ref_root))
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    rows_out = []
    try:
        from dionw.newton_schulz import NewtonSchulz, newton_schulz_fn

        fn = newton_schulz_fn(NewtonSchulz.GRAM)
        for m, n in NS_SHAPES:
            gen = torch.Generator(device=device).manual_seed(m * 31 + n)
            x = torch.randn(NS_BATCH, m, n, device=device, generator=gen)
            x = (x / torch.linalg.matrix_norm(x, keepdim=True)).bfloat16()
            for _ in range(max(3, args.warmup)):
                y = fn(x, 1e-8)
            times = []
            for _ in range(args.steps):
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                y = fn(x, 1e-8)
                end.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(end))
            call_ms = statistics.median(times)
            y0 = y[0].float()
            err = float(torch.linalg.matrix_norm(y0 @ y0.T - torch.eye(m, device=device)))
            rows_out.append({"shape": [m, n], "batch": NS_BATCH, "call_ms": call_ms,
                             "TFLOP/s_of_call": NS_BATCH * flops_newton_schulz(m, n) / call_ms / 1e9,
                             "orthogonality_error": err, "error_per_sqrt_m": err / m**0.5})
            del x, y, y0
            torch.cuda.empty_cache()
    except Exception as exc:  # noqa: BLE001
        import traceback
        print(json.dumps({"impl": "reference-gpu", "unavailable": f"failed under torch {torch.__version__}: {exc!r} | "
                          f"{traceback.format_exc()[-300:]}", "shapes": rows_out}), flush=True)
        return
    print(json.dumps({"impl": "reference-gpu", "metric": "gram_newton_schulz_tflops", "unit": "TFLOP/s",
                      "value": sum(NS_BATCH * flops_newton_schulz(*r["shape"]) for r in rows_out)
                      / sum(r["call_ms"] for r in rows_out) / 1e9,
                      "config": {"workload": "the reference's Gram Newton-Schulz entry, whole call"}, "shapes": rows_out}),
          flush=True)


# ---------------------------------------------------------------------------
# the Gram Newton-Schulz microbenchmark (``--config gram-ns``)
# ---------------------------------------------------------------------------
NS_SHAPES = ((1024, 1024), (1024, 4096), (4096, 14336), (8192, 28672))
NS_BATCH = 16


def run_ns_microbench(args) -> None:
    """Batches of 16 bf16 matrices ~N(0,1) scaled to unit Frobenius norm, orthogonalized by the
    public entry ``gram_polar_express(x, 1e-8)``.  Per shape: device time of the whole call and
    of the iteration alone (operands already packed), algorithmic TFLOP/s of the iteration and
    the orthogonality error ``||Y Y^T - I||_F`` of the first matrix."""
    from dionw_b200 import _native
    from dionw_b200.newton_schulz import NewtonSchulz, gram_polar_express, newton_schulz_fn, padded, run_iteration

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    _native.library()
    peaks, peaks_kind = measured_peaks()
    fn = newton_schulz_fn(NewtonSchulz.GRAM)
    sampler = ClockSampler(0)
    sampler.start()
    launches_before = _native.launch_count()
    rows_out = []
    for m, n in NS_SHAPES:
        gen = torch.Generator(device=device).manual_seed(m * 31 + n)
        x = torch.randn(NS_BATCH, m, n, device=device, generator=gen)
        x = (x / torch.linalg.matrix_norm(x, keepdim=True)).bfloat16()

        def whole():
            return gram_polar_express(x, 1e-8)

        packed = torch.empty(NS_BATCH, m, padded(n), dtype=torch.float16, device=device)
        packed[..., :n] = x
        scratch = torch.empty(fn.workspace_bytes(NS_BATCH, m, n), dtype=torch.uint8, device=device)
        work = packed.clone()

        def iteration():
            work.copy_(packed)
            return run_iteration(fn, work, m, n, scratch, None)

        def clock(call) -> float:
            for _ in range(args.warmup):
                call()
            times = []
            for _ in range(args.steps):
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                call()
                end.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(end))
            return statistics.median(times)

        # the refill of the operand is a 2-byte copy, timed alone and taken off the iteration's time
        refill = clock(lambda: work.copy_(packed))
        iter_ms = clock(iteration) - refill
        whole_ms = clock(whole)
        y = whole()[0].float()
        err = float(torch.linalg.matrix_norm(y @ y.T - torch.eye(m, device=device)))
        flops = NS_BATCH * flops_newton_schulz(m, n)
        executed = NS_BATCH * flops_newton_schulz_executed(m, n)
        rows_out.append({"shape": [m, n], "batch": NS_BATCH, "call_ms": whole_ms, "iteration_ms": iter_ms,
                         "TFLOP/s": flops / iter_ms / 1e9, "frac_of_burst_peak": flops / iter_ms / 1e9 / peaks["bf16_tflops"],
                         "executed_TFLOP/s": executed / iter_ms / 1e9,
                         "executed_frac_of_burst_peak": executed / iter_ms / 1e9 / peaks["bf16_tflops"],
                         "orthogonality_error": err, "error_per_sqrt_m": err / m**0.5})
        del x, packed, scratch, work, y
        torch.cuda.empty_cache()
    launches = _native.launch_count() - launches_before
    clocks = sampler.stop()
    big = rows_out[-1]
    total_flops = sum(NS_BATCH * flops_newton_schulz(m, n) for m, n in NS_SHAPES)
    total_ms = sum(r["iteration_ms"] for r in rows_out)
    line = {
        "metric": "gram_newton_schulz_tflops", "value": total_flops / total_ms / 1e9, "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp16 iteration, fp32 accumulate, bf16 result", "data": "synthetic",
        "config": {"workload": "Gram Newton-Schulz, batches of 16 at 1024x1024, 1024x4096, 4096x14336, 8192x28672",
                   "l2": "operands of the two large shapes exceed L2; medians of per-call CUDA-event times"},
        "roofline": {"kernel": f"gemm2_kernel (products of the {big['shape'][0]}x{big['shape'][1]} batch)",
                     "bound": "tensor", "achieved": big["TFLOP/s"], "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": big["TFLOP/s"] / peaks["bf16_tflops"], "traffic": None,
                     "peak_kind": f"{peaks_kind} bf16 cuBLAS, burst (each batch is timed alone)"},
        "shapes": rows_out, "gpu_launches": launches, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# sustained plain GEMM against cuBLAS (``--config gemm-sustained``)
# ---------------------------------------------------------------------------
def run_gemm_sustained(args) -> None:
    """One 8192^3 bf16 product (A B^T) looped for about four seconds, under the board's power cap:
    torch.matmul (cuBLAS) first, then this library's ``dionw_batched_gemm`` on the same operands,
    with the SM clock and the power sampled every 100 ms.  Says how much of cuBLAS's sustained
    rate the tcgen05 main loop reaches at equal power (the epilogue is 1/128 of the work here)."""
    from dionw_b200 import _native

    if int(os.environ.get("RANK", "0")) != 0:
        return
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    _native.library()
    n = 8192
    gen = torch.Generator(device=device).manual_seed(0)
    a = (torch.randn(1, n, n, device=device, generator=gen) / n**0.5).bfloat16()
    b = torch.randn(1, n, n, device=device, generator=gen).bfloat16()
    out = torch.empty(1, n, n, dtype=torch.bfloat16, device=device)
    arms = {"cublas": lambda: torch.matmul(a[0], b[0].T, out=out[0]),
            "dionw_b200": lambda: _native.batched_gemm(a, b, out, b_is_nk=True)}
    seconds = 4.0
    results = {}
    launches_before = _native.launch_count()
    for name, call in arms.items():
        for _ in range(max(3, args.warmup)):
            call()
        torch.cuda.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        count, t0 = 0, time.time()
        start.record()
        while time.time() - t0 < seconds:
            for _ in range(20):
                call()
            count += 20
            torch.cuda.synchronize()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        results[name] = {"TFLOP/s": 2.0 * n**3 * count / ms / 1e9, "products": count, "seconds": ms / 1e3,
                         "clocks": sampler.stop()}
    ours, theirs = results["dionw_b200"]["TFLOP/s"], results["cublas"]["TFLOP/s"]
    line = {
        "metric": "sustained_gemm_tflops", "value": ours, "unit": "TFLOP/s", "n_gpus": 1, "steps": results["dionw_b200"]["products"],
        "warmup": max(3, args.warmup), "ms_per_step": 1e3 * results["dionw_b200"]["seconds"] / results["dionw_b200"]["products"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16, fp32 accumulate",
        "data": "synthetic", "config": {"workload": "8192^3 bf16 A B^T looped for 4 s", "l2": "operands (268 MB) exceed L2"},
        "roofline": {"kernel": "gemm2_kernel" if os.environ.get("DIONW_GEMM_CTA_PAIRS", "1") != "0" else "gemm_kernel",
                     "bound": "tensor", "achieved": ours, "peak": theirs, "unit": "TFLOP/s", "frac": ours / theirs,
                     "traffic": None, "peak_kind": "torch.matmul (cuBLAS) on the same operands, same call, same power cap"},
        "arms": results, "gpu_launches": _native.launch_count() - launches_before,
    }
    print(json.dumps(line), flush=True)


def run_sub_bench(flags: list[str], timeout: float) -> dict:
    """Another arm of this file in a process of its own (it needs the GPU to itself); its JSON line."""
    try:
        done = subprocess.run([sys.executable, str(ROOT / "bench.py"), *flags], capture_output=True, text=True,
                              timeout=timeout, cwd=str(ROOT))
    except subprocess.TimeoutExpired:
        return {"unavailable": f"bench.py {' '.join(flags)} did not finish within {timeout:.0f} s"}
    for line in reversed(done.stdout.splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except json.JSONDecodeError:
                break
    return {"unavailable": f"bench.py {' '.join(flags)} printed no JSON line (exit code {done.returncode}): "
                           f"{done.stderr[-300:]}"}


# ---------------------------------------------------------------------------
# correctness of the sharded step, checked inside the distributed run (outside the timed region)
# ---------------------------------------------------------------------------
def sharded_parity(device, rank: int, dist) -> dict:
    """Three steps of ``ShardedDion`` on every rank and of single-GPU ``Dion`` on rank 0, on the
    ``tiny`` parameter set (blocks that select rows and blocks that do not, an AdamW table large
    enough to be cut into per-rank ranges) from identical seeds.  Reports whether the replicas
    hold identical weights, how far rank 0's weights are from the single-GPU ones (the design
    is bit-identical: 0.0 expected) and the same for the gathered ``state_dict()``."""
    import dionw_b200 as dionw
    from dionw_b200 import _workspace
    from dionw_b200.distributed import ShardedDion

    def build():
        model = build_model("tiny", device)
        model.init_(seed=7)
        routes = {model.lm_head.weight: dionw.Route(dionw.RouteKind.ADAMW)}
        groups, _ = dionw.param_groups(model, routes=routes)
        return model, groups

    model, groups = build()
    sharded = ShardedDion(groups, lr=LR, weight_decay=WEIGHT_DECAY)
    single_model = single = None
    if rank == 0:
        single_model, single_groups = build()
        single = dionw.Dion(single_groups, lr=LR, weight_decay=WEIGHT_DECAY)
    steps = 3
    for step in range(steps):
        gen = torch.Generator(device=device).manual_seed(100 + step)
        grads = [torch.empty_like(p).normal_(0.0, 1e-3, generator=gen) for p in model.parameters()]
        for p, g in zip(model.parameters(), grads):
            p.grad = g
        sharded.step()
        if single is not None:
            for p, g in zip(single_model.parameters(), grads):
                p.grad = g.clone()
            single.step()
    torch.cuda.synchronize()
    spread = torch.zeros((), device=device)
    for p in model.parameters():
        reference = p.detach().clone()
        dist.broadcast(reference, src=0)
        spread = torch.maximum(spread, (p.detach() - reference).abs().max())
    dist.all_reduce(spread, op=dist.ReduceOp.MAX)
    gathered = sharded.state_dict()   # a collective call: every rank makes it
    result = {"workload": "tiny parameter set (2 layers, d = 1024), 3 steps, identical seeds", "steps": steps,
              "replicas_identical": bool(float(spread) == 0.0), "replicas_max_abs": float(spread)}
    if single is not None:
        worst = max(float((a.detach() - b.detach()).abs().max())
                    for a, b in zip(model.parameters(), single_model.parameters()))
        want = single.state_dict()
        state_worst, compared = 0.0, 0
        for index, entry in want["state"].items():
            for key, value in entry.items():
                if isinstance(value, torch.Tensor):
                    got = gathered["state"][index][key]
                    state_worst = max(state_worst, float((got.float() - value.float()).abs().max()))
                    compared += 1
        result.update({"vs_single_gpu_max_abs": worst, "state_dict_vs_single_gpu_max_abs": state_worst,
                       "state_tensors_compared": compared})
    del sharded, single, model, single_model, gathered
    _workspace.release()
    torch.cuda.empty_cache()
    return result


# ---------------------------------------------------------------------------
# the GPU arm
# ---------------------------------------------------------------------------
def run_gpu_arm(args) -> None:
    import dionw_b200 as dionw
    from dionw_b200 import _matrix_step, _native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    distributed = world > 1 or args.sharded
    if distributed:
        import torch.distributed as dist

        if world == 1:   # --sharded on one GPU: the sharded step's machinery with a group of one
            for key, value in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29533"), ("RANK", "0"),
                               ("WORLD_SIZE", "1")):
                os.environ.setdefault(key, value)
        options = None
        if args.nccl_high_priority:   # NCCL's kernels on a high-priority stream (an experiment switch)
            options = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=device, pg_options=options)
    _native.library()
    # The reference's own GPU step on the same workload (its Triton + cuBLAS path), measured first, in a
    # process of its own, while this one holds no device memory: the denominator of "times faster than
    # the reference's step on one B200".
    reference_gpu = None
    if world == 1 and not args.sharded and not args.no_reference_gpu and not args.graph_replay and args.ema == "config":
        reference_gpu = run_sub_bench(["--impl", "reference-gpu", "--config", args.config, "--steps",
                                       str(min(10, args.steps)), "--warmup", "3"], timeout=300)
        reference_gpu = {k: reference_gpu.get(k) for k in ("value", "median_ms", "unit", "steps", "warmup", "clocks",
                                                           "config", "unavailable") if k in reference_gpu}
    parity = sharded_parity(device, rank, dist) if distributed and not args.no_parity else None

    layers, d, dkv, dff, vocab = CONFIGS[args.config]
    weights_bytes = 4.0 * (layers * (2 * d * d + 2 * d * dkv + 3 * d * dff)
                           + vocab * d * (1 if args.config in EMBED_ONLY_WITH_EMA else 2))
    # replicated weights + this rank's share of momentum (+ EMA shadows) + scratch must fit beside the gradients
    need = weights_bytes * (1.0 + (1.0 + (1.0 if args.config in EMBED_ONLY_WITH_EMA else 0.0)) / world) + 16e9
    have = torch.cuda.get_device_properties(device).total_memory
    if need > have:
        raise SystemExit(f"bench.py: config {args.config} needs about {need / 1e9:.0f} GB per GPU on {world} GPU(s), "
                         f"this GPU has {have / 1e9:.0f} GB: run it on more GPUs")
    model = build_model(args.config, device)
    model.init_(seed=0)
    routes = {} if model.lm_head is None else {model.lm_head.weight: dionw.Route(dionw.RouteKind.ADAMW)}
    groups, _ = dionw.param_groups(model, routes=routes)
    ema_kind = args.ema if args.ema != "config" else ("gpu" if args.config in EMBED_ONLY_WITH_EMA else "none")
    ema = None if ema_kind == "none" else dionw.EMAConfig(
        decay=0.9999, device=dionw.EMADevice.GPU if ema_kind == "gpu" else dionw.EMADevice.CPU)
    if distributed:
        from dionw_b200.distributed import ShardedDion

        optimizer = ShardedDion(groups, lr=LR, weight_decay=WEIGHT_DECAY, ema=ema, fused_decay=args.fused_decay)
        if args.no_overlap:
            optimizer.overlap_apply = False
        if args.overlap_apply:
            optimizer.overlap_apply = True
        if args.round_elements:
            optimizer.round_elements = args.round_elements
        if args.adamw_first:
            optimizer.adamw_first = True
        if args.adamw_late:
            optimizer.adamw_first = False
        if args.costliest_first:
            optimizer.costliest_second = False
        if args.static_tiles:
            _native.gemm_dynamic_tiles(False)
        if args.decay_rows_per_wait >= 0:
            optimizer.decay_rows_per_wait = args.decay_rows_per_wait
        if args.adamw_delay_rounds >= 0:
            optimizer.adamw_delay_rounds = args.adamw_delay_rounds
        if args.apply_warps:
            optimizer.apply_warps = args.apply_warps
    else:
        optimizer = dionw.Dion(groups, lr=LR, weight_decay=WEIGHT_DECAY, ema=ema)
    if args.no_overlap:
        optimizer.overlap_streams = False
    if args.max_run_elements:
        import dionw_b200.optimizer as optimizer_module_for_runs

        optimizer_module_for_runs.MAX_RUN_ELEMENTS = args.max_run_elements
    gen = torch.Generator(device=device).manual_seed(1)
    param_bytes = sum(p.numel() * 4 for p in model.parameters())
    shared_grads = 2 * param_bytes > SHARED_GRADS_ABOVE
    by_shape: dict[tuple, torch.Tensor] = {}
    for p in model.parameters():
        if shared_grads:
            if tuple(p.shape) not in by_shape:
                by_shape[tuple(p.shape)] = torch.empty_like(p).normal_(0.0, 1e-3, generator=gen)
            p.grad = by_shape[tuple(p.shape)]
        else:
            p.grad = torch.empty_like(p).normal_(0.0, 1e-3, generator=gen)
    work = census(groups)

    def barrier() -> None:
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    timer = StageTimer()
    replay = bool(args.graph_replay) and not distributed
    if replay:
        optimizer.graph_replay = True   # the stage hook is installed only while stages are timed
    else:
        _matrix_step.STAGE_HOOK = timer
    if ema_kind == "cpu":
        # the snapshot kernel runs on the tracker's copy stream: the events land there
        real_stage = _native.ema_stage_pack

        def timed_stage(sources, offsets, staging):
            with timer("ema_stage"):
                real_stage(sources, offsets, staging)

        _native.ema_stage_pack = timed_stage
    if optimizer.ema is not None:
        real_flush = optimizer.ema._flush_gpu

        def timed_flush():
            with timer("ema"):
                real_flush()

        optimizer.ema._flush_gpu = timed_flush

    # nvidia-smi needs about a second to deliver its first sample: it is started before the warm-up
    # steps (the same workload) and, after the timed region, the same steps go on untimed until ten
    # samples exist, so short timed regions (27 ms steps on 8 GPUs) still get their clock record.
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        optimizer.step()
    barrier()

    # ---- timed region: exactly K steps, device time, max over ranks.  Then, right after it (the GPU
    # is still in the same power and clock state), K more steps with every stage of every run bracketed
    # by CUDA events on the launching stream: the per-stage figures describe the steady state the
    # headline was measured in, and the event records stay out of the headline.  A replayed step
    # cannot carry events: its stages are timed below, in steps run as launches.
    launches_before = _native.launch_count()
    replays_before = optimizer.graph_replays if replay else 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        optimizer.step()
    end.record()
    barrier()
    total_ms = start.elapsed_time(end)
    launches = _native.launch_count() - launches_before
    if replay:   # a replayed step executes the kernels of its recording without passing the library's counter
        launches += (optimizer.graph_replays - replays_before) * optimizer.graph_kernels
    stages: dict[str, float] = {}
    ns_by_shape: list[dict] = []
    whole_ms = None
    if not replay:
        timer.enabled = True
        for _ in range(args.steps):
            with timer("whole_step"):
                optimizer.step()
        timer.enabled = False
        barrier()
        stages = {k: v / args.steps for k, v in timer.collect().items()}
        whole_ms = stages.pop("whole_step", None)   # the same steps, bracketed once: shows what lies between the stages
        ns_by_shape = split_ns_shapes(stages, timer.blocks, args.steps)
    extra_deadline = time.time() + 4.0
    while True:
        need = rank == 0 and sampler.samples() < 10 and time.time() < extra_deadline
        if distributed:   # every rank takes the same number of extra steps: rank 0 decides
            flag = torch.tensor([1.0 if need else 0.0], device=device)
            dist.broadcast(flag, src=0)
            need = bool(flag.item() > 0.0)
        if not need:
            break
        optimizer.step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    if distributed:
        t = torch.tensor([total_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t)
    ms_per_step = total_ms / args.steps

    # ---- per-stage device time of a replayed step: separate steps, run as launches with the hook installed
    if replay:
        timer.enabled = True
        _matrix_step.STAGE_HOOK = timer
        stage_steps = max(1, min(3, args.steps))
        for _ in range(stage_steps):
            with timer("whole_step"):
                optimizer.step()
        stages = {k: v / stage_steps for k, v in timer.collect().items()}
        timer.enabled = False
        _matrix_step.STAGE_HOOK = None
        whole_ms = stages.pop("whole_step", None)
        ns_by_shape = split_ns_shapes(stages, timer.blocks, stage_steps)

    # ---- host dispatch: wall time for step() to return with the GPU idle at the start and
    # no synchronize inside (one step's launches fit the driver's launch queue)
    host_times = []
    for _ in range(3):
        barrier()
        t0 = time.perf_counter()
        optimizer.step()
        host_times.append((time.perf_counter() - t0) * 1e3)
    barrier()
    host_ms = statistics.median(host_times)

    # ---- end to end: gradients come from pinned host memory, one scalar goes back
    pool: dict[tuple, torch.Tensor] = {}
    for p in model.parameters():
        key = tuple(p.shape)
        if key not in pool:
            pool[key] = torch.empty(p.shape, dtype=torch.float32, pin_memory=True).normal_(0.0, 1e-3)
    result_host = torch.empty((), dtype=torch.float32, pin_memory=True)
    h2d_bytes = sum(p.numel() * 4 for p in model.parameters())
    e2e_steps = max(1, min(3, args.steps))

    def e2e_step() -> None:
        for p in model.parameters():
            p.grad.copy_(pool[tuple(p.shape)], non_blocking=True)
        optimizer.step()
        result_host.copy_(model.norm.sum(), non_blocking=True)

    e2e_step()
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2.record()
    barrier()
    e2e_ms = s2.elapsed_time(e2) / e2e_steps
    if distributed:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t)

    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return

    peaks, peaks_kind = measured_peaks()
    share = 1.0 / world  # matrix blocks and the AdamW space are sharded evenly by cost
    ns_ms = stages.get("newton_schulz", 0.0)
    ns_tflops = work["ns_flops"] * share / ns_ms / 1e9 if ns_ms else None
    ns_exec_tflops = work["ns_flops_executed"] * share / ns_ms / 1e9 if ns_ms else None
    peak_tf = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])

    def gbs(key: str, stage: str, scale: float = 1.0) -> float | None:
        ms = stages.get(stage, 0.0)
        return work[key] * scale / ms / 1e6 if ms else None

    stage_report = {
        "accumulate": {"ms": stages.get("accumulate"), "GB/s": gbs("bytes_accumulate", "accumulate", share)},
        "select": {"ms": stages.get("select")},
        "pack": {"ms": stages.get("pack"), "GB/s": gbs("bytes_pack", "pack", share)},
        "newton_schulz": {"ms": ns_ms, "TFLOP/s": ns_tflops, "by_operand": ns_by_shape},
        "finish": {"ms": stages.get("finish")},   # per-row scalars only: the row sums come from the last product
        "apply": {"ms": stages.get("apply"), "GB/s": gbs("bytes_apply", "apply")},
        "adamw": {"ms": stages.get("adamw"), "GB/s": gbs("bytes_adamw", "adamw", share if distributed else 1.0)},
        "gather_wait": {"ms": stages.get("gather_wait")},   # the stream blocked on an all-gather that has not landed yet
        "hbm_peak_GB/s": peaks["hbm_gbs"],
        "between_stages_ms": (whole_ms - sum(v for v in stages.values())) if whole_ms is not None else None,
    }
    if "ema" in stages:
        stage_report["ema"] = {"ms": stages["ema"], "GB/s": gbs("bytes_ema", "ema", share)}
    for entry in stage_report.values():   # each HBM-bound stage against the measured copy bandwidth
        if isinstance(entry, dict) and entry.get("GB/s"):
            entry["frac_of_hbm_peak"] = entry["GB/s"] / peaks["hbm_gbs"]
    if "ema_stage" in stages:
        # fp32 snapshot of every parameter written by one kernel into pinned host memory: bound by
        # the host link (PCIe), not HBM; the worker thread's lerp on the host follows it
        snapshot = 4.0 * (work["matrix_elements"] + work["adamw_elements"]) * share
        stage_report["ema_stage"] = {"ms": stages["ema_stage"], "GB/s": snapshot / stages["ema_stage"] / 1e6,
                                     "bound": "host link (device-to-host writes)", "bytes": snapshot}
    cpu = cpu_sample_step(args.config, 3, 1) if world == 1 and not args.no_cpu_baseline else None
    # The Newton-Schulz microbenchmark (batches of 16 at the four shapes), after this arm's own numbers
    # are taken and its memory is given back.
    gram_ns = None
    if reference_gpu is not None and args.config == "llama3-8b":
        from dionw_b200 import _workspace

        # give the device memory back whoever still refers to the tensors: storages are replaced
        for p in model.parameters():
            p.grad = None
            p.data = torch.empty(0, device=device)
        optimizer.state.clear()
        optimizer._buckets = None
        by_shape.clear()
        pool.clear()
        _workspace.release()
        torch.cuda.empty_cache()
        sub = run_sub_bench(["--config", "gram-ns", "--steps", "3", "--warmup", "3"], timeout=240)
        gram_ns = sub if "unavailable" in sub else {
            "shapes": [{k: row[k] for k in ("shape", "batch", "iteration_ms", "call_ms", "TFLOP/s", "executed_TFLOP/s",
                                            "frac_of_burst_peak", "executed_frac_of_burst_peak", "orthogonality_error")
                        if k in row} for row in sub.get("shapes", [])],
            "clocks": sub.get("clocks"), "steps": sub.get("steps"), "warmup": sub.get("warmup")}
        # the reference's own Gram Newton-Schulz entry on the same batches (whole call; its Triton + cuBLAS products)
        theirs = run_sub_bench(["--impl", "reference-gpu", "--config", "gram-ns", "--steps", "3", "--warmup", "3"],
                               timeout=240)
        gram_ns["reference"] = theirs if "unavailable" in theirs else [
            {k: row[k] for k in ("shape", "call_ms", "TFLOP/s_of_call", "orthogonality_error") if k in row}
            for row in theirs.get("shapes", [])]
    line = {
        "metric": "optimizer_step_ms", "value": ms_per_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp32 state, fp16 Newton-Schulz (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{args.config}-shaped parameter set, fp32 masters, Dion3 fraction 0.25 + AdamW",
                   "lr": LR, "weight_decay": WEIGHT_DECAY, "l2": "working set >> L2 (126 MB), no flush needed",
                   "parallelism": f"blocks sharded by Newton-Schulz cost over {world} GPU(s)",
                   "sharded_step": ({"overlap_apply": bool(optimizer.overlap_apply),
                                     "apply_warps": int(optimizer.apply_warps),
                                     "round_elements": int(optimizer.round_elements),
                                     "adamw_first": bool(optimizer.adamw_first),
                                     "adamw_delay_rounds": int(optimizer.adamw_delay_rounds),
                                     "costliest_second": bool(optimizer.costliest_second),
                                     "dynamic_tiles": _native.gemm_dynamic_tiles(),
                                     "fused_decay": bool(optimizer.fused_decay),
                                     "decay_rows_per_wait": int(optimizer.decay_rows_per_wait)} if distributed else None),
                   "ema": (None if ema is None else
                           f"{ema_kind.upper()} shadows, decay 0.9999, every step"
                           + (" (pinned host shadows, one snapshot kernel + host worker thread per step; the "
                              "step waits for the previous update)" if ema_kind == "cpu" else "")),
                   "graph_replay": ({"recordings": optimizer._graph_recordings, "kernels_per_replay": optimizer.graph_kernels}
                                    if replay else None),
                   "gradients": ("one tensor per shape shared by all layers (weights + gradients would not fit "
                                 "beside the state)" if shared_grads else "one tensor per parameter")},
        "roofline": {
            "kernel": "gemm2_kernel (all Newton-Schulz products of a step)",
            "bound": "tensor", "achieved": ns_exec_tflops, "peak": peak_tf, "unit": "TFLOP/s",
            "frac": ns_exec_tflops / peak_tf if ns_exec_tflops else None, "traffic": work["ns_traffic"] * share,
            "achieved_kind": ("FLOPs the kernels execute, 2(3m^2n + 7m^3) per m x n operand (the products Q Z, G Z and "
                              "Z RZ run on the lower-triangle schedule), / the summed CUDA-event time of the stage"),
            "traffic_kind": ("DRAM bytes of all gemm2_kernel launches of one step on this rank: the operand census "
                             "of the products, calibrated x1.06 on an ncu capture of the 18 products of four "
                             "3584x4096 blocks and scaled by blocks (traffic grows with the blocks processed)"),
            "peak_kind": f"{peaks_kind} bf16 cuBLAS, sustained (the kernel is timed inside the step)",
            "flops_per_step": work["ns_flops_executed"] * share,
            "algorithmic": {"TFLOP/s": ns_tflops, "flops_per_step": work["ns_flops"] * share,
                            "note": "the reference's product census 2(3m^2n + 11.5m^3) per operand / the same time: "
                                    "an effective rate, not comparable with a hardware peak"},
        },
        "stages": stage_report,
        "reference_gpu": reference_gpu,
        "gram_ns": gram_ns,
        "parity": parity,
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4,
                "steps": e2e_steps},
        "gpu_launches": launches,
        "host_dispatch_ms": host_ms,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("b200", "reference", "reference-gpu"), default="b200")
    parser.add_argument("--config", choices=sorted(CONFIGS) + ["gram-ns", "gemm-sustained"], default="llama3-8b")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-reference-gpu", action="store_true",
                        help="one GPU: do not time the reference's own GPU step and the Newton-Schulz microbenchmark "
                             "in processes of their own before and after this arm")
    parser.add_argument("--no-overlap", action="store_true", help="one-stream step (for comparison)")
    parser.add_argument("--nccl-high-priority", action="store_true",
                        help="create the process group with NCCL's kernels on a high-priority stream")
    parser.add_argument("--adamw-delay-rounds", type=int, default=-1,
                        help="sharded step: rounds between the costliest bucket's last round and AdamW (default 1)")
    parser.add_argument("--adamw-late", action="store_true",
                        help="sharded step: AdamW and its all-gathers after the costliest bucket's rounds (for comparison)")
    parser.add_argument("--adamw-first", action="store_true",
                        help="sharded step: AdamW and its all-gathers before the first round (for comparison)")
    parser.add_argument("--ema", choices=("config", "none", "gpu", "cpu"), default="config",
                        help="EMA of every parameter: 'config' = GPU shadows for the 70B-shaped configs, none otherwise")
    parser.add_argument("--graph-replay", action="store_true",
                        help="single GPU: replay the step from a CUDA graph (Dion.graph_replay); gpu_launches then "
                             "counts only the steps that ran as launches")
    parser.add_argument("--round-elements", type=int, default=0, help="sharded step: update elements per round")
    parser.add_argument("--max-run-elements", type=int, default=0,
                        help="update elements one run orthogonalizes at once (default: the reference's 2^28)")
    parser.add_argument("--fused-decay", action="store_true",
                        help="sharded step: the tensor-core products' waiting epilogue warps decay the unselected rows")
    parser.add_argument("--decay-rows-per-wait", type=int, default=-1,
                        help="sharded step: rows of the decay job an epilogue warp may take per tile it waits for")
    parser.add_argument("--static-tiles", action="store_true",
                        help="sharded step: tensor-core products take their tiles in a fixed stride (for comparison)")
    parser.add_argument("--costliest-first", action="store_true",
                        help="sharded step: the costliest bucket's rounds first (for comparison; default: second)")
    parser.add_argument("--sharded", action="store_true",
                        help="one GPU: step with ShardedDion in a process group of one (its rounds, streams and "
                             "single-launch weight update) instead of Dion")
    parser.add_argument("--no-parity", action="store_true", help="sharded step: skip the correctness check before the run")
    parser.add_argument("--apply-warps", type=int, default=0, help="sharded step with --overlap-apply: warps per CTA of the weight update")
    parser.add_argument("--overlap-apply", action="store_true",
                        help="sharded step: weight update of a round on a side stream beside the next round")
    args = parser.parse_args()
    if args.config in ("gram-ns", "gemm-sustained"):
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": f"the {args.config} microbenchmark has no CPU arm"}))
        elif args.impl == "reference-gpu" and args.config == "gram-ns":
            run_reference_gpu_ns(args)
        elif args.config == "gram-ns":
            run_ns_microbench(args)
        else:
            run_gemm_sustained(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
