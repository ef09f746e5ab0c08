"""``Dion``: row-selected NorMuon on matrices, AdamW on the rest, one learning rate.

The API, validation, messages, ``state_dict`` layout and resume checks are those
of the reference's ``dionw.Dion`` (src/dionw/optimizer.py:81-424); the step runs
on this package's sm_100a kernels through the C ABI of ``include/dionw_b200.h``.

Per matrix block and step: ``M += G``; keep the top ``k = ceil(fraction * rows)``
rows of ``M`` by l1 norm and decay them by ``momentum`` (error feedback); run
five Newton-Schulz steps on the kept rows; NorMuon divides each row by the root
of an EMA of its mean square and restores the block's Frobenius norm;
``W[rows] -= lr * 0.2 * sqrt(max(rows, cols)) * sqrt(min(rows, cols) / min(k, cols)) * O``;
weight decay is decoupled and touches every row.  Parameters must be float32 on
a CUDA device.
"""

from __future__ import annotations

import warnings
from collections.abc import Callable, Iterable
from typing import Any

import torch
from torch import Tensor
from torch.optim import Optimizer

from dionw_b200 import _matrix_step
from dionw_b200._adamw import adamw_step, init_adamw_state
from dionw_b200._buckets import Bucket, block_shape, build_buckets
from dionw_b200._keys import (
    ADAMW_STEP_STATE, EXP_AVG_SQ_STATE, EXP_AVG_STATE, FRACTION_KEY, MOMENTUM_FORM_KEY, MOMENTUM_KEY, MUON_BETA2_KEY, NEWTON_SCHULZ_KEY,
    NUM_HEADS_KEY, ROUTE_KEY, ROW_NORMALIZATION_KEY, STRUCTURAL_KEYS,
)
from dionw_b200._matrix_step import (
    MAX_RUN_ELEMENTS, apply_result, open_run, run_core, run_elements, run_front, step_run, step_size,
)
from dionw_b200.ema import EMAConfig, IntegratedEMAOptimizer, ProfileRegion, no_profile
from dionw_b200.matrix_update import DION3_UPDATE, MatrixUpdate, MomentumForm, RowNormalization
from dionw_b200.newton_schulz import NewtonSchulz
from dionw_b200.routing import RouteKind

__all__ = ["MAX_RUN_ELEMENTS", "NEWTON_SCHULZ_KEY", "Dion", "step_run"]

# ``step_run`` is a module attribute so that it can be replaced; the overlapped step only
# takes over while it is still this function.
_sequential_step_run = step_run


def _require_param(param: Tensor) -> None:
    """float32 on CUDA, or raise (ValueError off CUDA, TypeError for another dtype)."""
    if not param.is_cuda:
        raise ValueError(f"Dion runs on CUDA devices, got a parameter on {param.device}")
    if param.dtype != torch.float32:
        raise TypeError(
            f"Dion needs float32 parameters, got {param.dtype}: keep float32 master weights and run the "
            "forward and backward in bfloat16 (autocast)")


def _require_group(group: dict[str, Any]) -> None:
    """Validate a fully-defaulted group.

    Raises:
        TypeError: Without a route (the group was not built by ``param_groups``).
        ValueError: On unknown enum values, negative lr / weight decay, a bad
            fraction, Nesterov with row selection, a vector in a matrix group, or
            a head split that does not divide the rows.
    """
    if ROUTE_KEY not in group:
        raise TypeError(
            "Dion param groups need a route: build them with dionw.param_groups(model) instead of "
            "passing parameters directly")
    NewtonSchulz(group[NEWTON_SCHULZ_KEY])
    RowNormalization(group[ROW_NORMALIZATION_KEY])
    form = MomentumForm(group[MOMENTUM_FORM_KEY])
    if float(group["lr"]) < 0.0 or float(group["weight_decay"]) < 0.0:
        raise ValueError("a group's lr and weight_decay must be >= 0")
    kind = RouteKind(group[ROUTE_KEY])
    if kind is RouteKind.ADAMW:
        return
    if kind is not RouteKind.MATRIX:
        raise RuntimeError(f"Unhandled RouteKind: {kind}")
    fraction = float(group[FRACTION_KEY])
    if not 0.0 < fraction <= 1.0:
        raise ValueError(f"fraction must be in (0, 1], got {fraction}")
    if form is MomentumForm.NESTEROV and fraction < 1.0:
        raise ValueError(
            f"Nesterov momentum needs every row per step, got fraction {fraction}: build the groups with "
            "fraction=1.0 or use MomentumForm.HEAVY_BALL")
    for param in group["params"]:
        if param.ndim < 2:
            raise ValueError(f"a matrix group holds a {param.ndim}-D parameter; route it to AdamW")
        block_shape(param, group[NUM_HEADS_KEY])


def _fill_legacy_keys(saved: list[dict[str, Any]]) -> list[dict[str, Any]]:
    """Groups saved before the row-normalization / momentum-form options meant NorMuon + heavy ball."""
    legacy = {
        ROW_NORMALIZATION_KEY: RowNormalization.NORMUON.value,
        MOMENTUM_FORM_KEY: MomentumForm.HEAVY_BALL.value,
    }
    return [{**legacy, **group} if ROUTE_KEY in group else group for group in saved]


def _require_same_structure(saved: list[dict[str, Any]], current: list[dict[str, Any]]) -> None:
    """torch's loader restores every group setting from the checkpoint; a changed route,
    fraction, head split, iteration, normalization or momentum form must be refused instead.

    Raises:
        ValueError: On a different group count, a missing key, or a mismatch.
    """
    if len(saved) != len(current):
        raise ValueError(f"Dion state has {len(saved)} param groups, the optimizer {len(current)}")
    for index, (old, new) in enumerate(zip(saved, current)):
        for key in STRUCTURAL_KEYS:
            if key not in old:
                raise ValueError(f"Dion state group {index} has no {key!r}: it was not saved by dionw.Dion")
            if old[key] != new[key]:
                raise ValueError(
                    f"Dion state group {index} {key!r}: checkpoint={old[key]!r}, optimizer={new[key]!r}. "
                    "Build the groups as the checkpoint was built to resume it.")


def step_scalar_values(groups: list[dict[str, Any]], owners: list[Any]) -> tuple[list[float], int]:
    """The step's scalars in table order, and the index of the first per-bucket slot.

    Four slots per group -- lr, weight decay, ``1 - lr * weight_decay`` (computed in Python doubles and
    rounded once when the table is written, as src/dionw/_matrix_step.py:280 computes it), one unused --
    then one slot per owner: ``-step_size`` for a ``Bucket`` (src/dionw/_matrix_step.py:115, :147-159),
    0 for anything else (a sharded optimizer lists buckets owned elsewhere, which need only their
    group's decay factor)."""
    values: list[float] = []
    for group in groups:
        lr, weight_decay = float(group["lr"]), float(group["weight_decay"])
        values += [lr, weight_decay, 1.0 - lr * weight_decay, 0.0]
    base = len(values)
    for owner in owners:
        values.append(-step_size(owner, float(groups[owner.group_index]["lr"])) if isinstance(owner, Bucket) else 0.0)
    return values, base


class _DionCore(Optimizer):
    """The matrix and AdamW updates over routed param groups (no EMA)."""

    def __init__(self, params: Iterable[dict[str, Any]], *, lr: float, momentum: float, muon_beta2: float,
                 betas: tuple[float, float], weight_decay: float, eps: float,
                 matrix_update: MatrixUpdate) -> None:
        if lr < 0.0 or weight_decay < 0.0 or eps <= 0.0:
            raise ValueError("lr and weight_decay must be >= 0 and eps > 0")
        for name, value in ((MOMENTUM_KEY, momentum), (MUON_BETA2_KEY, muon_beta2),
                            ("beta1", betas[0]), ("beta2", betas[1])):
            if not 0.0 <= value < 1.0:
                raise ValueError(f"{name} must be in [0, 1), got {value}")
        defaults = {
            "lr": lr,
            MOMENTUM_KEY: momentum,
            MUON_BETA2_KEY: muon_beta2,
            "betas": betas,
            "weight_decay": weight_decay,
            "eps": eps,
            FRACTION_KEY: 1.0,
            NUM_HEADS_KEY: None,
            NEWTON_SCHULZ_KEY: matrix_update.newton_schulz.value,
            ROW_NORMALIZATION_KEY: matrix_update.row_normalization.value,
            MOMENTUM_FORM_KEY: matrix_update.momentum_form.value,
        }
        self._buckets: list[Bucket] | None = None
        self._side_streams: dict[torch.device, torch.cuda.Stream] = {}
        self._graph: tuple[tuple[Any, ...], torch.cuda.CUDAGraph] | None = None
        self._graph_warm: tuple[Any, ...] | None = None
        self._graph_recordings = 0
        self._scalar_tables: dict[torch.device, Tensor] = {}
        self._scalar_layout: tuple[Any, ...] | None = None
        self._scalar_values: list[float] | None = None
        self.graph_kernels = 0   # kernel launches held by the current recording
        self.graph_replays = 0   # steps executed by replaying a recording
        super().__init__(params, defaults)

    def add_param_group(self, param_group: dict[str, Any]) -> None:
        """Validate and add a group; matrix state is repacked on the next step.

        Raises:
            TypeError: Without a route, for unordered params (a set), or a non-float32 parameter.
            ValueError: On an invalid route, iteration or fraction, or a parameter off CUDA.
        """
        members = param_group["params"]
        if isinstance(members, set):
            raise TypeError("Dion param group params must be ordered, not a set")
        group = {**param_group, "params": [members] if isinstance(members, Tensor) else list(members)}
        for param in group["params"]:
            _require_param(param)
        _require_group({**self.defaults, **group})
        super().add_param_group(group)
        self._buckets = None
        self._graph = self._graph_warm = None
        # AdamW state exists from the start so that an integrated EMA tracks every
        # parameter, also one that never gets a gradient; matrix state appears with
        # the buckets at the first step.
        if RouteKind(group[ROUTE_KEY]) is RouteKind.ADAMW:
            for param in group["params"]:
                self._new_adamw_state(param)

    def _new_adamw_state(self, param: Tensor) -> None:
        """Fresh AdamW moments and step counter for ``param`` (a sharded optimizer keeps less)."""
        init_adamw_state(param, self.state[param])

    def initialize_state(self, param: Tensor) -> None:
        """Create a parameter's fresh state before its first step, without updating it.

        Raises:
            ValueError: If ``param`` is not in the optimizer.
        """
        owner = None
        for group in self.param_groups:
            if any(p is param for p in group["params"]):
                owner = group
                break
        if owner is None:
            raise ValueError("parameter is not in the optimizer")
        kind = RouteKind(owner[ROUTE_KEY])
        if kind is RouteKind.MATRIX:
            self._ensure_buckets()
        elif kind is RouteKind.ADAMW:
            if EXP_AVG_STATE not in self.state[param]:
                self._new_adamw_state(param)
        else:
            raise RuntimeError(f"Unhandled RouteKind: {kind}")

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        """Load a checkpoint; matrix state is repacked into buckets on the next step.

        Raises:
            ValueError: If the saved groups differ from the optimizer's in count or
                in any structural key.
        """
        saved = _fill_legacy_keys(state_dict["param_groups"])
        _require_same_structure(saved, self.param_groups)
        super().load_state_dict({**state_dict, "param_groups": saved})
        self._buckets = None
        self._graph = self._graph_warm = None

    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:
        """Update every parameter that has a gradient; returns the closure's loss, if any."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        runs = [(bucket, run) for bucket in self._ensure_buckets() for run in self._runs_of(bucket)]
        devices = {bucket.momentum.device for bucket, _ in runs}
        self._refresh_scalars()
        if self.graph_replay and self._graph_eligible(runs):
            self._step_replayed(runs)
        elif self.overlap_streams and len(runs) > 1 and len(devices) == 1 and step_run is _sequential_step_run:
            self._step_overlapped(runs, devices.pop())
        else:
            self._step_in_sequence(runs)
        return loss

    def _step_in_sequence(self, runs: list[tuple[Bucket, list[int]]]) -> None:
        for bucket, run in runs:
            # the library looks up per-device facts (SM count, status word) for the current device
            with torch.cuda.device(bucket.momentum.device):
                step_run(bucket, run, self.param_groups[bucket.group_index], self.state)
        self._step_adamw_groups()

    # The scalars of a step that follow the learning rate -- ``-step_size`` per bucket,
    # ``1 - lr * weight_decay`` per group, AdamW's lr and weight decay -- live in a small fp32 table
    # on each device, as the reference keeps ``-step_size`` in a 0-d device tensor
    # (src/dionw/_buckets.py:57-58, _matrix_step.py:115, _row_normalization.py:48-49): kernels read
    # them from there, so a scheduled learning rate changes no launch and a recorded step stays
    # valid.  Layout: four slots per group (lr, weight decay, decay factor, unused), then one per
    # bucket.  The table is rewritten, by one small launch ordered before the step's kernels,
    # only when a value differs from what was written last.
    def _scalar_slots(self) -> list[Any]:
        """What owns a per-bucket slot, in slot order (a sharded optimizer adds to it)."""
        return list(self._ensure_buckets())

    def _refresh_scalars(self) -> None:
        from dionw_b200 import _native

        owners = self._scalar_slots()
        groups = self.param_groups
        values, base = step_scalar_values(groups, owners)
        layout = (len(groups), sum(len(group["params"]) for group in groups), tuple(id(o) for o in owners))
        if layout != self._scalar_layout:
            devices = sorted({p.device for group in groups for p in group["params"] if p.is_cuda},
                             key=lambda d: d.index or 0)
            self._scalar_tables = {d: torch.zeros(len(values), dtype=torch.float32, device=d) for d in devices}
            self._scalar_layout, self._scalar_values = layout, None
            for slot, owner in enumerate(owners):
                table = self._scalar_tables[owner.params[0].device]
                at = 4 * owner.group_index + 2
                owner.decay_device = table[at:at + 1]
                if isinstance(owner, Bucket):
                    owner.step_device = table[base + slot:base + slot + 1]
        if values != self._scalar_values:
            for device, table in self._scalar_tables.items():
                with torch.cuda.device(device):
                    _native.write_scalars(table, values)
            self._scalar_values = values

    def _adamw_hyper(self, group_index: int, device: torch.device) -> Tensor | None:
        """``{lr, weight_decay}`` of a group in the device table."""
        table = self._scalar_tables.get(device)
        return None if table is None else table[4 * group_index:4 * group_index + 2]

    # Optional replay of the step from a CUDA graph.  The reference measures 7-17 ms of host
    # dispatch per step of its own (README.md:514-516 and bench/host_dispatch.py:28-56 there); here a step
    # is a few hundred launches through ctypes.  With ``graph_replay = True`` the first step of a
    # configuration runs as launches (it creates state, grows the scratch arenas and does the
    # one-time device set-up), the second is recorded on a capture stream and replayed, and every
    # later one is a single ``cudaGraphLaunch``.  A recording holds addresses and host scalars by
    # value, so it is keyed on everything a step reads from the host: which parameters have
    # gradients and where parameters, gradients, state and arenas lie, and each group's lr,
    # weight decay, momentum, betas and eps.  Any change (a learning-rate schedule, gradients
    # reallocated by ``zero_grad(set_to_none=True)``) costs one step as launches and one new
    # recording; after ``GRAPH_RECORDINGS_MAX`` recordings the optimizer stops recording and
    # steps as launches, since a loop that changes every step gains nothing from a graph.
    # Keep gradients in place (``zero_grad(set_to_none=False)``) and change lr rarely to use it.
    # The arithmetic is the same kernels in the same order: results are bit-identical.
    graph_replay = False
    GRAPH_RECORDINGS_MAX = 8

    def _graph_eligible(self, runs: list[tuple[Bucket, list[int]]]) -> bool:
        """Whether this step can be recorded: one CUDA device, the built-in stages, nothing that
        makes the step allocate (packed copies of strided tensors, dtype casts of gradients)."""
        from dionw_b200 import _matrix_step
        from dionw_b200.newton_schulz import NativeOrthogonalizer

        if self.overlap_streams:
            return False
        if step_run is not _sequential_step_run or _matrix_step.STAGE_HOOK is not None:
            return False
        devices = set()
        for group in self.param_groups:
            for param in group["params"]:
                grad = param.grad
                if grad is None:
                    continue
                if not (param.is_contiguous() and grad.is_contiguous() and grad.dtype is torch.float32):
                    return False
                devices.add(param.device)
        return len(devices) == 1 and all(isinstance(b.orthogonalize, NativeOrthogonalizer) for b, _ in runs)

    def _step_signature(self, runs: list[tuple[Bucket, list[int]]]) -> tuple[Any, ...]:
        """Everything a recorded step bakes in (see ``graph_replay``)."""
        from dionw_b200 import _workspace

        parts: list[Any] = [_workspace.generation, torch.cuda.current_device(),
                            tuple(t.data_ptr() for t in self._scalar_tables.values())]
        for group in self.param_groups:
            # lr and the weight decay's value are read from the device table; only whether there is
            # a decay at all selects code
            parts.append((float(group["weight_decay"]) > 0.0, float(group[MOMENTUM_KEY]),
                          float(group[MUON_BETA2_KEY]), tuple(map(float, group["betas"])), float(group["eps"])))
            adamw = RouteKind(group[ROUTE_KEY]) is RouteKind.ADAMW
            for p in group["params"]:
                if p.grad is None:
                    continue
                parts.append((p.data_ptr(), p.grad.data_ptr()))
                if adamw:   # a loaded checkpoint replaces these tensors
                    entry = self.state[p]
                    parts.append(tuple(entry[key].data_ptr() for key in (EXP_AVG_STATE, EXP_AVG_SQ_STATE, ADAMW_STEP_STATE)
                                       if key in entry))
        for bucket, run in runs:
            parts.append((bucket.momentum.data_ptr(), bucket.variance.data_ptr(), tuple(run)))
        return tuple(parts)

    def _step_replayed(self, runs: list[tuple[Bucket, list[int]]]) -> None:
        signature = self._step_signature(runs)
        if self._graph is not None and self._graph[0] == signature:
            self._graph[1].replay()
            self.graph_replays += 1
            return
        self._graph = None
        if self._graph_recordings >= self.GRAPH_RECORDINGS_MAX:
            self._step_in_sequence(runs)
            return
        if self._graph_warm != signature:
            self._step_in_sequence(runs)
            self._graph_warm = self._step_signature(runs)  # the arenas may have grown
            return
        from dionw_b200 import _native

        graph = torch.cuda.CUDAGraph()
        before = _native.launch_count()
        try:
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self._step_in_sequence(runs)
        except Exception as exc:  # noqa: BLE001 - a capture executes nothing: the step can still run as launches
            warnings.warn(f"Dion.graph_replay: recording the step failed ({exc!r}); stepping as launches from now on",
                          RuntimeWarning, stacklevel=3)
            self._graph_recordings = self.GRAPH_RECORDINGS_MAX
            self._step_in_sequence(runs)
            return
        self.graph_kernels = _native.launch_count() - before
        graph.replay()
        self.graph_replays += 1
        self._graph = (signature, graph)
        self._graph_recordings += 1

    def _step_adamw_groups(self) -> None:
        for index, group in enumerate(self.param_groups):
            if RouteKind(group[ROUTE_KEY]) is RouteKind.ADAMW:
                with _matrix_step._stage("adamw"):
                    adamw_step(group, self.state, hyper=lambda device, index=index: self._adamw_hyper(index, device))

    # Optional two-stream step: the tensor-core part of run i (Newton-Schulz, on the
    # caller's stream) overlaps the HBM-bound parts of its neighbours on a side
    # stream: accumulate/select/pack of run i+1, the weight update of run i-1,
    # and AdamW.  Three scratch arenas rotate.  The arithmetic and its order per
    # run are unchanged, so results are bit-identical to the one-stream step.
    # Off by default: on a B200 under its 1 kW power cap the Llama-3-8B-shaped
    # step takes the same 127.7 ms either way (SM clock 1230 MHz overlapped against
    # 1365 MHz in sequence: the step is limited by power, not by idle units).  It
    # pays where the step is not power-capped.
    overlap_streams = False

    def _step_overlapped(self, runs: list[tuple[Bucket, list[int]]], device: torch.device) -> None:
        main = torch.cuda.current_stream(device)
        side = self._side_streams.get(device)
        if side is None:
            side = self._side_streams[device] = torch.cuda.Stream(device=device)
        side.wait_stream(main)
        contexts: list[Any] = [None] * len(runs)
        front_done: list[Any] = [None] * len(runs)

        def front(i: int) -> None:
            bucket, run = runs[i]
            with torch.cuda.stream(side):
                contexts[i] = open_run(bucket, run, self.param_groups[bucket.group_index], arena=f"overlap{i % 3}")
                run_front(contexts[i])
                front_done[i] = torch.cuda.Event()
                front_done[i].record(side)

        with torch.cuda.stream(side):
            self._step_adamw_groups()
        front(0)
        for i in range(len(runs)):
            if i + 1 < len(runs):
                front(i + 1)
            main.wait_event(front_done[i])
            result = run_core(contexts[i])
            core_done = torch.cuda.Event()
            core_done.record(main)
            with torch.cuda.stream(side):
                side.wait_event(core_done)
                apply_result(result, contexts[i].group)
            contexts[i] = None
        main.wait_stream(side)

    def _ensure_buckets(self) -> list[Bucket]:
        if self._buckets is None:
            self._buckets = build_buckets(self.param_groups, self.state)
        return self._buckets

    def _runs_of(self, bucket: Bucket) -> list[list[int]]:
        """The bucket's parameters that have gradients, as runs of consecutive positions.

        A run ends at a parameter without a gradient or when it would exceed
        ``MAX_RUN_ELEMENTS`` update elements (a larger parameter runs alone).
        """
        runs: list[list[int]] = []
        pending: list[int] = []
        elements = 0
        for position, param in enumerate(bucket.params):
            size = run_elements(bucket, position)
            if pending and (param.grad is None or elements + size > MAX_RUN_ELEMENTS):
                runs.append(pending)
                pending, elements = [], 0
            if param.grad is not None:
                pending.append(position)
                elements += size
        if pending:
            runs.append(pending)
        return runs

    def _step_bucket(self, bucket: Bucket) -> None:
        """Step one bucket, run after run, on the current stream."""
        group = self.param_groups[bucket.group_index]
        for run in self._runs_of(bucket):
            step_run(bucket, run, group, self.state)


class Dion(IntegratedEMAOptimizer, _DionCore):
    """Dion on matrices, AdamW on the rest, with an optional integrated EMA.

    Build the groups with ``param_groups(model)``.  ``lr`` is an AdamW-equivalent
    learning rate for every parameter.

    Args:
        params: Groups from ``param_groups``.
        lr: Learning rate.
        momentum: Matrix momentum (error-feedback decay of selected rows).
        muon_beta2: EMA decay of each row's squared update (NorMuon).
        betas: AdamW betas of AdamW-routed parameters.
        weight_decay: Decoupled weight decay of groups without their own.
        eps: AdamW epsilon.
        matrix_update: ``DION3_UPDATE`` (default) or ``MUON_UPDATE``.
        ema: EMA schedule and placement, or None.
        profile_region: Named profiling region entered around EMA work.

    Raises:
        TypeError: For groups without a route or non-float32 parameters.
        ValueError: On out-of-range hyperparameters, Nesterov momentum with row
            selection, or parameters off CUDA.
    """

    def __init__(self, params: Iterable[dict[str, Any]], *, lr: float, momentum: float = 0.95,
                 muon_beta2: float = 0.95, betas: tuple[float, float] = (0.9, 0.95),
                 weight_decay: float = 0.0, eps: float = 1e-8, matrix_update: MatrixUpdate = DION3_UPDATE,
                 ema: EMAConfig | None = None, profile_region: ProfileRegion = no_profile) -> None:
        super().__init__(params, lr=lr, momentum=momentum, muon_beta2=muon_beta2, betas=betas,
                         weight_decay=weight_decay, eps=eps, matrix_update=matrix_update)
        self._init_integrated_ema(ema, profile_region)
