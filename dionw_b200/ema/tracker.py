"""``OptimizerIntegratedEMA``: shadows kept in ``optimizer.state[p]``, on the GPU or the CPU.

Schedule and bookkeeping follow src/dionw/ema/tracker.py:39-299.  The work itself
differs: GPU shadows update in one multi-tensor launch per step; CPU shadows are
fed by ONE kernel that writes every parameter's fp32 snapshot straight into a
pinned host buffer on a side stream (no per-parameter copies), and the update
runs on a native worker thread.  The next optimizer step waits for the snapshot
on the device (a stream dependency), not on the host.
"""

from __future__ import annotations

import os
from collections.abc import Callable
from typing import TYPE_CHECKING, Any

import torch
from torch import Tensor

from dionw_b200 import _native
from dionw_b200._keys import EMA_EVENT, EMA_INITIALIZED, EMA_PENDING, EMA_SHADOW, EMA_TMP_CPU
from dionw_b200.ema.config import EMAConfig, EMADevice, ProfileRegion

if TYPE_CHECKING:
    from torch.optim import Optimizer

FP32 = torch.float32
_STAGE_REGION = "ema_stage_copy"
_FINALIZE_REGION = "ema_finalize"


class OptimizerIntegratedEMA:
    """EMA shadows stored in ``optimizer.state[p]`` (created at the first update after
    the optimizer has created ``p``'s state)."""

    def __init__(self, optimizer: "Optimizer", config: EMAConfig, profile_region: ProfileRegion) -> None:
        if config.device not in (EMADevice.GPU, EMADevice.CPU):
            raise RuntimeError(f"Unhandled EMADevice: {config.device}")
        self.optimizer = optimizer
        self.config = config
        self._profile_region = profile_region
        self._on_gpu = config.device is EMADevice.GPU
        self._step_count = 0
        self._due = True
        self._reseed = False               # this step copies the live weights (start_step)
        self._decay_now: float | None = None
        # GPU: work queued by update_param until finalize_updates
        self._copy_queue: list[tuple[Tensor, Tensor]] = []
        self._lerp_queue: list[tuple[Tensor, Tensor]] = []
        # CPU: one pinned staging buffer, one update in flight at most (its jobs: one per
        # chunk of the snapshot, so the host averages chunk i while chunk i + 1 crosses the link)
        self._staged: list[tuple[Tensor, dict[str, Any]]] = []
        self._staging: Tensor | None = None
        self._jobs: list[_native.CpuEmaJob] = []
        self._job_states: list[dict[str, Any]] = []
        self._snapshot_event: torch.cuda.Event | None = None
        self._copy_streams: dict[torch.device, torch.cuda.Stream] = {}
        self._threads = max(1, min(16, (os.cpu_count() or 2) // 2))
        # What of a parameter this tracker follows: the whole tensor, unless the owning
        # optimizer keeps only a slice of each shadow (an optimizer sharded over ranks).
        self.source_view: Callable[[Tensor], Tensor] = lambda param: param

    # ---- schedule ---------------------------------------------------------
    @property
    def step_count(self) -> int:
        """Optimizer steps the schedule has seen (saved with the state)."""
        return self._step_count

    @step_count.setter
    def step_count(self, value: int) -> None:
        if value < 0:
            raise ValueError(f"EMA step_count must be non-negative, got {value}")
        self._step_count = value

    @property
    def uses_gpu_shadow(self) -> bool:
        """Whether shadows live on the parameters' GPU (else in host memory)."""
        return self._on_gpu

    def begin_step(self) -> None:
        """Advance the schedule; called before the optimizer's own step."""
        if not self._on_gpu:
            self._order_after_snapshot()
        self._step_count += 1
        cfg = self.config
        start, every = cfg.start_step, cfg.update_every_n_steps
        self._reseed = start > 0 and self._step_count == start
        if start > 0 and self._step_count < start:
            self._due = False
        elif self._reseed:
            self._due = True
        else:
            since = self._step_count - start
            self._due = since > 0 and since % every == 0
        decay = cfg.decay_at_step(self._step_count)
        self._decay_now = decay**every if self._due and not self._reseed else None
        # The previous CPU update is awaited at this step's first ``update_param``, not here: the
        # optimizer's own step, which runs in between, touches neither the shadows nor the staging
        # buffer, so its GPU work overlaps the tail of that update.

    def should_update_this_step(self) -> bool:
        """Whether this step updates the shadows."""
        return self._due

    # ---- staging one parameter -------------------------------------------
    @torch.no_grad()
    def update_param(self, param: Tensor) -> None:
        """Stage one parameter for this step's update (applied by ``finalize_updates``)."""
        with self._profile_region(_STAGE_REGION):
            if not self._due or param not in self.optimizer.state:
                return
            if self._jobs:   # CPU: the update in flight owns the shadows and the staging buffer
                self._finish_job()
            state = self.optimizer.state[param]
            if EMA_SHADOW not in state:
                self._new_shadow(param, state)
            source = self.source_view(param)
            if self._on_gpu:
                if self._reseed or not state[EMA_INITIALIZED]:
                    self._copy_queue.append((state[EMA_SHADOW], source))
                    state[EMA_INITIALIZED] = True
                else:
                    self._lerp_queue.append((state[EMA_SHADOW], source))
                state[EMA_PENDING] = False
            else:
                if self._reseed:
                    state[EMA_INITIALIZED] = False
                self._staged.append((source, state))
                state[EMA_PENDING] = True

    def _new_shadow(self, param: Tensor, state: dict[str, Any]) -> None:
        if self._on_gpu and not param.is_cuda:
            raise ValueError("EMA configured for the GPU but a parameter is on the CPU")
        pin = self.config.pin_memory and not self._on_gpu
        state[EMA_SHADOW] = torch.zeros_like(
            self.source_view(param), dtype=FP32, device=param.device if self._on_gpu else torch.device("cpu"),
            pin_memory=pin)
        state[EMA_INITIALIZED] = False

    # ---- applying ---------------------------------------------------------
    @torch.no_grad()
    def finalize_updates(self) -> None:
        """Apply this step's GPU updates, or hand the CPU snapshot to the worker."""
        with self._profile_region(_FINALIZE_REGION):
            if self._on_gpu:
                self._flush_gpu()
            elif self._due:
                self._launch_cpu_update()

    def flush_pending_updates(self) -> None:
        """Finish queued EMA work before the shadows are read.

        Raises:
            RuntimeError: If the CPU worker failed.
        """
        if self._on_gpu:
            self._flush_gpu()
        else:
            self._finish_job()

    @torch.no_grad()
    def _flush_gpu(self) -> None:
        weight = 1.0 - (self.config.decay if self._decay_now is None else self._decay_now)
        for queue, first in ((self._copy_queue, True), (self._lerp_queue, False)):
            by_kind: dict[tuple[torch.device, torch.dtype], tuple[list[Tensor], list[Tensor]]] = {}
            for shadow, source in queue:
                if shadow.dtype is not FP32:
                    raise TypeError("EMA shadows must be float32")
                if not source.is_contiguous():
                    source = source.contiguous()
                pair = by_kind.setdefault((source.device, source.dtype), ([], []))
                pair[0].append(shadow)
                pair[1].append(source)
            for (device, dtype), (shadows, sources) in by_kind.items():
                if dtype not in (torch.float32, torch.float16, torch.bfloat16):
                    sources = [s.float() for s in sources]
                with torch.cuda.device(device):
                    _native.ema_multi(shadows, sources, weight=weight, first=first)
            queue.clear()

    def _copy_stream(self, device: torch.device) -> torch.cuda.Stream:
        stream = self._copy_streams.get(device)
        if stream is None:
            stream = self._copy_streams[device] = torch.cuda.Stream(device=device)
        return stream

    # A snapshot of at least this many elements is taken in SNAPSHOT_CHUNKS pieces.
    SNAPSHOT_CHUNK_MIN_ELEMENTS = 1 << 24
    SNAPSHOT_CHUNKS = 4

    def _snapshot_chunks(self, items: list[tuple[int, Tensor]]) -> list[list[tuple[int, Tensor]]]:
        """``items`` (index, parameter) cut, in order, into pieces of about equal element counts."""
        total = sum(p.numel() for _, p in items)
        if total < self.SNAPSHOT_CHUNK_MIN_ELEMENTS or len(items) < 2:
            return [items]
        target = -(-total // self.SNAPSHOT_CHUNKS)
        chunks: list[list[tuple[int, Tensor]]] = [[]]
        filled = 0
        for item in items:
            if filled >= target and len(chunks) < self.SNAPSHOT_CHUNKS:
                chunks.append([])
                filled = 0
            chunks[-1].append(item)
            filled += item[1].numel()
        return chunks

    def _launch_cpu_update(self) -> None:
        staged, self._staged = self._staged, []
        if not staged:
            return
        if self._jobs:
            raise RuntimeError("CPU EMA job already pending after the pre-step wait")
        total = sum(p.numel() for p, _ in staged)
        pin = self.config.pin_memory
        if self._staging is None or self._staging.numel() < total or self._staging.is_pinned() != pin:
            self._staging = torch.empty(total, dtype=FP32, device="cpu", pin_memory=pin)
        staging = self._staging
        offsets, cursor = [], 0
        for param, state in staged:
            offsets.append(cursor)
            state[EMA_TMP_CPU] = staging[cursor : cursor + param.numel()].view(param.shape)
            cursor += param.numel()
        # (members, event) per job: the worker of a job waits for its event, then averages its members
        pieces: list[tuple[list[int], torch.cuda.Event | None]] = []
        cuda_items = [(i, p) for i, (p, _) in enumerate(staged) if p.is_cuda]
        if cuda_items and pin:
            device = cuda_items[0][1].device
            side = self._copy_stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                for chunk in self._snapshot_chunks(cuda_items):
                    by_dtype: dict[torch.dtype, list[int]] = {}
                    for i, p in chunk:
                        by_dtype.setdefault(p.dtype, []).append(i)
                    for dtype, members in by_dtype.items():
                        sources = [staged[i][0] if staged[i][0].is_contiguous() else staged[i][0].contiguous()
                                   for i in members]
                        if dtype not in (torch.float32, torch.float16, torch.bfloat16):
                            sources = [s.float() for s in sources]
                        # The kernel writes through the pinned buffer's device mapping.
                        _native.ema_stage_pack(sources, [offsets[i] for i in members], staging)
                        for s in sources:
                            s.record_stream(side)
                    event = torch.cuda.Event(blocking=False)
                    event.record(side)
                    pieces.append(([i for i, _ in chunk], event))
            self._snapshot_event = pieces[-1][1]   # the last piece is recorded after all the others
            rest = [i for i, (p, _) in enumerate(staged) if not p.is_cuda]
        else:
            rest = list(range(len(staged)))
        for i in rest:  # host parameters, or unpinned staging: plain blocking copies
            staged[i][1][EMA_TMP_CPU].copy_(staged[i][0].detach(), non_blocking=False)
        if rest:
            pieces.append((rest, None))
        weight = 1.0 - (self.config.decay if self._decay_now is None else self._decay_now)
        self._job_states = [state for _, state in staged]
        for members, event in pieces:
            states = [staged[i][1] for i in members]
            for state in states:
                state[EMA_EVENT] = event
            self._jobs.append(_native.CpuEmaJob(
                [state[EMA_SHADOW].view(-1) for state in states],
                [state[EMA_TMP_CPU].view(-1) for state in states],
                [not state[EMA_INITIALIZED] for state in states], weight, event, self._threads))

    def _order_after_snapshot(self) -> None:
        """Make the device wait until the last snapshot no longer reads the live parameters."""
        event, self._snapshot_event = self._snapshot_event, None
        if event is not None:
            torch.cuda.current_stream().wait_event(event)
        if self._jobs and all(job.done() for job in self._jobs):
            self._finish_job()

    def _finish_job(self) -> None:
        """Wait for every job of the update in flight; the first failure is re-raised after all are closed."""
        jobs, self._jobs = self._jobs, []
        if not jobs:
            return
        states, self._job_states = self._job_states, []
        failure: Exception | None = None
        for job in jobs:
            try:
                job.wait_update()
            except Exception as exc:  # noqa: BLE001 - re-raised below with the reference's message
                failure = failure or exc
            finally:
                job.close()
        if failure is not None:
            raise RuntimeError("Asynchronous CPU EMA update failed") from failure
        for state in states:
            state[EMA_INITIALIZED] = True
            state[EMA_PENDING] = False
            state.pop(EMA_EVENT, None)
