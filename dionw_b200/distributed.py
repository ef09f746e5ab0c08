"""``ShardedDion``: the Dion step over several GPUs of one node.

The reference is single-GPU by design (README.md:446-456 there); this is new
design on top of the same kernels.  Weights and gradients are replicated on
every rank (the state after a data-parallel gradient all-reduce).  What is
sharded is the optimizer's work and state:

* matrix parameters are dealt to ranks by Newton-Schulz cost (longest first, to
  the least loaded rank); a rank keeps momentum and variance only for the
  parameters it owns and runs stages 1-4 of the step (accumulate, select, pack,
  orthogonalize, NorMuon scales) for them alone;
* per round, ONE all-gather ships what a replica needs to apply a run: the bf16
  update rows, the row map, the row divisors and the block scales (they lie
  contiguously at the head of the run's scratch arena, so the arena is the send
  buffer); every rank then applies every run to its replica of the weights with
  the same kernel and the same inputs, so replicas stay bit-identical;
* large AdamW tensors are cut into ``world`` equal element ranges: each rank
  updates its range (moments exist only for it) and an in-place all-gather
  rebuilds the parameter; small ones are updated on every rank;
* the EMA (``ema=EMAConfig(...)``) keeps, of every large parameter, the shadow of
  this rank's element range only: replicas are identical after the step, so each
  rank averages its range with no communication, on the GPU or through the
  pinned-host worker; small parameters keep whole shadows on every rank.

The all-gather of round t is in flight while round t+1 computes (two scratch
arenas alternate).  Received data is in local memory before any kernel reads it;
no kernel touches a peer's memory.
"""

from __future__ import annotations

import math
from collections.abc import Callable, Iterable, Sequence
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

from dionw_b200 import _matrix_step, _native, _workspace
from dionw_b200._adamw import init_adamw_state
from dionw_b200._buckets import Bucket, block_shape, build_buckets
from dionw_b200._keys import (
    ADAMW_STEP_STATE, EMA_PENDING, EMA_SCRATCH_KEYS, EMA_SHADOW, EMA_STEP_COUNT_KEY, EXP_AVG_SQ_STATE,
    EXP_AVG_STATE, FRACTION_KEY, MOMENTUM_STATE, NUM_HEADS_KEY, ROUTE_KEY, VARIANCE_STATE,
)
from dionw_b200.ema import EMAConfig, IntegratedEMAOptimizer, ProfileRegion, no_profile
from dionw_b200.matrix_update import DION3_UPDATE, MatrixUpdate
from dionw_b200.optimizer import _DionCore, _fill_legacy_keys, _require_same_structure
from dionw_b200.routing import RouteKind

SHARD_KEY = "_dionw_shard"   # top-level entry of a per-rank checkpoint

__all__ = ["SHARD_KEY", "ShardedDion", "assign_by_cost", "bucket_order", "is_cut", "newton_schulz_cost", "shard_range", "split_runs"]

# AdamW tensors at least this large are cut into per-rank element ranges.
ADAMW_SHARD_MIN_ELEMENTS = 1 << 20


# ---------------------------------------------------------------------------
# host-side planning (pure functions; the same on every rank)
# ---------------------------------------------------------------------------
def newton_schulz_cost(rows: int, cols: int, k: int, blocks: int = 1) -> float:
    """FLOPs of orthogonalizing ``blocks`` operands of ``k`` selected rows by ``cols`` columns."""
    m, n = min(k, cols), max(k, cols)
    per_block = 20.0 * m**3 if m == n else 2.0 * (3.0 * m * m * n + 11.5 * m**3)
    return blocks * per_block


def assign_by_cost(costs: Sequence[float], world: int) -> list[int]:
    """Owner rank of each unit: longest processing time first, to the least loaded rank.

    Ties go to the lower unit index and the lower rank, so every rank computes the same answer.
    """
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0.0] * world
    owner = [0] * len(costs)
    for i in order:
        rank = min(range(world), key=lambda r: (load[r], r))
        owner[i] = rank
        load[rank] += costs[i]
    return owner


def bucket_order(costs: Sequence[float], costliest_second: bool) -> list[int]:
    """Order in which the buckets' rounds are taken: by cost, highest first (ties to the lower
    index); with ``costliest_second`` and at least three buckets the two costliest change places,
    so that the costliest bucket's gather has a weight update and a round's own work to hide behind."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    if costliest_second and len(order) >= 3:
        order[0], order[1] = order[1], order[0]
    return order


def split_runs(sizes: Sequence[int | None], limit: int) -> list[list[int]]:
    """Positions grouped into runs of consecutive entries, as ``_DionCore._step_bucket`` does.

    ``sizes[i]`` is the update-element count of entry ``i``, or None when it has no gradient
    (which ends the current run).  A run holds at most ``limit`` elements; a larger entry runs alone.
    """
    runs: list[list[int]] = []
    current: list[int] = []
    total = 0
    for position, size in enumerate(sizes):
        if current and (size is None or total + size > limit):
            runs.append(current)
            current, total = [], 0
        if size is not None:
            current.append(position)
            total += size
    if current:
        runs.append(current)
    return runs


def is_cut(numel: int, world: int, contiguous: bool, multiple: int = 1) -> bool:
    """Whether a tensor of ``numel`` elements is kept as one element range per rank: more than one
    rank, at least ``ADAMW_SHARD_MIN_ELEMENTS`` elements, contiguous, and a size that divides into
    ``world`` ranges of a multiple of ``multiple`` elements (4 keeps fp32 ranges 16-byte aligned)."""
    return world > 1 and numel >= ADAMW_SHARD_MIN_ELEMENTS and numel % (multiple * world) == 0 and contiguous


def shard_range(numel: int, rank: int, world: int) -> tuple[int, int]:
    """Element range ``[start, stop)`` of ``rank`` when ``numel`` divides evenly by ``world``."""
    per = numel // world
    return rank * per, (rank + 1) * per


@dataclass
class _SharedBucket:
    """Same-shape matrix parameters of one group across all ranks."""

    group_index: int
    rows: int
    cols: int
    k: int
    params: list[Tensor]
    blocks: list[int]           # blocks per parameter
    owners: list[int]           # owner rank per parameter
    local: Bucket | None = None  # this rank's slab (owned parameters only)
    decay_device: Tensor | None = None  # 1 - lr * weight_decay of the group, in the device table of step scalars


@dataclass
class _Round:
    """One all-gather in flight: who contributed what, and where it lands."""

    work: Any
    recv: Tensor
    slot: int
    counts: list[int]
    params: list[list[Tensor]]
    blocks: list[list[int]]
    bucket: _SharedBucket
    group: dict[str, Any]
    job: Tensor | None = None   # the decay job the round's products carried


class _ShardedCore(_DionCore):
    """The sharded step and its checkpoint layout, without the EMA."""

    def __init__(self, params: Iterable[dict[str, Any]], *, lr: float, momentum: float = 0.95,
                 muon_beta2: float = 0.95, betas: tuple[float, float] = (0.9, 0.95), weight_decay: float = 0.0,
                 eps: float = 1e-8, matrix_update: MatrixUpdate = DION3_UPDATE, process_group: Any = None,
                 fused_decay: bool = False) -> None:
        import torch.distributed as dist

        if not dist.is_initialized():
            raise RuntimeError("ShardedDion needs torch.distributed to be initialised (one process per GPU)")
        self._dist = dist
        self._pg = process_group
        self._world = dist.get_world_size(process_group)
        self._rank = dist.get_rank(process_group)
        self.fused_decay = bool(fused_decay)
        # The rounds' row maps travel on a communicator of their own: NCCL runs the collectives of one
        # communicator in the order they were issued, and a 60 KB exchange that the round's products
        # wait for must not queue behind the previous round's results or AdamW's ranges (2 GPUs,
        # one communicator: 6.9 ms of a 58.9 ms step spent there).  Every rank issues the same
        # collectives in the same order on both communicators.
        self._pg_maps = process_group
        if self._world > 1 and self.fused_decay:
            self._pg_maps = dist.new_group(ranks=dist.get_process_group_ranks(process_group or dist.group.WORLD))
        if self._world > 1 and self.dynamic_tiles:
            # The rounds' tensor-core products run beside NCCL's kernels, which hold a few SMs for
            # milliseconds: with tiles drawn from a counter a product loses those SMs' share of its
            # tiles instead of waiting for the SM pairs that cannot start (process-wide setting).
            _native.gemm_dynamic_tiles(True)
        self._shared: list[_SharedBucket] | None = None
        self._costliest: _SharedBucket | None = None
        self._round_streams: dict[torch.device, tuple[Any, Any]] = {}
        super().__init__(params, lr=lr, momentum=momentum, muon_beta2=muon_beta2, betas=betas,
                         weight_decay=weight_decay, eps=eps, matrix_update=matrix_update)

    # ---- layout --------------------------------------------------------------
    def _is_cut(self, param: Tensor) -> bool:
        """Whether an AdamW tensor is updated by element range rather than whole on every rank."""
        return is_cut(param.numel(), self._world, param.is_contiguous())

    def _new_adamw_state(self, param: Tensor) -> None:
        entry = self.state[param]
        if not self._is_cut(param):
            init_adamw_state(param, entry)
            return
        per = param.numel() // self._world
        entry[EXP_AVG_STATE] = torch.zeros(per, dtype=param.dtype, device=param.device)
        entry[EXP_AVG_SQ_STATE] = torch.zeros(per, dtype=param.dtype, device=param.device)
        entry[ADAMW_STEP_STATE] = torch.zeros((), dtype=torch.float32, device=param.device)

    def add_param_group(self, param_group: dict[str, Any]) -> None:
        super().add_param_group(param_group)
        self._shared = None

    def owners(self) -> dict[Tensor, int]:
        """Owner rank of every matrix parameter."""
        return {p: o for sb in self._ensure_shared() for p, o in zip(sb.params, sb.owners)}

    def _ensure_shared(self) -> list[_SharedBucket]:
        if self._shared is not None:
            return self._shared
        units: list[tuple[int, Tensor, int, int, int, int]] = []
        for gi, group in enumerate(self.param_groups):
            if RouteKind(group[ROUTE_KEY]) is not RouteKind.MATRIX:
                continue
            for param in group["params"]:
                blocks, rows, cols = block_shape(param, group[NUM_HEADS_KEY])
                k = min(rows, math.ceil(float(group[FRACTION_KEY]) * rows))
                units.append((gi, param, blocks, rows, cols, k))
        owners = assign_by_cost([newton_schulz_cost(r, c, k, b) for _, _, b, r, c, k in units], self._world)
        shared: dict[tuple, _SharedBucket] = {}
        owned: dict[int, list[Tensor]] = {}
        for (gi, param, blocks, rows, cols, k), owner in zip(units, owners):
            sb = shared.setdefault((gi, rows, cols, param.device),
                                   _SharedBucket(gi, rows, cols, k, [], [], []))
            sb.params.append(param)
            sb.blocks.append(blocks)
            sb.owners.append(owner)
            if owner == self._rank:
                owned.setdefault(gi, []).append(param)
        filtered = [
            {**group, "params": owned.get(gi, [])} if RouteKind(group[ROUTE_KEY]) is RouteKind.MATRIX else group
            for gi, group in enumerate(self.param_groups)
        ]
        for bucket in build_buckets(filtered, self.state):
            shared[(bucket.group_index, bucket.rows, bucket.cols, bucket.params[0].device)].local = bucket
        mine = {id(p) for ps in owned.values() for p in ps}
        for sb in shared.values():
            for param in sb.params:
                entry = self.state[param]   # every rank keeps an entry: the EMA hangs its shadow there
                if id(param) not in mine:   # a loaded checkpoint leaves full state everywhere: keep the owner's only
                    entry.pop(MOMENTUM_STATE, None)
                    entry.pop(VARIANCE_STATE, None)
        # Costliest buckets first: the gathers and weight updates of the large rounds then have the
        # later rounds' work to hide behind, and the last gather of the step, which nothing
        # hides, is the smallest.  With ``costliest_second`` the second costliest bucket goes before
        # the costliest: the costliest bucket's gather (1.9 GB into every rank at the Llama-3-8B
        # shapes on 8 ranks, about 2.7 ms) is then followed by a weight update AND a round's own
        # work before its result is needed, instead of by one short round.  Parameters are
        # independent, so the order changes no result.
        buckets = list(shared.values())
        costs = [sum(newton_schulz_cost(sb.rows, sb.cols, sb.k, b) for b in sb.blocks) for sb in buckets]
        self._costliest = buckets[max(range(len(costs)), key=lambda i: (costs[i], -i))] if buckets else None
        self._shared = [buckets[i] for i in bucket_order(costs, self.costliest_second)]
        self._buckets = [sb.local for sb in self._shared if sb.local is not None]
        return self._shared

    def _ensure_buckets(self) -> list[Bucket]:
        self._ensure_shared()
        return self._buckets or []

    def _scalar_slots(self) -> list[Any]:
        # every rank applies every bucket's update, so the buckets owned elsewhere need their
        # group's decay factor in the device table too
        return list(self._ensure_buckets()) + list(self._ensure_shared())

    # ---- the step ------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        gathers: list[Any] = []
        self._refresh_scalars()
        if self.adamw_first:
            gathers.extend(self._step_adamw())
            self._step_matrices(None)
        else:
            done: list[bool] = []

            def adamw() -> None:
                done.append(True)
                gathers.extend(self._step_adamw())

            self._step_matrices(adamw)
            if not done:   # no matrix round took place
                adamw()
        with _matrix_step._stage("gather_wait"):
            for work in gathers:
                work.wait()
        return loss

    # Where the AdamW tensors are updated and their ranges gathered.  Their all-gathers move 4 B per
    # AdamW element into every rank (3.7 GB at the Llama-3-8B shapes on 8 ranks), NCCL runs the
    # collectives of one communicator in the order they were issued, and its kernels need SMs: beside
    # the tensor-core products they take about a fifth of them, beside the HBM-bound weight update,
    # whose CTAs fill every SM's thread slots, they hardly get to run at all.  Issued first in the step
    # (the default) the gathers are out of the queue before the first large round's results arrive
    # behind them, and run beside the front stages and the Newton-Schulz of the first rounds, whose
    # products draw their tiles from a counter (``dynamic_tiles``) and lose only the SMs NCCL holds.
    # Measured, Llama-3-8B shapes, ms per step (Newton-Schulz stage; time the step waits for gathers):
    #                                                       4 GPUs                8 GPUs
    #   AdamW first, tiles from a counter (default)         34.8 (17.1; 0.2)      25.0 (10.1; 0.3)
    #   AdamW first, fixed stride                           35.9 (19.0; 0.1)
    #   right after the costliest bucket, fixed stride      36.7 (16.5; 3.3)      28.0 (8.5; 3.5)
    #   one round after the costliest bucket, counter       37.3 (16.3; 3.3)
    # (alone on a GPU the same blocks take 16.1 and 8.2 ms of Newton-Schulz).  A communicator of the
    # AdamW gathers' own, limited to 2-8 CTAs so that it takes fewer SMs, was also measured on 4 GPUs:
    # 8 CTAs 35.4 ms (no better), 4 CTAs 50 ms, 2 CTAs 81 ms (about 12 GB/s per CTA: the gathers no
    # longer fit in the step).  ``adamw_first = False`` issues AdamW ``adamw_delay_rounds`` rounds
    # after the costliest bucket's last round.  The order changes no result.
    adamw_first = True
    adamw_delay_rounds = 1
    costliest_second = True
    dynamic_tiles = True

    def _all_gather(self, out: Tensor, piece: Tensor) -> Any:
        return self._dist.all_gather_into_tensor(out, piece, group=self._pg, async_op=True)

    # Update elements one round may hold per rank (the single-GPU cap bounds it from above), and
    # whether the weight update of round t runs beside the Newton-Schulz of round t+1.
    #
    # The update of a round is 8 B per weight element on EVERY rank (decoupled decay of all rows):
    # it does not shrink with the number of GPUs and is the largest stage of the step on 8.  With
    # ``overlap_apply`` the rounds' own work (accumulate ... Newton-Schulz, and the gathers) runs on
    # a high-priority stream, the updates and AdamW on a default-priority one.  Two things make
    # that pay, where a first version only moved the time around: the update is launched with
    # CTAs of four warps (``apply_warps``), small enough in registers that two of them fit beside a
    # resident tensor-core CTA, and the priority lets a product's CTAs take an SM before the
    # update's queued CTAs do, so a product no longer waits for the update's grid to drain.
    # ``round_elements`` cuts the costliest bucket into several rounds so that its own update has
    # later Newton-Schulz work to hide behind.  Same kernels, same inputs: the results are
    # bit-identical to the in-line order.
    round_elements = 1 << 28
    overlap_apply = False
    apply_warps = 4

    def _streams(self, device: torch.device) -> tuple[Any, Any]:
        """(high-priority stream for the rounds, default-priority stream for the updates)."""
        pair = self._round_streams.get(device)
        if pair is None:
            pair = self._round_streams[device] = (torch.cuda.Stream(device=device, priority=-1),
                                                  torch.cuda.Stream(device=device))
        return pair

    def _step_matrices(self, after_costliest: Callable[[], None] | None) -> None:
        """Every round of the matrix step; ``after_costliest`` is called ``adamw_delay_rounds`` rounds
        after the costliest bucket's last round, once that round's results are on their way."""
        import dionw_b200.optimizer as optimizer_module  # MAX_RUN_ELEMENTS is looked up at call time

        limit = min(optimizer_module.MAX_RUN_ELEMENTS, self.round_elements)
        world, me = self._world, self._rank
        shared = self._ensure_shared()
        if not shared:
            return
        device = shared[0].params[0].device
        main = torch.cuda.current_stream(device)
        if self.overlap_apply:
            compute, side = self._streams(device)
            compute.wait_stream(main)
            side.wait_stream(main)
        else:
            compute = side = main
        pending: _Round | None = None
        applied: list[Any] = []  # applied[t]: event recorded on the side stream after round t's update
        round_id = 0
        fire_round = -1          # the round after whose gather AdamW is issued
        with torch.cuda.stream(compute):
            for sb in shared:
                group = self.param_groups[sb.group_index]
                selecting = sb.k < sb.rows
                per_rank = [[i for i, o in enumerate(sb.owners) if o == r] for r in range(world)]
                runs = []
                for members in per_rank:
                    sizes = [None if sb.params[i].grad is None else sb.blocks[i] * sb.k * sb.cols for i in members]
                    runs.append([[members[j] for j in run] for run in split_runs(sizes, limit)])
                rounds = max((len(r) for r in runs), default=0)
                for t in range(rounds):
                    chosen = [r[t] if t < len(r) else [] for r in runs]
                    counts = [sum(sb.blocks[i] for i in c) for c in chosen]
                    slot = max(_workspace.layout(_matrix_step.exchange_plan(c, sb.rows, sb.k, sb.cols, selecting))[1]
                               if c else 0 for c in counts)
                    if round_id >= 2:
                        # This round reuses the send and receive arenas of round_id - 2.
                        compute.wait_event(applied[round_id - 2])
                    name = f"run{round_id % 2}"
                    _workspace.arena(device, slot, name)
                    ctx = None
                    if chosen[me]:
                        local_index = {id(p): j for j, p in enumerate(sb.local.params)}
                        positions = [local_index[id(sb.params[i])] for i in chosen[me]]
                        ctx = _matrix_step.open_run(sb.local, positions, group, arena=name)
                        _matrix_step.run_front(ctx)
                    job = None
                    if (self.fused_decay and selecting and compute is main and float(group["weight_decay"]) > 0.0
                            and 0 < sum(len(c) for c in chosen) <= 64):
                        job = self._begin_decay_job(sb, group, chosen, counts, slot, name, round_id, device)
                    if ctx is not None:
                        _native.gemm_side_job(job)
                        try:
                            _matrix_step.run_core(ctx)
                        finally:
                            _native.gemm_side_job(None)
                    send = _workspace.arena(device, slot, name)[:slot]
                    if world == 1:
                        recv, work = send, None
                    else:
                        recv = _workspace.arena(device, slot * world, f"recv{round_id % 2}")[: slot * world]
                        work = self._all_gather(recv, send)
                    issued = _Round(work, recv, slot, counts, [[sb.params[i] for i in c] for c in chosen],
                                    [[sb.blocks[i] for i in c] for c in chosen], sb, group, job)
                    if sb is self._costliest and t == rounds - 1:
                        fire_round = round_id + max(0, int(self.adamw_delay_rounds))
                    if round_id == fire_round and after_costliest is not None:
                        with torch.cuda.stream(side):
                            after_costliest()
                    if pending is not None:
                        applied.append(self._apply_round(pending, compute, side))
                    pending = issued
                    round_id += 1
            if pending is not None:
                applied.append(self._apply_round(pending, compute, side))
        if compute is not main:
            main.wait_stream(compute)
            main.wait_stream(side)

    # The decoupled decay of the rows a round does NOT select (three quarters of the 8 B per weight
    # element that every rank spends on the update) depends on nothing but the row maps, which exist
    # after `select`, before the round's first product.  With ``fused_decay=True`` (constructor
    # argument; off by default) the ranks exchange their row maps right there (a small all-gather on
    # a communicator of its own), describe the round's weights in a decay job (csrc/decay_job.cuh),
    # and the round's tensor-core products carry it: their epilogue warps decay rows while they wait
    # for their accumulators.  The update kernel then skips what the job's cursor covers.  Same
    # multiplication, once per element: bit-identical weights.  Measured (Llama-3-8B shapes, ms,
    # off -> on): 2 GPUs update 10.7 -> 7.7, Newton-Schulz 32.8 -> 34.6, step 56.8 -> 56.5; 4 GPUs update
    # 10.6 -> 7.5, Newton-Schulz 17.6 -> 19.8, step 35.4 -> 34.9: during the products the board is at its
    # power cap, so the joules of the rows streamed beside them come out of the products' clock.
    decay_rows_per_wait = 2

    def _begin_decay_job(self, sb: _SharedBucket, group: dict[str, Any], chosen: list[list[int]], counts: list[int],
                         slot: int, name: str, round_id: int, device: torch.device) -> Tensor | None:
        world, me = self._world, self._rank
        plans = [_workspace.layout(_matrix_step.exchange_plan(c, sb.rows, sb.k, sb.cols, True))[0]["rowmap"] if c else (0, 0)
                 for c in counts]
        piece_bytes = max(nbytes for _, nbytes in plans)
        piece_bytes = (piece_bytes + 255) // 256 * 256
        own_offset = plans[me][0]
        send = _workspace.arena(device, slot, name)
        if world == 1:
            maps = send[own_offset:own_offset + piece_bytes]
            stride = 0
        else:
            maps = _workspace.arena(device, piece_bytes * world, f"rowmaps{round_id % 2}")[: piece_bytes * world]
            # the piece may run past this rank's own row maps into what follows them in the arena
            # (the largest contribution's layout bounds it): the other ranks never look there
            self._dist.all_gather_into_tensor(maps, send[own_offset:own_offset + piece_bytes], group=self._pg_maps)
            stride = piece_bytes
        weights: list[Tensor] = []
        rowmaps: list[int] = []
        rows_per_tensor: list[int] = []
        base = maps.data_ptr()
        for rank in range(world):
            block = 0
            for i in chosen[rank]:
                weights.append(sb.params[i])
                rowmaps.append(base + rank * stride + block * sb.rows * 4)
                rows_per_tensor.append(sb.blocks[i] * sb.rows)
                block += sb.blocks[i]
        if not all(w.is_contiguous() for w in weights):
            return None   # a strided weight is updated through a packed copy: nothing to decay in place
        job = _workspace.arena(device, _native.decay_job_bytes(), f"decayjob{round_id % 2}")
        lr, weight_decay = float(group["lr"]), float(group["weight_decay"])
        _native.decay_job_begin(job, weights, rowmaps, rows_per_tensor, rows=sb.rows, cols=sb.cols,
                                decay_factor=1.0 - lr * weight_decay, decay_device=sb.decay_device,
                                rows_per_wait=self.decay_rows_per_wait)
        return job

    def _apply_round(self, rnd: _Round, compute: Any, side: Any) -> Any:
        """Every rank's contribution of one round applied to this replica with one launch, on the side stream."""
        with torch.cuda.stream(side):
            if rnd.work is not None:
                with _matrix_step._stage("gather_wait"):
                    rnd.work.wait()         # the side stream waits for the gather
            elif side is not compute:
                side.wait_stream(compute)   # one rank: the "received" data is the local result
            sb = rnd.bucket
            selecting = sb.k < sb.rows
            results = []
            for rank, count in enumerate(rnd.counts):
                if count == 0:
                    continue
                got = _workspace.views(rnd.recv,
                                       _matrix_step.exchange_plan(count, sb.rows, sb.k, sb.cols, selecting),
                                       base=rank * rnd.slot)
                results.append(_matrix_step.RunResult(
                    params=rnd.params[rank], rows_per_tensor=[b * sb.rows for b in rnd.blocks[rank]], count=count,
                    rows=sb.rows, k=sb.k, cols=sb.cols, orthogonal=got["x"], rowmap=got.get("rowmap"),
                    denom=got["denom"], scale=got["scale"], decay_device=sb.decay_device))
            if results:
                _matrix_step.apply_results(results, rnd.group,
                                           warps=self.apply_warps if side is not compute else 0, decay_job=rnd.job)
            done = torch.cuda.Event()
            done.record(side)
        return done

    def _step_adamw(self) -> list[Any]:
        gathers: list[Any] = []
        for index, group in enumerate(self.param_groups):
            if RouteKind(group[ROUTE_KEY]) is not RouteKind.ADAMW:
                continue
            lists: tuple[list[Tensor], ...] = ([], [], [], [], [])
            rebuilt: list[tuple[Tensor, Tensor]] = []
            for param in group["params"]:
                grad = param.grad
                if grad is None:
                    continue
                entry = self.state[param]
                if EXP_AVG_STATE not in entry:
                    self._new_adamw_state(param)
                if grad.dtype is not torch.float32 or not grad.is_contiguous():
                    grad = grad.float().contiguous()
                target, source = param, grad
                if self._is_cut(param):
                    start, stop = shard_range(param.numel(), self._rank, self._world)
                    target, source = param.view(-1)[start:stop], grad.view(-1)[start:stop]
                    rebuilt.append((param.view(-1), target))
                elif not param.is_contiguous():
                    raise NotImplementedError("ShardedDion needs contiguous AdamW parameters")
                for store, value in zip(lists, (target, source, entry[EXP_AVG_STATE], entry[EXP_AVG_SQ_STATE],
                                                entry[ADAMW_STEP_STATE])):
                    store.append(value)
            if not lists[0]:
                continue
            beta1, beta2 = group["betas"]
            with _matrix_step._stage("adamw"):
                _native.adamw_multi(*lists, lr=float(group["lr"]), beta1=float(beta1), beta2=float(beta2),
                                    weight_decay=float(group["weight_decay"]), eps=float(group["eps"]),
                                    hyper_device=self._adamw_hyper(index, lists[0][0].device))
            gathers.extend(self._all_gather(whole, piece) for whole, piece in rebuilt)
        return gathers

    # ---- checkpoints ---------------------------------------------------------
    def state_dict(self) -> dict[str, Any]:
        """The single-GPU layout, on every rank: owners broadcast their momentum and variance,
        cut AdamW moments are gathered.  A collective call: every rank must make it."""
        packed = super().state_dict()
        dist = self._dist
        owners = self.owners()
        index = 0
        for group in self.param_groups:
            matrix = RouteKind(group[ROUTE_KEY]) is RouteKind.MATRIX
            for param in group["params"]:
                entry = dict(packed["state"].get(index, {}))
                if matrix and param in owners:
                    owner = owners[param]
                    if owner == self._rank:
                        momentum = self.state[param][MOMENTUM_STATE].clone()
                        variance = self.state[param][VARIANCE_STATE].clone()
                    else:
                        momentum = torch.empty_like(param)
                        variance = torch.empty(param.shape[0], 1, dtype=param.dtype, device=param.device)
                    if self._world > 1:
                        src = dist.get_global_rank(self._pg, owner) if self._pg is not None else owner
                        dist.broadcast(momentum, src=src, group=self._pg)
                        dist.broadcast(variance, src=src, group=self._pg)
                    entry[MOMENTUM_STATE], entry[VARIANCE_STATE] = momentum, variance
                elif not matrix and self._is_cut(param) and EXP_AVG_STATE in self.state.get(param, {}):
                    for key in (EXP_AVG_STATE, EXP_AVG_SQ_STATE):
                        whole = torch.empty_like(param)
                        dist.all_gather_into_tensor(whole.view(-1), self.state[param][key], group=self._pg)
                        entry[key] = whole
                shard = self.state.get(param, {}).get(EMA_SHADOW)
                if shard is not None and self._ema_is_cut(param):
                    entry[EMA_SHADOW] = self._gather_shadow(param, shard)
                if entry:
                    packed["state"][index] = entry
                index += 1
        return packed

    # ---- EMA shards ------------------------------------------------------------
    def _ema_is_cut(self, param: Tensor) -> bool:
        """Whether the EMA keeps only this rank's element range of ``param``'s shadow."""
        return is_cut(param.numel(), self._world, param.is_contiguous(), multiple=4)

    def _ema_view(self, param: Tensor) -> Tensor:
        if not self._ema_is_cut(param):
            return param
        start, stop = shard_range(param.numel(), self._rank, self._world)
        return param.detach().view(-1)[start:stop]

    def _gather_shadow(self, param: Tensor, shard: Tensor) -> Tensor:
        """The whole shadow, in the parameter's shape, on the shard's device (a collective call)."""
        whole = torch.empty(param.shape, dtype=shard.dtype, device=param.device)
        self._dist.all_gather_into_tensor(whole.view(-1), shard.to(param.device).contiguous(), group=self._pg)
        return whole if shard.device == param.device else whole.to(shard.device)

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        """Takes the single-GPU layout; each rank keeps its own share of it."""
        super().load_state_dict(state_dict)
        self._shared = None
        for group in self.param_groups:
            if RouteKind(group[ROUTE_KEY]) is not RouteKind.ADAMW:
                continue
            for param in group["params"]:
                entry = self.state.get(param)
                if not entry or EXP_AVG_STATE not in entry or not self._is_cut(param):
                    continue
                start, stop = shard_range(param.numel(), self._rank, self._world)
                for key in (EXP_AVG_STATE, EXP_AVG_SQ_STATE):
                    if entry[key].numel() == param.numel():
                        entry[key] = entry[key].reshape(-1)[start:stop].clone()


class ShardedDion(IntegratedEMAOptimizer, _ShardedCore):
    """``Dion`` with work and state sharded over the ranks of ``process_group``.

    Same arguments as ``Dion``.  Every rank must hold identical parameters and, at
    each step, identical gradients; after the step the parameters are again
    identical on every rank, and equal bit for bit to what a single-GPU ``Dion``
    computes.  ``state_dict()`` returns the single-GPU layout on every rank (it
    gathers; a collective call); ``load_state_dict()`` takes that layout and keeps
    this rank's share.  ``swap_ema_weights`` / ``restore_non_ema_weights`` are
    collective calls too: shadow ranges are all-gathered straight into the parameters.
    """

    def __init__(self, params: Iterable[dict[str, Any]], *, lr: float, momentum: float = 0.95,
                 muon_beta2: float = 0.95, betas: tuple[float, float] = (0.9, 0.95), weight_decay: float = 0.0,
                 eps: float = 1e-8, matrix_update: MatrixUpdate = DION3_UPDATE, process_group: Any = None,
                 ema: EMAConfig | None = None, profile_region: ProfileRegion = no_profile,
                 fused_decay: bool = False) -> None:
        super().__init__(params, lr=lr, momentum=momentum, muon_beta2=muon_beta2, betas=betas,
                         weight_decay=weight_decay, eps=eps, matrix_update=matrix_update,
                         process_group=process_group, fused_decay=fused_decay)
        self._init_integrated_ema(ema, profile_region)
        if self._ema_helper is not None:
            self._ema_helper.source_view = self._ema_view

    def _loaded_shadow_share(self, param: Tensor, shadow: Tensor) -> Tensor:
        if not self._ema_is_cut(param) or shadow.numel() != param.numel():
            return shadow
        start, stop = shard_range(param.numel(), self._rank, self._world)
        return shadow.reshape(-1)[start:stop]

    def _swap_in(self, param: Tensor, shadow: Tensor) -> Tensor:
        if not self._ema_is_cut(param):
            return super()._swap_in(param, shadow)
        kept = self._ema_view(param).clone()
        self._dist.all_gather_into_tensor(param.data.view(-1), shadow.to(device=param.device, dtype=param.dtype),
                                          group=self._pg)
        return kept

    def _swap_out(self, param: Tensor, kept: Tensor) -> None:
        if not self._ema_is_cut(param):
            super()._swap_out(param, kept)
            return
        self._dist.all_gather_into_tensor(param.data.view(-1), kept, group=self._pg)

    # ---- per-rank checkpoints -----------------------------------------------
    def sharded_state_dict(self) -> dict[str, Any]:
        """This rank's share of the state, as it is held: no collective, nothing gathered.

        For sizes whose gathered ``state_dict()`` does not fit one GPU (the momentum of a
        70B-shaped slice alone is 68 GB).  Every rank saves its own; ``load_sharded_state_dict``
        takes it back on the same rank of a group of the same size with the same parameters.
        """
        self.check_device()
        helper = self._ema_helper
        if helper is not None:
            helper.flush_pending_updates()
        self._ensure_shared()
        packed = torch.optim.Optimizer.state_dict(self)
        packed["state"] = {index: {k: v for k, v in entry.items() if k not in EMA_SCRATCH_KEYS}
                           for index, entry in packed["state"].items()}
        if helper is not None:
            packed[EMA_STEP_COUNT_KEY] = helper.step_count
        owners = self.owners()
        packed[SHARD_KEY] = {
            "rank": self._rank, "world": self._world,
            "owners": [owners.get(p, -1) for group in self.param_groups for p in group["params"]],
        }
        return packed

    def load_sharded_state_dict(self, state_dict: dict[str, Any]) -> None:
        """Take back what ``sharded_state_dict`` of this rank saved.

        Raises:
            ValueError: If it is not a per-rank checkpoint, was saved by another rank or group
                size, assigns the parameters differently, or differs in a structural key.
        """
        meta = state_dict.get(SHARD_KEY)
        if not isinstance(meta, dict):
            raise ValueError("not a per-rank checkpoint: use load_state_dict for the gathered layout")
        if meta.get("rank") != self._rank or meta.get("world") != self._world:
            raise ValueError(
                f"per-rank checkpoint of rank {meta.get('rank')} of {meta.get('world')} "
                f"cannot be loaded on rank {self._rank} of {self._world}")
        saved_groups = _fill_legacy_keys(state_dict["param_groups"])
        _require_same_structure(saved_groups, self.param_groups)
        owners = self.owners()
        if meta.get("owners") != [owners.get(p, -1) for group in self.param_groups for p in group["params"]]:
            raise ValueError("per-rank checkpoint assigns the matrix parameters to other ranks")
        helper = self._ema_helper
        carries_ema = EMA_STEP_COUNT_KEY in state_dict
        if carries_ema and helper is None:
            raise ValueError("the per-rank checkpoint carries EMA shadows but this optimizer has no EMA")
        if helper is not None:
            helper.flush_pending_updates()
            count = state_dict.get(EMA_STEP_COUNT_KEY)
            if type(count) is not int or count < 0:
                raise ValueError(f"per-rank checkpoint has no valid EMA step count ({count!r})")
        on_gpu = helper is not None and helper.uses_gpu_shadow
        pin = helper is not None and helper.config.pin_memory and not on_gpu
        self.state.clear()
        for saved, group in zip(saved_groups, self.param_groups, strict=True):
            for key, value in saved.items():
                if key != "params":
                    group[key] = value
            for index, param in zip(saved["params"], group["params"], strict=True):
                source = state_dict["state"].get(index)
                if source is None:
                    continue
                entry = self.state[param]
                for key, value in source.items():
                    if key == EMA_SHADOW:
                        entry[key] = torch.empty_like(
                            value, device=param.device if on_gpu else torch.device("cpu"), dtype=torch.float32,
                            pin_memory=pin).copy_(value)
                        entry[EMA_PENDING] = False
                    elif isinstance(value, Tensor):
                        entry[key] = value.to(param.device, copy=True)
                    else:
                        entry[key] = value
        if helper is not None:
            helper.step_count = state_dict[EMA_STEP_COUNT_KEY]
        self._shared = None
        self._buckets = None
