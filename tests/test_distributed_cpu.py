"""Host logic of the sharded step, on CPU: the planning functions, and the byte-level
exchange of run results between two ``gloo`` ranks (the same layout arithmetic and the same
collective call the GPU path uses; the kernels themselves need a GPU)."""

from __future__ import annotations

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dionw_b200 import _matrix_step, _workspace
from dionw_b200.distributed import assign_by_cost, newton_schulz_cost, shard_range, split_runs


def test_cost_model_counts_the_gram_schedule() -> None:
    assert newton_schulz_cost(14336, 4096, 3584) == 2 * (3 * 3584**2 * 4096 + 11.5 * 3584**3)
    assert newton_schulz_cost(768, 768, 768) == 20 * 768**3
    assert newton_schulz_cost(3072, 768, 3072) == newton_schulz_cost(768, 3072, 768)  # tall == its transpose
    assert newton_schulz_cost(64, 32, 64, blocks=3) == 3 * newton_schulz_cost(64, 32, 64)


def test_llama8b_blocks_balance_perfectly_over_8_ranks() -> None:
    layer = [(4096, 4096, 1024), (1024, 4096, 256), (1024, 4096, 256), (4096, 4096, 1024),
             (14336, 4096, 3584), (14336, 4096, 3584), (4096, 14336, 1024)]
    costs = [newton_schulz_cost(r, c, k) for _ in range(32) for r, c, k in layer]
    owners = assign_by_cost(costs, 8)
    load = [sum(c for c, o in zip(costs, owners) if o == rank) for rank in range(8)]
    assert max(load) == pytest.approx(min(load), rel=1e-12)
    assert assign_by_cost(costs, 8) == owners  # deterministic
    assert assign_by_cost([3.0, 3.0, 3.0], 2) == [0, 1, 0]  # ties: lower unit first, lower rank first


def test_split_runs_follows_the_single_gpu_rule() -> None:
    assert split_runs([4, 4, None, 4, 9, 1], 8) == [[0, 1], [3], [4], [5]]
    assert split_runs([None, None], 8) == []
    assert split_runs([100], 8) == [[0]]  # an oversized entry still runs, alone
    assert split_runs([3, 3, 3], 9) == [[0, 1, 2]]
    assert shard_range(128256 * 4096, 3, 8) == (3 * 65667072, 4 * 65667072)


def _exchange_worker(rank: int, world: int, port: int, failures) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, k, cols = 48, 12, 40
        counts = [3, 1]  # rank 0 contributes a run of 3 blocks, rank 1 a run of 1
        plans = [_matrix_step.exchange_plan(c, rows, k, cols, True) for c in counts]
        slot = max(_workspace.layout(p)[1] for p in plans)
        arena = torch.zeros(slot + 4096, dtype=torch.uint8)
        mine = _workspace.views(arena, plans[rank])
        mine["x"].fill_(1.0 + rank)
        mine["rowmap"].copy_(torch.arange(counts[rank] * rows, dtype=torch.int32).view(counts[rank], rows) + 1000 * rank)
        mine["denom"].fill_(0.5 + rank)
        mine["scale"].fill_(-0.25 - rank)
        recv = torch.empty(slot * world, dtype=torch.uint8)
        dist.all_gather_into_tensor(recv, arena[:slot])
        for src in range(world):
            got = _workspace.views(recv, plans[src], base=src * slot)
            assert got["x"].shape == (counts[src], k, 40) and got["x"].dtype == torch.bfloat16
            assert bool((got["x"] == 1.0 + src).all())
            assert int(got["rowmap"][0, 5]) == 5 + 1000 * src and got["rowmap"].shape == (counts[src], rows)
            assert bool((got["denom"] == 0.5 + src).all()) and got["denom"].numel() == counts[src] * k
            assert bool((got["scale"] == -0.25 - src).all()) and got["scale"].numel() == counts[src]
        # in-place gather of a cut AdamW tensor: every rank ends with every range
        whole = torch.full((10,), -1.0)
        start, stop = shard_range(10, rank, world)
        whole[start:stop] = float(rank)
        dist.all_gather_into_tensor(whole, whole[start:stop].clone())
        assert whole.tolist() == [0.0] * 5 + [1.0] * 5
    except Exception as exc:  # reported to the parent
        failures.put(f"rank {rank}: {exc!r}")
    finally:
        dist.destroy_process_group()


def test_two_ranks_exchange_run_results_over_gloo() -> None:
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_exchange_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert failures.empty(), failures.get()


def test_cut_predicate() -> None:
    from dionw_b200.distributed import ADAMW_SHARD_MIN_ELEMENTS, is_cut

    big = ADAMW_SHARD_MIN_ELEMENTS
    assert not is_cut(big, 1, True)                      # one rank: nothing is cut
    assert is_cut(big, 8, True) and is_cut(big, 8, True, multiple=4)
    assert not is_cut(big - 8, 8, True)                  # too small
    assert not is_cut(big + 4, 8, True)                  # does not divide into 8 ranges
    assert is_cut(big + 8, 8, True) and not is_cut(big + 8, 8, True, multiple=4)   # ranges not 16-byte aligned
    assert not is_cut(big, 8, False)                     # not contiguous
    assert [shard_range(64, r, 4) for r in range(4)] == [(0, 16), (16, 32), (32, 48), (48, 64)]


def _ema_shard_worker(rank: int, world: int, port: int, failures) -> None:
    """The EMA range helpers of ``ShardedDion`` on CPU tensors over gloo (no kernel involved)."""
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from dionw_b200 import distributed
        from dionw_b200.distributed import ShardedDion

        distributed.ADAMW_SHARD_MIN_ELEMENTS = 64
        opt = ShardedDion.__new__(ShardedDion)
        opt._dist, opt._pg, opt._world, opt._rank = dist, None, world, rank
        gen = torch.Generator().manual_seed(0)
        big = torch.randn(16, 8, generator=gen)           # 128 elements: cut into two ranges of 64
        small = torch.randn(5, 3, generator=gen)          # whole on every rank
        assert opt._ema_is_cut(big) and not opt._ema_is_cut(small)
        view = opt._ema_view(big)
        assert view.shape == (64,) and view.data_ptr() == big.view(-1)[64 * rank:].data_ptr()
        assert opt._ema_view(small) is small
        # a rank's shadow range, gathered into the reference layout
        shard = view.clone() * 2.0
        whole = opt._gather_shadow(big, shard)
        assert whole.shape == big.shape and torch.equal(whole, big * 2.0)
        # a loaded full shadow is cut back to this rank's range; a range stays a range
        assert torch.equal(opt._loaded_shadow_share(big, whole), shard)
        assert opt._loaded_shadow_share(big, shard) is shard
        assert opt._loaded_shadow_share(small, small) is small
        # swap: every replica receives all ranges; restore brings the live values back
        live = big.clone()
        kept = opt._swap_in(big, shard)
        assert torch.equal(big, live * 2.0) and torch.equal(kept, live.view(-1)[64 * rank: 64 * rank + 64])
        opt._swap_out(big, kept)
        assert torch.equal(big, live)
    except Exception as exc:  # reported to the parent
        import traceback
        failures.put(f"rank {rank}: {exc!r}\n{traceback.format_exc()}")
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_ema_ranges_gather_and_swap_over_gloo() -> None:
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_ema_shard_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert failures.empty(), failures.get()
    assert all(p.exitcode == 0 for p in procs)


def test_bucket_order_puts_the_costliest_second() -> None:
    """Rounds go by cost; with three or more buckets the costliest goes second so that its gather,
    the largest of the step, is followed by a weight update and a round before it is needed."""
    from dionw_b200.distributed import bucket_order

    costs = [3.2e12, 88.0e12, 0.13e12, 3.7e12]          # q/o, gate/up, k/v, down at the Llama-3-8B shapes
    assert bucket_order(costs, costliest_second=False) == [1, 3, 0, 2]
    assert bucket_order(costs, costliest_second=True) == [3, 1, 0, 2]
    assert bucket_order([5.0, 9.0], costliest_second=True) == [1, 0]     # two buckets: plain order
    assert bucket_order([2.0, 2.0, 2.0], costliest_second=False) == [0, 1, 2]
    assert bucket_order([], costliest_second=True) == []
