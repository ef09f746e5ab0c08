"""``ShardedDion`` on 2 GPUs against single-GPU ``Dion``: same bits in the weights after
every step, the same checkpoint, and a resume from it.  Skipped with fewer than 2 GPUs."""

from __future__ import annotations

import os

import pytest
import torch
import torch.multiprocessing as mp
from torch import nn

pytestmark = pytest.mark.gpu

SHAPES = [(128, 256)] * 5 + [(512, 128)] * 3 + [(96, 96)] * 2


def _model(device) -> nn.Module:
    torch.manual_seed(0)
    net = nn.Module()
    net.mats = nn.ParameterList([nn.Parameter(torch.randn(s) * 0.02) for s in SHAPES])
    net.big = nn.Embedding(4096, 512)          # 2 M elements: cut into per-rank ranges
    net.norm = nn.Parameter(torch.randn(256) * 0.02)
    return net.to(device)


def _grads(net, step: int) -> None:
    gen = torch.Generator().manual_seed(100 + step)
    for i, p in enumerate(net.parameters()):
        p.grad = None if (step == 1 and i == 2) else (torch.randn(p.shape, generator=gen) * 1e-3).to(p.device)


def _worker(rank: int, world: int, port: int, failures, overlap: bool = False) -> None:
    import torch.distributed as dist

    import dionw_b200 as dionw
    from dionw_b200.distributed import ShardedDion

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import dionw_b200.optimizer as optimizer_module
        optimizer_module.MAX_RUN_ELEMENTS = 3 * 32 * 256  # several rounds per bucket, uneven run lengths

        def build(cls, **kw):
            net = _model(device)
            groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=128)
            return net, cls(groups, lr=3e-4, weight_decay=0.05, **kw)

        single_net, single = build(dionw.Dion)
        sharded_net, sharded = build(ShardedDion)
        if overlap:   # the rounds on a high-priority stream, the weight updates beside them on another
            sharded.overlap_apply = True
            sharded.round_elements = 2 * 32 * 256
        owners = sharded.owners()
        assert set(range(world)) == set(owners.values())
        for step in range(3):
            _grads(single_net, step)
            _grads(sharded_net, step)
            single.step()
            sharded.step()
            for a, b in zip(single_net.parameters(), sharded_net.parameters()):
                assert torch.equal(a, b), f"step {step}: weights differ"
        # state lives with the owner only
        for p, owner in owners.items():
            assert ("momentum" in sharded.state[p]) == (owner == rank)
        assert sharded.state[sharded_net.big.weight]["exp_avg"].numel() == 4096 * 512 // world
        # the gathered checkpoint equals the single-GPU one
        want, got = single.state_dict(), sharded.state_dict()
        assert want["param_groups"] == got["param_groups"]
        assert set(want["state"]) == set(got["state"])
        for index, entry in want["state"].items():
            for key, value in entry.items():
                assert torch.equal(value, got["state"][index][key]), (index, key)
        # resume: a fresh sharded optimizer loaded from it continues identically
        resumed_net, resumed = build(ShardedDion)
        resumed_net.load_state_dict(sharded_net.state_dict())
        resumed.load_state_dict({**got, "state": {i: {k: v.clone() for k, v in e.items()}
                                                  for i, e in got["state"].items()}})
        for net, opt in ((single_net, single), (resumed_net, resumed)):
            _grads(net, 3)
            opt.step()
        for a, b in zip(single_net.parameters(), resumed_net.parameters()):
            assert torch.equal(a, b), "resumed weights differ"
        torch.cuda.synchronize()
    except Exception as exc:  # reported to the parent
        import traceback
        failures.put(f"rank {rank}: {exc!r}\n{traceback.format_exc()}")
    finally:
        dist.destroy_process_group()


def _ema_worker(rank: int, world: int, port: int, failures, ema_device: str) -> None:
    import torch.distributed as dist

    import dionw_b200 as dionw
    from dionw_b200.distributed import ShardedDion

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        config = dionw.EMAConfig(decay=0.9, device=dionw.EMADevice(ema_device), update_every_n_steps=1)

        def build(cls):
            net = _model(device)
            net.wide = nn.Parameter(torch.randn(1024, 1024, generator=torch.Generator().manual_seed(5)).to(device) * 0.02)
            groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=128)
            return net, cls(groups, lr=3e-4, weight_decay=0.05, ema=config)

        single_net, single = build(dionw.Dion)
        sharded_net, sharded = build(ShardedDion)
        for step in range(3):
            _grads(single_net, step)
            _grads(sharded_net, step)
            single.step()
            sharded.step()
        # large parameters keep this rank's range of the shadow only, small ones the whole
        for name in ("wide", "big.weight"):
            p = dict(sharded_net.named_parameters())[name]
            shadow = sharded.state[p]["ema_shadow"]
            assert shadow.numel() == p.numel() // world, name
            assert shadow.is_cuda == (ema_device == "gpu")
        assert sharded.state[sharded_net.norm]["ema_shadow"].shape == sharded_net.norm.shape
        # the gathered checkpoint equals the single-GPU one, shadows included
        want, got = single.state_dict(), sharded.state_dict()
        assert want["_ema_step_count"] == got["_ema_step_count"] == 3
        assert set(want["state"]) == set(got["state"])
        for index, entry in want["state"].items():
            assert set(entry) == set(got["state"][index]), index
            for key, value in entry.items():
                mine = got["state"][index][key]
                if isinstance(value, torch.Tensor):
                    assert value.device == mine.device and value.shape == mine.shape, (index, key)
                    assert torch.equal(value, mine), (index, key)
                else:
                    assert value == mine, (index, key)
        # evaluation weights: swap (a collective), compare, restore
        live = [p.detach().clone() for p in sharded_net.parameters()]
        assert single.swap_ema_weights() and sharded.swap_ema_weights()
        for a, b in zip(single_net.parameters(), sharded_net.parameters()):
            assert torch.equal(a, b), "swapped weights differ"
        assert sharded.ema_weights_swapped
        single.restore_non_ema_weights()
        sharded.restore_non_ema_weights()
        for a, b in zip(live, sharded_net.parameters()):
            assert torch.equal(a, b), "restored weights differ"
        # resume from the gathered checkpoint and continue identically
        resumed_net, resumed = build(ShardedDion)
        resumed_net.load_state_dict(sharded_net.state_dict())
        resumed.load_state_dict({**got, "state": {i: {k: (v.clone() if isinstance(v, torch.Tensor) else v)
                                                      for k, v in e.items()} for i, e in got["state"].items()}})
        wide = resumed.state[resumed_net.wide]["ema_shadow"]
        assert wide.numel() == 1024 * 1024 // world and wide.is_cuda == (ema_device == "gpu")
        for net, opt in ((single_net, single), (resumed_net, resumed)):
            _grads(net, 3)
            opt.step()
        want, got = single.state_dict(), resumed.state_dict()
        for index, entry in want["state"].items():
            for key, value in entry.items():
                if isinstance(value, torch.Tensor):
                    assert torch.equal(value, got["state"][index][key]), ("resumed", index, key)
        # per-rank checkpoint: saved and loaded without any collective, through a file per rank
        import io
        import pytest as _pytest
        from dionw_b200.distributed import SHARD_KEY
        buffer = io.BytesIO()
        torch.save(resumed.sharded_state_dict(), buffer)
        buffer.seek(0)
        mine = torch.load(buffer, weights_only=False)
        assert mine[SHARD_KEY]["rank"] == rank and mine[SHARD_KEY]["world"] == world
        again_net, again = build(ShardedDion)
        again_net.load_state_dict(resumed_net.state_dict())
        with _pytest.raises(ValueError, match="rank"):
            again.load_sharded_state_dict({**mine, SHARD_KEY: {**mine[SHARD_KEY], "rank": 1 - rank}})
        with _pytest.raises(ValueError, match="per-rank"):
            again.load_sharded_state_dict(got)
        again.load_sharded_state_dict(mine)
        for net, opt in ((single_net, single), (again_net, again)):
            _grads(net, 4)
            opt.step()
        for a, b in zip(single_net.parameters(), again_net.parameters()):
            assert torch.equal(a, b), "weights after the per-rank resume differ"
        want, got = single.state_dict(), again.state_dict()
        assert want["_ema_step_count"] == got["_ema_step_count"] == 5
        for index, entry in want["state"].items():
            for key, value in entry.items():
                if isinstance(value, torch.Tensor):
                    assert torch.equal(value, got["state"][index][key]), ("per-rank resume", index, key)
        torch.cuda.synchronize()
    except Exception as exc:  # reported to the parent
        import traceback
        failures.put(f"rank {rank}: {exc!r}\n{traceback.format_exc()}")
    finally:
        dist.destroy_process_group()


def _decay_job_worker(rank: int, world: int, port: int, failures) -> None:
    """Blocks whose products are long enough to carry the round's decay job (K >= 1536): the sharded
    step with the job equals single-GPU ``Dion`` bit for bit, and the job did take rows."""
    import torch.distributed as dist

    import dionw_b200 as dionw
    from dionw_b200 import _workspace
    from dionw_b200.distributed import ShardedDion

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        def build(cls, **kw):
            torch.manual_seed(3)
            net = nn.Module()
            net.tall = nn.ParameterList([nn.Parameter(torch.randn(4096, 2048) * 0.02) for _ in range(3)])
            net.wide = nn.ParameterList([nn.Parameter(torch.randn(1024, 4096) * 0.02) for _ in range(2)])
            net.norm = nn.Parameter(torch.randn(256) * 0.02)
            net = net.to(device)
            groups, _ = dionw.param_groups(net, fraction=0.25)
            return net, cls(groups, lr=3e-4, weight_decay=0.05, **kw)

        single_net, single = build(dionw.Dion)
        sharded_net, sharded = build(ShardedDion, fused_decay=True)
        assert sharded.fused_decay
        taken = 0
        for step in range(3):
            gen = torch.Generator().manual_seed(200 + step)
            for a, b in zip(single_net.parameters(), sharded_net.parameters()):
                g = (torch.randn(a.shape, generator=gen) * 1e-3).to(device)
                a.grad, b.grad = g.clone(), g.clone()
            single.step()
            sharded.step()
            torch.cuda.synchronize()
            for a, b in zip(single_net.parameters(), sharded_net.parameters()):
                assert torch.equal(a, b), f"step {step}: weights differ"
            for parity in (0, 1):
                job = _workspace._arenas.get((device, f"decayjob{parity}"))
                if job is not None:
                    taken += int(job[20:24].view(torch.int32))
        assert taken > 0, "no product took a row of a decay job"
        want, got = single.state_dict(), sharded.state_dict()
        for index, entry in want["state"].items():
            for key, value in entry.items():
                assert torch.equal(value, got["state"][index][key]), (index, key)
    except Exception as exc:  # reported to the parent
        import traceback
        failures.put(f"rank {rank}: {exc!r}\n{traceback.format_exc()}")
    finally:
        dist.destroy_process_group()


def _run_two_ranks(target, *extra) -> None:
    _run_ranks(2, target, *extra)


def _run_ranks(world: int, target, *extra) -> None:
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=target, args=(r, world, port, failures, *extra)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    assert failures.empty(), failures.get()
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("overlap", [False, True])
def test_sharded_step_equals_single_gpu_step(overlap) -> None:
    _run_two_ranks(_worker, overlap)


def test_decay_job_in_a_group_of_one_equals_single_gpu_step() -> None:
    _run_ranks(1, _decay_job_worker)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_decay_job_on_two_gpus_equals_single_gpu_step() -> None:
    _run_two_ranks(_decay_job_worker)


@pytest.mark.parametrize("overlap", [False, True])
def test_sharded_step_in_a_group_of_one_equals_single_gpu_step(overlap) -> None:
    """The sharded step's own machinery -- rounds, alternating arenas, one weight-update launch per
    round, the gathered checkpoint, the resume -- on ONE GPU, in a process group of one: same bits
    as ``Dion``, in line and with the updates overlapped on a second stream."""
    _run_ranks(1, _worker, overlap)


@pytest.mark.parametrize("ema_device", ["gpu", "cpu"])
def test_sharded_ema_and_per_rank_checkpoints_in_a_group_of_one(ema_device) -> None:
    """The EMA of ``ShardedDion``, its gathered checkpoint, the evaluation swap, the resume and the
    per-rank checkpoint files (saved and loaded without a collective, refused for another rank) on
    ONE GPU in a process group of one, against ``Dion``."""
    _run_ranks(1, _ema_worker, ema_device)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("ema_device", ["gpu", "cpu"])
def test_sharded_ema_equals_single_gpu_ema(ema_device) -> None:
    """Each rank averages its element range of the large parameters; gathered, the shadows,
    the swapped-in evaluation weights and a resumed run equal the single-GPU optimizer's."""
    _run_two_ranks(_ema_worker, ema_device)
