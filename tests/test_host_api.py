"""Host-side behaviour that needs no GPU: EMA schedules, option enums, key strings,
constructor and checkpoint-structure errors (reference: tests/test_ema.py:141-205,
tests/test_optimizer.py:456-469, :753-798)."""

from __future__ import annotations

import pytest
import torch
from torch import nn

import dionw_b200 as dionw
from dionw_b200 import EMAConfig, EMASchedule, _keys
from dionw_b200.optimizer import _fill_legacy_keys, _require_group, _require_same_structure


def test_key_strings_are_the_checkpoint_format() -> None:
    assert _keys.ROUTE_KEY == "dion_route" and _keys.FRACTION_KEY == "fraction"
    assert _keys.STRUCTURAL_KEYS == (
        "dion_route", "fraction", "num_heads", "newton_schulz", "row_normalization", "momentum_form")
    assert (_keys.MOMENTUM_STATE, _keys.VARIANCE_STATE) == ("momentum", "variance")
    assert (_keys.EXP_AVG_STATE, _keys.EXP_AVG_SQ_STATE, _keys.ADAMW_STEP_STATE) == (
        "exp_avg", "exp_avg_sq", "adamw_step")
    assert _keys.EMA_STEP_COUNT_KEY == "_ema_step_count"
    assert _keys.EMA_SCRATCH_KEYS == ("ema_pending", "ema_tmp_cpu", "ema_event")
    assert [k.value for k in dionw.NewtonSchulz] == [
        "polar_express", "polar_express_triton", "gram", "keller", "keller_triton"]
    assert dionw.DION3_UPDATE.newton_schulz is dionw.NewtonSchulz.GRAM
    assert dionw.MUON_UPDATE.momentum_form is dionw.MomentumForm.NESTEROV
    assert dionw.MUON_UPDATE.row_normalization is dionw.RowNormalization.NONE


def test_ema_schedules() -> None:
    assert EMAConfig().schedule is EMASchedule.CONSTANT
    assert EMAConfig(decay=0.99).decay_at_step(10**6) == 0.99
    ramp = EMAConfig(decay=0.9, decay_final=0.99, decay_ramp_steps=10)
    assert ramp.schedule is EMASchedule.LINEAR_RAMP
    assert ramp.decay_at_step(0) == 0.9
    assert ramp.decay_at_step(5) == pytest.approx(0.945)
    assert ramp.decay_at_step(50) == pytest.approx(0.99)
    power = EMAConfig(decay=0.9999, power_gamma=6.94)
    assert power.schedule is EMASchedule.POWER
    assert power.decay_at_step(0) == 0.0
    assert power.decay_at_step(1) == 0.0
    assert power.decay_at_step(100) == pytest.approx((1 - 1 / 100) ** 7.94)
    assert power.decay_at_step(10**9) == 0.9999
    with pytest.raises(ValueError, match="non-negative"):
        power.decay_at_step(-1)


@pytest.mark.parametrize("kwargs,match", [
    ({"update_every_n_steps": 0}, "update_every_n_steps must be positive"),
    ({"start_step": -1}, "start_step must be non-negative"),
    ({"decay": 1.0}, r"decay must be in \[0, 1\)"),
    ({"decay_final": 0.5}, "set together"),
    ({"decay_ramp_steps": 5}, "set together"),
    ({"decay_final": 1.5, "decay_ramp_steps": 5}, "decay_final must be"),
    ({"decay_final": 0.5, "decay_ramp_steps": 0}, "decay_ramp_steps must be positive"),
    ({"power_gamma": 1.0, "decay_final": 0.5, "decay_ramp_steps": 5}, "exclusive"),
    ({"power_gamma": 0.0}, "power_gamma must be positive"),
])
def test_ema_config_validation(kwargs, match) -> None:
    with pytest.raises(ValueError, match=match):
        EMAConfig(**kwargs)


def _group(**extra):
    base = {"params": [nn.Parameter(torch.zeros(16, 16))], "dion_route": "matrix", "fraction": 1.0,
            "num_heads": None, "newton_schulz": "gram", "row_normalization": "normuon",
            "momentum_form": "heavy_ball", "lr": 1e-3, "weight_decay": 0.0}
    base.update(extra)
    return base


def test_group_validation_messages() -> None:
    _require_group(_group())
    broken = _group()
    del broken["dion_route"]
    with pytest.raises(TypeError, match="dionw.param_groups"):
        _require_group(broken)
    with pytest.raises(ValueError, match=r"fraction must be in \(0, 1\]"):
        _require_group(_group(fraction=0.0))
    with pytest.raises(ValueError, match="Nesterov momentum needs every row"):
        _require_group(_group(fraction=0.5, momentum_form="nesterov"))
    with pytest.raises(ValueError, match="route it to AdamW"):
        _require_group(_group(params=[nn.Parameter(torch.zeros(4))]))
    with pytest.raises(ValueError, match="does not divide"):
        _require_group(_group(num_heads=5))
    with pytest.raises(ValueError, match="lr and weight_decay"):
        _require_group(_group(lr=-1.0))
    with pytest.raises(ValueError):
        _require_group(_group(newton_schulz="nope"))


def test_constructor_refuses_cpu_and_non_float32_parameters() -> None:
    model = nn.Linear(16, 16)
    groups, _ = dionw.param_groups(model)
    with pytest.raises(ValueError, match="CUDA"):
        dionw.Dion(groups, lr=1e-3)
    with pytest.raises(ValueError, match=r"momentum must be in \[0, 1\)"):
        dionw.Dion(groups, lr=1e-3, momentum=1.0)
    with pytest.raises(ValueError, match="lr and weight_decay must be >= 0 and eps > 0"):
        dionw.Dion(groups, lr=1e-3, eps=0.0)


def test_checkpoint_structure_checks() -> None:
    current = [_group(), _group(dion_route="adamw")]
    same = [dict(g) for g in current]
    _require_same_structure(same, current)
    with pytest.raises(ValueError, match="has 1 param groups, the optimizer 2"):
        _require_same_structure(same[:1], current)
    changed = [dict(g) for g in current]
    changed[0]["fraction"] = 0.5
    with pytest.raises(ValueError, match="Dion state group 0 'fraction'"):
        _require_same_structure(changed, current)
    missing = [dict(g) for g in current]
    del missing[1]["newton_schulz"]
    with pytest.raises(ValueError, match="Dion state group 1 has no 'newton_schulz'"):
        _require_same_structure(missing, current)
    old = [{k: v for k, v in g.items() if k not in ("row_normalization", "momentum_form")} for g in current]
    filled = _fill_legacy_keys(old)
    assert filled[0]["row_normalization"] == "normuon" and filled[0]["momentum_form"] == "heavy_ball"
    _require_same_structure(filled, current)
    muon = [_group(row_normalization="none", momentum_form="nesterov"), current[1]]
    with pytest.raises(ValueError, match="row_normalization"):
        _require_same_structure(filled, muon)


# ---------------------------------------------------------------------------
# the pinned-host EMA worker (no GPU involved: host tensors, no event)
# ---------------------------------------------------------------------------
def test_cpu_ema_job_lerps_host_segments() -> None:
    from dionw_b200 import _native

    gen = torch.Generator().manual_seed(3)
    shadows = [torch.randn(n, generator=gen) for n in (1000, 7, 4096)]
    staged = [torch.randn(n, generator=gen) for n in (1000, 7, 4096)]
    expect = [s.clone() for s in shadows]
    expect[0].lerp_(staged[0], 0.25)
    expect[1].copy_(staged[1])          # first update of a shadow copies
    expect[2].lerp_(staged[2], 0.25)
    job = _native.CpuEmaJob(shadows, staged, [False, True, False], 0.25, None, 3)
    job.wait_copy()
    job.wait_update()
    assert job.done()
    job.close()
    for got, want in zip(shadows, expect):
        assert torch.equal(got, want)


def test_cpu_ema_worker_failure_reaches_the_waiting_thread() -> None:
    """Failure injected on the host: a segment whose staged buffer is missing.  The worker stores
    the error and releases both waits; the tracker re-raises it as the reference does
    (src/dionw/ema/_cpu_job.py:108-137, tracker.py:274-277)."""
    from dionw_b200 import _native
    from dionw_b200.ema.tracker import OptimizerIntegratedEMA

    class Missing:
        def data_ptr(self) -> int:
            return 0

        def numel(self) -> int:
            return 16

    shadow = torch.zeros(16)
    job = _native.CpuEmaJob([shadow], [Missing()], [False], 0.5, None, 2)
    with pytest.raises(RuntimeError, match="no shadow or no staged buffer"):
        job.wait_update()
    assert job.done()

    tracker = OptimizerIntegratedEMA.__new__(OptimizerIntegratedEMA)
    good = torch.ones(16)
    tracker._jobs = [_native.CpuEmaJob([shadow], [Missing()], [False], 0.5, None, 2),
                     _native.CpuEmaJob([good], [torch.zeros(16)], [False], 0.5, None, 2)]
    tracker._job_states = [{}, {}]
    with pytest.raises(RuntimeError, match="Asynchronous CPU EMA update failed"):
        tracker._finish_job()
    assert tracker._jobs == []
    assert torch.equal(good, torch.full((16,), 0.5))   # the other job of the update still ran to its end
    assert torch.equal(shadow, torch.zeros(16))


def test_snapshot_chunks_keep_order_and_balance() -> None:
    """The CPU EMA cuts a large snapshot into pieces so that the host averages one piece while the
    next one crosses the link: every parameter lands in exactly one piece, in order."""
    from dionw_b200.ema.tracker import OptimizerIntegratedEMA

    tracker = OptimizerIntegratedEMA.__new__(OptimizerIntegratedEMA)
    small = [(i, torch.empty(1000, device="meta")) for i in range(5)]
    assert tracker._snapshot_chunks(small) == [small]
    sizes = [1 << 22] * 9 + [1 << 25, 4096, 1 << 23]
    items = [(i, torch.empty(n, device="meta")) for i, n in enumerate(sizes)]
    chunks = tracker._snapshot_chunks(items)
    assert 1 < len(chunks) <= tracker.SNAPSHOT_CHUNKS
    assert [i for chunk in chunks for i, _ in chunk] == list(range(len(sizes)))
    assert all(chunk for chunk in chunks)
    one = [(0, torch.empty(1 << 26, device="meta"))]
    assert tracker._snapshot_chunks(one) == [one]


def test_step_scalar_table_layout_and_values() -> None:
    """The device table of step scalars: four slots per group, then ``-step_size`` per bucket, with the
    reference's formulas (src/dionw/_matrix_step.py:147-159 for the step size, :280 for the decay)."""
    import math

    from dionw_b200._buckets import Bucket
    from dionw_b200.optimizer import step_scalar_values

    groups = [{"lr": 3e-4, "weight_decay": 0.0}, {"lr": 1e-3, "weight_decay": 0.05}]
    empty = torch.zeros(0)
    selecting = Bucket(group_index=1, orthogonalize=None, params=[], slices=[], rows=14336, cols=4096,
                       selected_rows=3584, momentum=empty, variance=empty)
    full = Bucket(group_index=1, orthogonalize=None, params=[], slices=[], rows=768, cols=2304,
                  selected_rows=768, momentum=empty, variance=empty)

    class Elsewhere:   # a bucket another rank owns: only its group's decay factor matters
        group_index = 1

    values, base = step_scalar_values(groups, [selecting, Elsewhere(), full])
    assert base == 8 and len(values) == 11
    assert values[:4] == [3e-4, 0.0, 1.0, 0.0]
    assert values[4:8] == [1e-3, 0.05, 1.0 - 1e-3 * 0.05, 0.0]
    assert values[8] == -(1e-3 * 0.2 * math.sqrt(14336) * math.sqrt(4096 / 3584))
    assert values[9] == 0.0
    assert values[10] == -(1e-3 * 0.2 * math.sqrt(2304) * math.sqrt(768 / 768))
