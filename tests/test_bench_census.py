"""The benchmark's algorithmic work (the numerators of its roofline figures) against the
hand-computed figures of the configurations it names."""

from __future__ import annotations

import pytest
import torch

import bench
import dionw_b200 as dionw


def _groups(config: str):
    model = bench.build_model(config, torch.device("meta"))
    routes = {} if model.lm_head is None else {model.lm_head.weight: dionw.Route(dionw.RouteKind.ADAMW)}
    return dionw.param_groups(model, routes=routes).groups


def test_llama3_8b_census() -> None:
    work = bench.census(_groups("llama3-8b"))
    assert work["matrix_elements"] == 32 * (2 * 4096 * 4096 + 2 * 1024 * 4096 + 3 * 14336 * 4096)   # 6.98 G
    assert work["selected_elements"] == work["matrix_elements"] / 4
    assert work["adamw_elements"] == 2 * 128256 * 4096 + 65 * 4096                                      # 1.05 G
    # 64 x (1024, 4096), 64 x (256, 4096), 64 x (3584, 4096), 32 x (1024, 14336): 95.0 TFLOP per step
    assert work["ns_flops"] == pytest.approx(95.0e12, rel=2e-3)
    assert work["ns_flops_executed"] / work["ns_flops"] == pytest.approx(0.71, abs=0.01)
    # 12 B per element accumulated, 10 per selected element packed, 8 + 2 applied, 28 per AdamW element
    assert work["bytes_accumulate"] == 12 * work["matrix_elements"]
    assert work["bytes_pack"] == 10 * work["selected_elements"]
    assert work["bytes_apply"] == 8 * work["matrix_elements"] + 2 * work["selected_elements"]
    assert work["bytes_adamw"] == 28 * work["adamw_elements"]
    total = work["bytes_accumulate"] + work["bytes_pack"] + work["bytes_apply"]
    assert total == pytest.approx(160.5e9, rel=2e-3)           # 20 E + 12 Es


def test_gpt2_small_census_takes_the_full_row_path() -> None:
    work = bench.census(_groups("gpt2-small"))
    assert work["matrix_elements"] == work["selected_elements"] == 12 * (768 * 2304 + 768 * 768 + 2 * 768 * 3072)
    assert work["ns_flops"] == pytest.approx(0.843e12, rel=2e-3)
    assert work["bytes_accumulate"] == 16 * work["matrix_elements"]
    assert work["adamw_elements"] == pytest.approx(39.4e6, rel=5e-3)


def test_single_matrix_and_70b_slice_census() -> None:
    one = bench.census(_groups("single-1024x4096"))
    assert one["matrix_elements"] == 1024 * 4096 and one["selected_elements"] == 256 * 4096
    assert one["adamw_elements"] == 4096
    assert one["ns_flops"] == pytest.approx(2.00e9, rel=5e-3)
    big = bench.census(_groups("llama3-70b-20layers"))
    assert big["ns_flops"] == pytest.approx(474.5e12, rel=2e-3)
    assert big["matrix_elements"] + big["adamw_elements"] == pytest.approx(18.16e9, rel=2e-3)


def test_cpu_arm_runs_the_single_matrix_workload_whole() -> None:
    """The reference arm's sample on the one workload it runs unscaled (config 1)."""
    base = bench.cpu_sample_step("single-1024x4096", steps=2, warmup=1)
    # the reference package itself where a copy of it sits under baseline/_ref, else the oracle port
    assert base["kind"] in ("reference", "port") and base["unit"] == "ms" and base["cores"] >= 1
    assert base["extrapolated"] is False and base["scale"] == {"matrix": 1.0, "adamw": 1.0}
    assert 0.0 < base["sample_ms"] <= base["value"] * 1.0001
    assert base["value"] == pytest.approx(base["sample_ms"], rel=1e-6)   # scale factors are 1
    assert "whole workload" in base["sample"]


def test_per_operand_newton_schulz_rows_are_split_out_of_the_stages() -> None:
    """``ns:<m>x<n>`` entries leave the stage dictionary (so that the stage sum still is the step) and
    come back as rows with executed and algorithmic rates."""
    stages = {"accumulate": 14.6, "newton_schulz": 59.2, "ns:3584x4096": 51.0, "ns:256x4096": 0.55}
    blocks = {"ns:3584x4096": 64 * 10, "ns:256x4096": 64 * 10}
    rows = bench.split_ns_shapes(stages, blocks, steps=10)
    assert set(stages) == {"accumulate", "newton_schulz"} and not blocks
    by_operand = {tuple(r["operand"]): r for r in rows}
    big = by_operand[(3584, 4096)]
    assert big["blocks"] == 64 and big["ms"] == 51.0
    assert big["executed_TFLOP/s"] == pytest.approx(64 * bench.flops_newton_schulz_executed(3584, 4096) / 51.0 / 1e9)
    assert big["algorithmic_TFLOP/s"] == pytest.approx(64 * bench.flops_newton_schulz(3584, 4096) / 51.0 / 1e9)
    assert big["executed_TFLOP/s"] < big["algorithmic_TFLOP/s"]


def test_a_sub_benchmark_that_prints_no_line_is_reported_not_raised() -> None:
    """The embedded arms (the reference's GPU step, the microbenchmark) run in processes of their own; one
    that fails leaves an ``unavailable`` entry with the reason instead of stopping the run."""
    result = bench.run_sub_bench(["--config", "no-such-config"], timeout=120)
    assert "unavailable" in result and "no JSON line" in result["unavailable"]
