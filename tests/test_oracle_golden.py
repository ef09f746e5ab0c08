"""The CPU oracle against outputs of the reference itself (tests/golden/*.npz).

These fixtures were written by ``tests/golden/make_golden.py`` from the
reference's own code; they are what pins the oracle.
"""

from __future__ import annotations

import pytest
import torch

from conftest import PUBLISHED_ROUNDING, load_golden, rel_l2, spectrum_matrix
from oracle import dion_oracle as oracle

MATS = ("mats.0", "mats.1", "mats.2")


def _run_oracle(gold: dict[str, torch.Tensor], fractions: dict[str, float], steps: int):
    weights = {n: gold[f"init.{n}"].clone() for n in (*MATS, "bias", "table.weight") if f"init.{n}" in gold}
    mats = [n for n in MATS if n in weights]
    opt = oracle.OracleDion(
        matrix=[(weights[n], fractions[n]) for n in mats],
        adamw=[(weights["bias"], 0.0), (weights["table.weight"], None)],
        lr=3e-4, weight_decay=0.05,
        orthogonalize=lambda m, eps: oracle.gram_newton_schulz(m, eps, eager_diagonal=True),  # CPU-written fixtures
    )
    torch.set_num_threads(1)
    for s in range(steps):
        opt.step([gold[f"grad{s}.{n}"] for n in mats],
                 [gold[f"grad{s}.bias"], gold[f"grad{s}.table.weight"]])
        yield s, weights, opt


def test_selected_rows_step_matches_reference() -> None:
    gold = load_golden("step_selected")
    fractions = {"mats.0": 0.25, "mats.1": 0.25, "mats.2": 0.25}
    for s, weights, opt in _run_oracle(gold, fractions, 3):
        # (64,192) x2 share a bucket; (128,64) is the second bucket.
        for b, bucket in enumerate(opt.buckets):
            assert torch.equal(bucket.last_index.squeeze(-1), gold[f"index{s}.{b}"])
        # The reference lists the selected rows in topk's order, the oracle in
        # ascending order: the fp16 iteration sees permuted rows, so weights
        # agree to the rounding of the iteration, not bit for bit.
        for n in MATS:
            assert rel_l2(weights[n], gold[f"w{s}.{n}"]) <= 5e-5
        assert rel_l2(opt.buckets[0].momentum[0], gold[f"state{s}.mats.0.momentum"]) <= 1e-6
        assert rel_l2(opt.buckets[0].momentum[1], gold[f"state{s}.mats.1.momentum"]) <= 1e-6
        assert rel_l2(opt.buckets[1].momentum[0], gold[f"state{s}.mats.2.momentum"]) <= 1e-6
        # Row variance averages o^2 over only 64-192 bf16 entries here, so the
        # permuted-row rounding noise of the iteration shows at a few 1e-3; at
        # the benchmark's 4096-column blocks it is far below 2e-3.
        assert rel_l2(opt.buckets[0].variance[0], gold[f"state{s}.mats.0.variance"]) <= 5e-3
        assert rel_l2(opt.buckets[1].variance[0], gold[f"state{s}.mats.2.variance"]) <= 5e-3
        assert rel_l2(weights["bias"], gold[f"w{s}.bias"]) <= 1e-6
        assert rel_l2(weights["table.weight"], gold[f"w{s}.table.weight"]) <= 1e-6


def test_full_row_step_matches_reference() -> None:
    gold = load_golden("step_full_rows")
    fractions = {n: 1.0 for n in MATS}
    for s, weights, opt in _run_oracle(gold, fractions, 3):
        for n in MATS:
            assert rel_l2(weights[n], gold[f"w{s}.{n}"]) <= 1e-6
        for bucket, n in zip(opt.buckets, MATS):
            assert rel_l2(bucket.momentum[0], gold[f"state{s}.{n}.momentum"]) <= 1e-6
            assert rel_l2(bucket.variance[0], gold[f"state{s}.{n}.variance"]) <= 2e-3


@pytest.mark.parametrize("tag", ["wide", "tall", "square", "odd"])
def test_gram_newton_schulz_matches_reference(tag: str) -> None:
    gold = load_golden("newton_schulz")
    torch.set_num_threads(1)
    ours = oracle.gram_newton_schulz(gold[f"{tag}.x"], 1e-8, eager_diagonal=True)   # the fixtures were written on the CPU
    assert ours.dtype == torch.bfloat16
    assert torch.equal(ours, gold[f"{tag}.gram"])


@pytest.mark.parametrize("tag", ["wide", "tall", "square", "odd"])
@pytest.mark.parametrize("kind,coeffs,safety", [
    ("polar_express_triton", oracle.POLAR_EXPRESS_COEFFS, 1.02),
    ("keller_triton", oracle.KELLER_COEFFS, 1.0),
])
def test_bf16_quintic_matches_reference(tag: str, kind: str, coeffs, safety: float) -> None:
    gold = load_golden("newton_schulz")
    torch.set_num_threads(1)
    ours = oracle.quintic_bf16(gold[f"{tag}.x"], 1e-8, coeffs, safety)
    assert rel_l2(ours.float(), gold[f"{tag}.{kind}"].float()) <= 1e-6


def test_gram_is_close_to_the_exact_polar_factor() -> None:
    """tests/test_newton_schulz.py:46-64 and :125-134 of the reference: < 0.2."""
    gold = load_golden("newton_schulz")
    for tag in ("wide", "tall", "square"):
        x = gold[f"{tag}.x"]
        assert rel_l2(oracle.gram_newton_schulz(x).float(), oracle.exact_polar(x)) < 0.2


def test_adamw_matches_torch_fused() -> None:
    gold = load_golden("adamw")
    p = gold["p0"].clone()
    m, v, step = torch.zeros_like(p), torch.zeros_like(p), torch.zeros(())
    for s in range(4):
        oracle.adamw_(p, gold[f"g{s}"], m, v, step, lr=3e-4, beta1=0.9, beta2=0.95,
                      weight_decay=0.05, eps=1e-8)
        assert rel_l2(p, gold[f"p{s + 1}"]) <= 1e-6
        assert rel_l2(m, gold[f"m{s + 1}"]) <= 1e-6
        assert rel_l2(v, gold[f"v{s + 1}"]) <= 1e-6


def test_ema_shadow_matches_reference() -> None:
    """Shadow = copy at the first due step, then lerp with decay 0.9."""
    gold = load_golden("step_ema")
    shadow = None
    for s in range(4):
        w = gold[f"w{s}.mats.0"]
        if shadow is None:
            shadow = w.clone()
        else:
            oracle.ema_lerp_(shadow, w, 0.9)
        assert torch.equal(shadow, gold[f"state{s}.mats.0.ema_shadow"])


def test_row_scores_order_is_the_documented_one() -> None:
    torch.manual_seed(0)
    m = torch.randn(5, 3000)
    s = oracle.row_scores(m)
    torch.testing.assert_close(s, m.abs().sum(-1), rtol=1e-5, atol=1e-3)
    # lane fold by hand for one row
    lanes = [0.0] * 1024
    import numpy as np
    row = np.abs(m[0].numpy()).astype(np.float32)
    acc = np.zeros(1024, dtype=np.float32)
    for start in range(0, 3000, 1024):
        chunk = row[start:start + 1024]
        acc[: len(chunk)] += chunk
    w = 1024
    while w > 1:
        w //= 2
        acc = acc[:w] + acc[w:2 * w]
    assert float(acc[0]) == float(s[0])


@pytest.mark.parametrize("name", sorted(PUBLISHED_ROUNDING))
def test_oracle_rounding_error_matches_the_published_table(name) -> None:
    """Known answers: the reference publishes the rounding error of its Gram iteration (distance to
    the fp64 polynomial) on five spectra.  The oracle, iterating in fp16 on the CPU, lands on them
    (the Gaussian case uses another random matrix than the published one, hence the wider margin)."""
    torch.set_num_threads(8)
    x = spectrum_matrix(name)
    target = oracle.polynomial_fp64(x, oracle.GRAM_COEFFS, 1.0, eps=1e-7)
    error = rel_l2(oracle.gram_newton_schulz(x, eps=1e-7), target)
    slack = 0.004 if name == "gaussian" else 0.003
    assert abs(error - PUBLISHED_ROUNDING[name]) < slack, error
    if name != "gaussian":
        bf16_polar = oracle.quintic_bf16(x, 1e-7, oracle.POLAR_EXPRESS_COEFFS, 1.02)
        polar_target = oracle.polynomial_fp64(x, oracle.POLAR_EXPRESS_COEFFS, 1.02, eps=1e-7)
        assert error < 0.08 and error < rel_l2(bf16_polar, polar_target)
