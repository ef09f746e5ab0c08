"""``Dion.step()`` on the GPU against the reference's outputs (fixtures), the CPU
oracle at benchmark-shaped blocks, and the behaviours the reference's own
test-suite pins (tests/test_optimizer.py, tests/test_muon.py, tests/test_ema.py)."""

from __future__ import annotations

import io
import math
import sys

import pytest
import torch
from torch import nn

from conftest import GOLDEN, load_golden, rel_l2
from oracle import dion_oracle as oracle

import dionw_b200 as dionw
from dionw_b200 import EMAConfig, EMADevice, Route, RouteKind

sys.path.insert(0, str(GOLDEN))
from routing_models import StepNet  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _load_net(gold, shapes) -> StepNet:
    net = StepNet(shapes)
    with torch.no_grad():
        for name, p in net.named_parameters():
            p.copy_(gold[f"init.{name}"])
    return net.to(DEV)


def _set_grads(net, gold, s) -> None:
    for name, p in net.named_parameters():
        p.grad = gold[f"grad{s}.{name}"].to(DEV)


# ---------------------------------------------------------------------------
# against outputs of the reference itself
# ---------------------------------------------------------------------------
def test_selected_row_steps_match_reference_fixture() -> None:
    """Row sets exact; fp32-only state <= 1e-5; Newton-Schulz-dependent state within the
    bound these tiny blocks allow (variance averages only 64-192 bf16 entries per row)."""
    gold = load_golden("step_selected")
    shapes = [(64, 192), (64, 192), (128, 64)]
    net = _load_net(gold, shapes)
    groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=32)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05)
    for s in range(3):
        _set_grads(net, gold, s)
        opt.step()
        for name, p in net.named_parameters():
            tol = 2e-4 if name.startswith("mats") else 1e-5
            assert rel_l2(p, gold[f"w{s}.{name}"]) <= tol, (s, name)
            for key, value in opt.state[p].items():
                want = gold.get(f"state{s}.{name}.{key}")
                if want is None or not isinstance(value, torch.Tensor):
                    continue
                tol = 1e-2 if key == "variance" else 1e-5
                assert rel_l2(value, want) <= tol, (s, name, key)
        # the rows each block touched this step, read back from the decayed momentum
        for b, name in enumerate(["mats.0", "mats.1"]):
            assert _touched_rows(opt, net.mats[b]) == set(gold[f"index{s}.0"][b].tolist())
        assert _touched_rows(opt, net.mats[2]) == set(gold[f"index{s}.1"][0].tolist())


def _touched_rows(opt, param) -> set[int]:
    """Rows whose variance is non-zero have been selected at least once; for the
    per-step set compare the momentum's decayed rows instead."""
    return opt._last_rows[id(param)]


@pytest.fixture(autouse=True)
def _record_selected_rows(monkeypatch):
    """Record, per parameter, the rows the last run selected (from the kernels' own index buffer)."""
    from dionw_b200 import _matrix_step, _native

    real = _native.select_rows
    picked: dict[str, torch.Tensor] = {}

    def spy(scores, sumsq, k, index, rowmap, frob):
        real(scores, sumsq, k, index, rowmap, frob)
        picked["index"] = index

    real_step = _matrix_step.step_run

    def step_spy(bucket, positions, group, state):
        real_step(bucket, positions, group, state)
        if "index" in picked:
            start = bucket.slices[positions[0]].start
            rows = picked.pop("index").cpu()
            for i in positions:
                blocks = bucket.slices[i]
                owner = bucket.params[i]
                store = _ROWS.setdefault(id(owner), set())
                store.clear()
                if blocks.stop - blocks.start == 1:
                    store.update(rows[blocks.start - start].tolist())

    _ROWS.clear()
    monkeypatch.setattr(_native, "select_rows", spy)
    monkeypatch.setattr("dionw_b200.optimizer.step_run", step_spy)
    monkeypatch.setattr(dionw.Dion, "_last_rows", _ROWS, raising=False)
    yield


_ROWS: dict[int, set[int]] = {}


def test_full_row_steps_match_reference_fixture() -> None:
    gold = load_golden("step_full_rows")
    net = _load_net(gold, [(96, 160), (160, 96), (64, 64)])
    groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=1024)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05)
    for s in range(3):
        _set_grads(net, gold, s)
        opt.step()
        for name, p in net.named_parameters():
            assert rel_l2(p, gold[f"w{s}.{name}"]) <= (2e-4 if name.startswith("mats") else 1e-5)
            state = opt.state[p]
            if "momentum" in state:
                assert rel_l2(state["momentum"], gold[f"state{s}.{name}.momentum"]) <= 1e-5
                assert rel_l2(state["variance"], gold[f"state{s}.{name}.variance"]) <= 1e-2
            else:
                assert rel_l2(state["exp_avg"], gold[f"state{s}.{name}.exp_avg"]) <= 1e-5
                assert rel_l2(state["exp_avg_sq"], gold[f"state{s}.{name}.exp_avg_sq"]) <= 1e-5
                assert float(state["adamw_step"]) == s + 1


@pytest.mark.parametrize("device", [EMADevice.GPU, EMADevice.CPU])
def test_ema_steps_match_reference_fixture(device) -> None:
    gold = load_golden("step_ema")
    net = _load_net(gold, [(64, 96)])
    groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=1024)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05, ema=EMAConfig(decay=0.9, device=device))
    for s in range(4):
        _set_grads(net, gold, s)
        opt.step()
        opt.ema.flush_pending_updates()
        for name, p in net.named_parameters():
            shadow = opt.state[p]["ema_shadow"]
            assert shadow.device.type == ("cuda" if device is EMADevice.GPU else "cpu")
            assert rel_l2(shadow, gold[f"state{s}.{name}.ema_shadow"]) <= 2e-4
    assert opt.state_dict()["_ema_step_count"] == 4


# ---------------------------------------------------------------------------
# against the oracle at benchmark-shaped blocks
# ---------------------------------------------------------------------------
def _seeded(shape, scale, gen):
    return torch.randn(shape, generator=gen) * scale


def test_config1_ten_steps_match_oracle() -> None:
    """BASELINE config 1: W[1024, 4096] (Dion3, k = 256) + bias[4096] (AdamW), 10 steps.
    Row sets exact every step; W and variance rel-L2 <= 2e-3; momentum and AdamW state <= 1e-5."""
    gen = torch.Generator().manual_seed(0)
    w0, b0 = _seeded((1024, 4096), 0.02, gen), _seeded((4096,), 0.02, gen)
    net = nn.Module()
    net.weight = nn.Parameter(w0.clone())
    net.bias = nn.Parameter(b0.clone())
    net = net.to(DEV)
    groups, _ = dionw.param_groups(net)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05)
    w_ref, b_ref = w0.clone(), b0.clone()
    ref = oracle.OracleDion(matrix=[(w_ref, 0.25)], adamw=[(b_ref, 0.0)], lr=3e-4, weight_decay=0.05)
    torch.set_num_threads(8)
    for s in range(10):
        gw, gb = _seeded((1024, 4096), 1e-3, gen), _seeded((4096,), 1e-3, gen)
        net.weight.grad, net.bias.grad = gw.to(DEV), gb.to(DEV)
        opt.step()
        ref.step([gw], [gb])
        assert opt._last_rows[id(net.weight)] == set(ref.buckets[0].last_index[0, :, 0].tolist()), s
        assert rel_l2(net.weight, w_ref) <= 2e-3
        assert rel_l2(opt.state[net.weight]["momentum"], ref.buckets[0].momentum[0]) <= 1e-5
        assert rel_l2(opt.state[net.weight]["variance"], ref.buckets[0].variance[0]) <= 2e-3
        assert rel_l2(net.bias, b_ref) <= 1e-5
        assert rel_l2(opt.state[net.bias]["exp_avg_sq"], ref.adam_state[0].exp_avg_sq) <= 1e-5
    # the update itself (not just W, which is dominated by the unchanged rows)
    assert rel_l2(net.weight.cpu() - w0, w_ref - w0) <= 5e-3


@pytest.mark.parametrize("full_products", [False, True])
def test_gate_up_shaped_block_matches_oracle(monkeypatch, full_products) -> None:
    """BASELINE config 3's dominant block: 14336 x 4096, k = 3584 (operand 3584 x 4096, the
    least well conditioned shape of the set).  Two steps against the CPU oracle: row sets exact,
    W and variance rel-L2 <= 2e-3, momentum <= 1e-5 -- with the symmetric m x m products
    mirrored (the default) and computed in full."""
    import dataclasses

    from dionw_b200 import _native, newton_schulz

    if full_products:
        gram = dionw.NewtonSchulz.GRAM
        monkeypatch.setitem(newton_schulz._NATIVE, gram,
                            dataclasses.replace(newton_schulz._NATIVE[gram], code=_native.NS_GRAM_FULL))
    gen = torch.Generator().manual_seed(3)
    w0 = _seeded((14336, 4096), 0.02, gen)
    net = nn.Module()
    net.weight = nn.Parameter(w0.clone())
    net = net.to(DEV)
    opt = dionw.Dion(dionw.param_groups(net).groups, lr=3e-4, weight_decay=0.05)
    w_ref = w0.clone()
    ref = oracle.OracleDion(matrix=[(w_ref, 0.25)], adamw=[], lr=3e-4, weight_decay=0.05)
    torch.set_num_threads(max(1, (torch.get_num_threads(), 16)[1]))
    for s in range(2):
        g = _seeded((14336, 4096), 1e-3, gen)
        net.weight.grad = g.to(DEV)
        opt.step()
        ref.step([g], [])
        assert opt._last_rows[id(net.weight)] == set(ref.buckets[0].last_index[0, :, 0].tolist()), s
    update_error = rel_l2(net.weight.cpu() - w0, w_ref - w0)
    variance_error = rel_l2(opt.state[net.weight]["variance"], ref.buckets[0].variance[0])
    print(f"full_products={full_products}: W rel-L2 {rel_l2(net.weight, w_ref):.2e}, update rel-L2 "
          f"{update_error:.2e}, variance rel-L2 {variance_error:.2e}")
    assert rel_l2(net.weight, w_ref) <= 2e-3
    assert rel_l2(opt.state[net.weight]["momentum"], ref.buckets[0].momentum[0]) <= 1e-5
    # Two fp16 evaluations of the same product schedule (tensor cores here, the CPU's GEMM in the
    # oracle) leave row norms of this nearly square operand 1-2e-3 apart, with the products in
    # full exactly as much as mirrored (3.3e-3 on the variance either way).  That spread is between
    # the two machines' GEMMs: against the reference's own step on the GPU the same block is within
    # 1.6e-3 (mirrored) and 0.9e-3 (full), which is what the 2e-3 of the specification is checked
    # against (tests/test_reference_gpu.py, the large blocks).  The bound here is the measured spread
    # with a fifth of margin.
    assert variance_error <= 4e-3
    assert update_error <= 1e-2


def test_70b_shaped_blocks_with_gpu_ema_match_oracle() -> None:
    """BASELINE config 5's attention blocks (d = 8192): k/v 1024 x 8192 (k = 256) and q/o 8192 x 8192
    (k = 2048), RMSNorm[8192] through AdamW, GPU EMA with decay 0.9999.  Two steps against the CPU
    oracle: row sets exact, W and variance <= 2e-3 (5e-3 on the variance of the less well conditioned
    2048 x 8192 operand), momentum, AdamW and EMA shadows <= 1e-5."""
    gen = torch.Generator().manual_seed(8)
    shapes = {"kv": (1024, 8192), "qo": (8192, 8192)}
    init = {n: _seeded(s, 0.02, gen) for n, s in shapes.items()}
    norm0 = _seeded((8192,), 0.02, gen)
    net = nn.Module()
    net.kv, net.qo = nn.Parameter(init["kv"].clone()), nn.Parameter(init["qo"].clone())
    net.norm = nn.Parameter(norm0.clone())
    net = net.to(DEV)
    opt = dionw.Dion(dionw.param_groups(net).groups, lr=3e-4, weight_decay=0.05,
                     ema=dionw.EMAConfig(decay=0.9999, device=dionw.EMADevice.GPU))
    refs = {n: init[n].clone() for n in shapes}
    norm_ref = norm0.clone()
    ref = oracle.OracleDion(matrix=[(refs["kv"], 0.25), (refs["qo"], 0.25)], adamw=[(norm_ref, 0.0)],
                            lr=3e-4, weight_decay=0.05)
    shadows = {n: None for n in (*shapes, "norm")}
    torch.set_num_threads(16)
    for s in range(2):
        grads = {n: _seeded(shape, 1e-3, gen) for n, shape in shapes.items()}
        gnorm = _seeded((8192,), 1e-3, gen)
        net.kv.grad, net.qo.grad, net.norm.grad = grads["kv"].to(DEV), grads["qo"].to(DEV), gnorm.to(DEV)
        opt.step()
        ref.step([grads["kv"], grads["qo"]], [gnorm])
        for name, value in (("kv", refs["kv"]), ("qo", refs["qo"]), ("norm", norm_ref)):
            if shadows[name] is None:
                shadows[name] = value.clone()          # the first update copies
            else:
                oracle.ema_lerp_(shadows[name], value, 0.9999)
        for i, name in enumerate(("kv", "qo")):
            param = getattr(net, name)
            assert opt._last_rows[id(param)] == set(ref.buckets[i].last_index[0, :, 0].tolist()), (name, s)
    for i, name in enumerate(("kv", "qo")):
        param = getattr(net, name)
        assert rel_l2(param, refs[name]) <= 2e-3
        assert rel_l2(param.detach().cpu() - init[name], refs[name] - init[name]) <= 1e-2
        assert rel_l2(opt.state[param]["momentum"], ref.buckets[i].momentum[0]) <= 1e-5
        assert rel_l2(opt.state[param]["variance"], ref.buckets[i].variance[0]) <= (2e-3 if name == "kv" else 5e-3)
        assert rel_l2(opt.state[param]["ema_shadow"], shadows[name]) <= 1e-5
    assert rel_l2(net.norm, norm_ref) <= 1e-5
    assert rel_l2(opt.state[net.norm]["ema_shadow"], shadows["norm"]) <= 1e-5


def test_gpt2_shaped_layer_matches_oracle() -> None:
    """BASELINE config 2's block shapes (min dim 768 < 1024: every row, path of
    accumulate_copy_decay), one layer, 3 steps."""
    gen = torch.Generator().manual_seed(1)
    shapes = [(768, 2304), (768, 768), (768, 3072), (3072, 768)]
    net = StepNet(shapes, vec=768)
    with torch.no_grad():
        for p in net.parameters():
            p.copy_(_seeded(p.shape, 0.02, gen))
    start = {n: p.detach().clone() for n, p in net.named_parameters()}
    net = net.to(DEV)
    groups, _ = dionw.param_groups(net)
    opt = dionw.Dion(groups, lr=3e-4, weight_decay=0.05)
    ws = [start[f"mats.{i}"].clone() for i in range(4)]
    bias, table = start["bias"].clone(), start["table.weight"].clone()
    ref = oracle.OracleDion(matrix=[(w, 1.0) for w in ws], adamw=[(bias, 0.0), (table, None)], lr=3e-4,
                            weight_decay=0.05)
    torch.set_num_threads(8)
    for _ in range(3):
        grads = {n: _seeded(p.shape, 1e-3, gen) for n, p in net.named_parameters()}
        for n, p in net.named_parameters():
            p.grad = grads[n].to(DEV)
        opt.step()
        ref.step([grads[f"mats.{i}"] for i in range(4)], [grads["bias"], grads["table.weight"]])
    for i in range(4):
        assert rel_l2(net.mats[i], ws[i]) <= 2e-3
        assert rel_l2(net.mats[i].cpu() - start[f"mats.{i}"], ws[i] - start[f"mats.{i}"]) <= 1e-2
        bucket = next(b for b in ref.buckets if b.params[0] is ws[i])
        assert rel_l2(opt.state[net.mats[i]]["momentum"], bucket.momentum[0]) <= 1e-5
        assert rel_l2(opt.state[net.mats[i]]["variance"], bucket.variance[0]) <= 2e-3
    assert rel_l2(net.table.weight, table) <= 1e-5


# ---------------------------------------------------------------------------
# behaviours pinned by the reference's tests
# ---------------------------------------------------------------------------
def _exact_polar(x: torch.Tensor, eps: float) -> torch.Tensor:
    u, _, vh = torch.linalg.svd(x.double(), full_matrices=False)
    return (u @ vh).bfloat16()


def _reference_dion_step(w, m, v, g, *, k, lr, wd, momentum=0.95, beta2=0.95):
    """src/dionw/optimizer.py:3-22 in plain torch with an exact polar factor."""
    rows, cols = w.shape
    m.add_(g)
    idx = torch.sort(torch.topk(m.abs().sum(-1), k).indices).values
    sel = m[idx].clone()
    m[idx] = sel * momentum
    o = _exact_polar(sel[None], 0.0)[0].double()
    vs = v[idx]
    vs = torch.lerp(vs, o.square().mean(-1, keepdim=True), 1 - beta2)
    v[idx] = vs
    normalized = o / (vs.sqrt() + 1e-8)
    normalized = normalized * (o.norm() / normalized.norm().clamp_min(1e-8))
    step = lr * 0.2 * math.sqrt(max(rows, cols)) * math.sqrt(min(rows, cols) / min(k, cols))
    w.mul_(1 - lr * wd)
    w[idx] -= step * normalized


def test_elementwise_path_with_an_exact_polar_factor(monkeypatch) -> None:
    """The seam the reference's tests use: ``_buckets.newton_schulz_fn`` swapped for an SVD
    polar factor, so everything except Newton-Schulz is checked tightly (1e-6 here;
    tests/test_optimizer.py:90-166 uses atol 1e-7 against microsoft/dion)."""
    monkeypatch.setattr("dionw_b200._buckets.newton_schulz_fn", lambda kind: _exact_polar)
    gen = torch.Generator().manual_seed(2)
    net = nn.Linear(96, 64, bias=False)
    w0 = net.weight.detach().clone()
    net = net.to(DEV)
    groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=32)
    opt = dionw.Dion(groups, lr=1e-2, weight_decay=0.1)
    w, m, v = w0.clone().double(), torch.zeros(64, 96).double(), torch.zeros(64, 1).double()
    for _ in range(4):
        g = _seeded((64, 96), 1.0, gen)
        net.weight.grad = g.to(DEV)
        opt.step()
        _reference_dion_step(w, m, v, g.double(), k=16, lr=1e-2, wd=0.1)
    assert rel_l2(net.weight, w) <= 1e-6
    assert rel_l2(opt.state[net.weight]["momentum"], m) <= 1e-6
    assert rel_l2(opt.state[net.weight]["variance"], v) <= 1e-5


def test_bucket_state_shares_one_storage_and_survives_torch_save() -> None:
    """tests/test_optimizer.py:481-494 of the reference."""
    net = nn.Sequential(nn.Linear(64, 32, bias=False), nn.Linear(64, 32, bias=False), nn.Linear(32, 64)).to(DEV)
    groups, _ = dionw.param_groups(net)
    opt = dionw.Dion(groups, lr=1e-3)
    for p in net.parameters():
        p.grad = torch.randn_like(p)
    opt.step()
    a, b = opt.state[net[0].weight]["momentum"], opt.state[net[1].weight]["momentum"]
    assert a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()
    assert a.untyped_storage().nbytes() == 2 * 32 * 64 * 4
    assert a.shape == net[0].weight.shape and opt.state[net[0].weight]["variance"].shape == (32, 1)
    saved = io.BytesIO()
    torch.save(opt.state_dict(), saved)
    saved.seek(0)
    loaded = torch.load(saved, weights_only=False)
    s0, s1 = (loaded["state"][i]["momentum"] for i in (_index_of(opt, net[0].weight), _index_of(opt, net[1].weight)))
    assert s0.untyped_storage().data_ptr() == s1.untyped_storage().data_ptr()
    group = loaded["param_groups"][-1]
    assert set(group) == {"dion_route", "fraction", "num_heads", "newton_schulz", "row_normalization",
                          "momentum_form", "lr", "momentum", "muon_beta2", "betas", "weight_decay", "eps", "params"}


def _index_of(opt, param) -> int:
    index = 0
    for group in opt.param_groups:
        for p in group["params"]:
            if p is param:
                return index
            index += 1
    raise KeyError


def _make(seed: int, ema=None):
    torch.manual_seed(seed)
    net = nn.Sequential(nn.Linear(128, 64), nn.Linear(64, 128), nn.LayerNorm(128)).to(DEV)
    groups, _ = dionw.param_groups(net, fraction=0.5, selection_min_dim=64)
    return net, dionw.Dion(groups, lr=1e-3, weight_decay=0.01, ema=ema)


@pytest.mark.parametrize("ema", [None, EMAConfig(decay=0.9), EMAConfig(decay=0.9, device=EMADevice.CPU)])
def test_resume_is_bit_exact(ema) -> None:
    """tests/test_optimizer.py:309-374 of the reference: save after two steps, load into a
    fresh optimizer, a third step gives identical bits (weights, state, shadows)."""
    net_a, opt_a = _make(0, ema)
    gen = torch.Generator(device=DEV).manual_seed(5)
    grads = [[torch.randn(p.shape, device=DEV, generator=gen) for p in net_a.parameters()] for _ in range(3)]
    for s in range(2):
        for p, g in zip(net_a.parameters(), grads[s]):
            p.grad = g.clone()
        opt_a.step()
    net_b, opt_b = _make(1, ema)
    net_b.load_state_dict(net_a.state_dict())
    # through torch.save, as a real resume does (a state_dict holds the live state tensors)
    buffer = io.BytesIO()
    torch.save(opt_a.state_dict(), buffer)
    buffer.seek(0)
    opt_b.load_state_dict(torch.load(buffer, weights_only=False))
    for net, opt in ((net_a, opt_a), (net_b, opt_b)):
        for p, g in zip(net.parameters(), grads[2]):
            p.grad = g.clone()
        opt.step()
    sa, sb = opt_a.state_dict(), opt_b.state_dict()
    for pa, pb in zip(net_a.parameters(), net_b.parameters()):
        assert torch.equal(pa, pb)
    for index, entry in sa["state"].items():
        for key, value in entry.items():
            other = sb["state"][index][key]
            if isinstance(value, torch.Tensor):
                assert torch.equal(value.cpu(), other.cpu()), (index, key)
            else:
                assert value == other
    assert sa.get("_ema_step_count") == sb.get("_ema_step_count")


def test_structural_mismatch_is_refused() -> None:
    net, opt = _make(0)
    other_groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=64)
    other = dionw.Dion(other_groups, lr=1e-3)
    with pytest.raises(ValueError, match="'fraction'"):
        other.load_state_dict(opt.state_dict())
    with pytest.raises(ValueError, match="without EMA"):
        _, with_ema = _make(0, EMAConfig())
        opt.load_state_dict(with_ema.state_dict())
    with pytest.raises(ValueError, match="no valid EMA step count"):
        _, with_ema = _make(0, EMAConfig())
        with_ema.load_state_dict(opt.state_dict())


def test_parameters_without_gradients_are_skipped_and_split_runs() -> None:
    """tests/test_optimizer.py:377-386, :657-728: a missing gradient splits the bucket into
    runs; the result equals stepping each parameter as a run of its own."""
    def build():
        torch.manual_seed(3)
        net = nn.ModuleList([nn.Linear(64, 48, bias=False) for _ in range(5)]).to(DEV)
        groups, _ = dionw.param_groups(net, fraction=0.5, selection_min_dim=32)
        return net, dionw.Dion(groups, lr=1e-2, weight_decay=0.1)

    net_a, opt_a = build()
    net_b, opt_b = build()
    gen = torch.Generator(device=DEV).manual_seed(9)
    grads = [torch.randn(48, 64, device=DEV, generator=gen) for _ in range(5)]
    before = net_a[2].weight.detach().clone()
    for net in (net_a, net_b):
        for i, layer in enumerate(net):
            layer.weight.grad = None if i == 2 else grads[i].clone()
    opt_a.step()
    import dionw_b200.optimizer as optimizer_module
    limit = optimizer_module.MAX_RUN_ELEMENTS
    optimizer_module.MAX_RUN_ELEMENTS = 1  # every parameter becomes a run of its own
    try:
        opt_b.step()
    finally:
        optimizer_module.MAX_RUN_ELEMENTS = limit
    assert torch.equal(net_a[2].weight, before)
    for la, lb in zip(net_a, net_b):
        assert torch.equal(la.weight, lb.weight)
        assert torch.equal(opt_a.state[la.weight]["momentum"], opt_b.state[lb.weight]["momentum"])


def test_weight_decay_reaches_every_row_and_spares_exempt_groups() -> None:
    """tests/test_optimizer.py:570-587: decay is exact (atol 0) on unselected rows."""
    torch.manual_seed(4)
    net = nn.Sequential(nn.Linear(64, 64), nn.LayerNorm(64)).to(DEV)
    groups, _ = dionw.param_groups(net, fraction=0.25, selection_min_dim=32)
    opt = dionw.Dion(groups, lr=1e-2, weight_decay=0.1)
    w0, norm0 = net[0].weight.detach().clone(), net[1].weight.detach().clone()
    net[0].weight.grad = torch.randn_like(net[0].weight)
    net[1].weight.grad = torch.zeros_like(net[1].weight)
    net[0].bias.grad = torch.zeros_like(net[0].bias)
    net[1].bias.grad = torch.zeros_like(net[1].bias)
    opt.step()
    rows = sorted(opt._last_rows[id(net[0].weight)])
    untouched = [r for r in range(64) if r not in rows]
    assert len(rows) == 16
    assert torch.equal(net[0].weight[untouched], w0[untouched] * (1 - 1e-2 * 0.1))
    assert not torch.equal(net[0].weight[rows], w0[rows] * (1 - 1e-2 * 0.1))
    assert torch.equal(net[1].weight, norm0)  # zero grad, exempt from decay


def test_head_split_equals_separate_heads() -> None:
    """tests/test_optimizer.py:590-632: a num_heads split steps like independent matrices."""
    torch.manual_seed(5)
    fused = nn.Linear(64, 96, bias=False).to(DEV)
    heads = nn.ModuleList([nn.Linear(64, 32, bias=False) for _ in range(3)]).to(DEV)
    with torch.no_grad():
        for i, h in enumerate(heads):
            h.weight.copy_(fused.weight[32 * i: 32 * (i + 1)])
    g1, _ = dionw.param_groups(fused, routes={fused.weight: Route(RouteKind.MATRIX, num_heads=3)})
    g2, _ = dionw.param_groups(heads)
    o1, o2 = dionw.Dion(g1, lr=1e-2), dionw.Dion(g2, lr=1e-2)
    for _ in range(2):
        g = torch.randn(96, 64, device=DEV)
        fused.weight.grad = g
        for i, h in enumerate(heads):
            h.weight.grad = g[32 * i: 32 * (i + 1)].clone()
        o1.step()
        o2.step()
    for i, h in enumerate(heads):
        assert torch.equal(fused.weight[32 * i: 32 * (i + 1)], h.weight)


def test_channels_last_weights_step_like_contiguous_ones() -> None:
    """tests/test_optimizer.py:389-414 (1e-6)."""
    torch.manual_seed(6)
    a = nn.Conv2d(16, 32, 3, bias=False).to(DEV)
    b = nn.Conv2d(16, 32, 3, bias=False).to(DEV)
    with torch.no_grad():
        b.weight.copy_(a.weight)
    b = b.to(memory_format=torch.channels_last)
    oa = dionw.Dion(dionw.param_groups(a).groups, lr=1e-2, weight_decay=0.1)
    ob = dionw.Dion(dionw.param_groups(b).groups, lr=1e-2, weight_decay=0.1)
    for _ in range(2):
        g = torch.randn_like(a.weight)
        a.weight.grad = g.clone()
        b.weight.grad = g.clone().contiguous(memory_format=torch.channels_last)
        oa.step()
        ob.step()
    torch.testing.assert_close(a.weight, b.weight, rtol=0, atol=1e-6)


def test_add_param_group_after_a_step_repacks_state() -> None:
    """tests/test_optimizer.py:417-453."""
    torch.manual_seed(7)
    first, second = nn.Linear(64, 32, bias=False).to(DEV), nn.Linear(64, 32, bias=False).to(DEV)
    opt = dionw.Dion(dionw.param_groups(first).groups, lr=1e-2)
    first.weight.grad = torch.randn_like(first.weight)
    opt.step()
    kept = opt.state[first.weight]["momentum"].clone()
    opt.add_param_group(dionw.param_groups(second).groups[0])
    first.weight.grad = torch.zeros_like(first.weight)
    second.weight.grad = torch.randn_like(second.weight)
    opt.step()
    # carried into the new layout, then one more step with a zero gradient: M = 0.95 * (M + 0)
    assert torch.equal(opt.state[first.weight]["momentum"], kept * 0.95)
    assert opt.state[second.weight]["momentum"].abs().sum() > 0
    with pytest.raises(TypeError, match="ordered, not a set"):
        opt.add_param_group({"params": {second.weight}, "dion_route": "matrix"})
    with pytest.raises(ValueError, match="not in the optimizer"):
        opt.initialize_state(nn.Parameter(torch.zeros(4, 4, device=DEV)))


def test_muon_update_matches_an_eager_restatement() -> None:
    """MUON_UPDATE (Keller iteration, no row normalization, Nesterov momentum): the step of
    tests/test_muon.py:104-115 of the reference, with this package's own iteration."""
    torch.manual_seed(8)
    net = nn.Linear(96, 64, bias=False).to(DEV)
    groups, _ = dionw.param_groups(net, fraction=1.0)
    opt = dionw.Dion(groups, lr=1e-2, weight_decay=0.1, matrix_update=dionw.MUON_UPDATE)
    keller = dionw.newton_schulz.newton_schulz_fn(dionw.NewtonSchulz.KELLER_TRITON)
    w, buf = net.weight.detach().clone(), torch.zeros(64, 96, device=DEV)
    for _ in range(3):
        g = torch.randn(64, 96, device=DEV)
        net.weight.grad = g.clone()
        opt.step()
        buf = (buf + g) * 0.95
        update = keller((g + buf)[None], 1e-8)[0].float()
        w = w * (1 - 1e-2 * 0.1) - 1e-2 * 0.2 * math.sqrt(96) * update
    # The optimizer takes the block norm from fp32 row sums, the direct call from the
    # bf16-rounded matrix: the two can differ by one bf16 step of the normaliser.
    assert rel_l2(net.weight, w) <= 1e-4
    assert "variance" in opt.state[net.weight]
    with pytest.raises(ValueError, match="Nesterov momentum needs every row"):
        dionw.Dion(dionw.param_groups(net, fraction=0.5, selection_min_dim=8).groups, lr=1e-2,
                   matrix_update=dionw.MUON_UPDATE)


@pytest.mark.parametrize("kind", list(dionw.NewtonSchulz))
def test_every_kind_returns_bf16_close_to_the_polar_factor(kind) -> None:
    """tests/test_newton_schulz.py:125-134 of the reference."""
    x = torch.randn(2, 64, 96, generator=torch.Generator().manual_seed(0))
    out = dionw.newton_schulz.newton_schulz_fn(kind)(x.to(DEV), 1e-7)
    assert out.dtype == torch.bfloat16 and out.shape == x.shape
    assert rel_l2(out.float(), oracle.exact_polar(x)) < 0.2


# ---------------------------------------------------------------------------
# EMA
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("device", [EMADevice.GPU, EMADevice.CPU])
def test_ema_schedule_against_lerp(device) -> None:
    """tests/test_ema.py:87-138: start_step, cadence and decay**n against plain lerp."""
    torch.manual_seed(9)
    net = nn.Linear(32, 16).to(DEV)
    cfg = EMAConfig(decay=0.9, device=device, update_every_n_steps=2, start_step=3)
    opt = dionw.Dion(dionw.param_groups(net).groups, lr=1e-2, ema=cfg)
    shadow = None
    for step in range(1, 10):
        for p in net.parameters():
            p.grad = torch.randn_like(p)
        opt.step()
        opt.ema.flush_pending_updates()
        live = net.weight.detach().cpu().clone()
        if step == 3:
            shadow = live.clone()
        elif step > 3 and (step - 3) % 2 == 0:
            shadow.lerp_(live, 1 - 0.9**2)
        if shadow is None:
            assert "ema_shadow" not in opt.state[net.weight]
        else:
            torch.testing.assert_close(opt.state[net.weight]["ema_shadow"].cpu(), shadow, rtol=0, atol=1e-7)


@pytest.mark.parametrize("device", [EMADevice.GPU, EMADevice.CPU])
def test_swap_and_restore(device) -> None:
    """tests/test_ema.py:208-360."""
    torch.manual_seed(10)
    net = nn.Linear(32, 16).to(DEV)
    opt = dionw.Dion(dionw.param_groups(net).groups, lr=1e-2, ema=EMAConfig(decay=0.5, device=device))
    assert opt.swap_ema_weights() is False  # nothing to swap before the first update
    for _ in range(2):
        for p in net.parameters():
            p.grad = torch.randn_like(p)
        opt.step()
    live = net.weight.detach().clone()
    assert opt.swap_ema_weights(net) is True
    assert opt.ema_weights_swapped
    torch.testing.assert_close(net.weight.detach().cpu(), opt.state[net.weight]["ema_shadow"].cpu())
    with pytest.raises(RuntimeError, match="swapped in"):
        opt.step()
    with pytest.raises(RuntimeError, match="already swapped"):
        opt.swap_ema_weights()
    assert opt.restore_non_ema_weights() is True
    assert torch.equal(net.weight, live) and not opt.ema_weights_swapped
    stranger = nn.Linear(4, 4).to(DEV)
    with pytest.raises(ValueError, match="outside the optimizer"):
        opt.swap_ema_weights(stranger)
    saved = opt.state_dict()
    assert all(k not in entry for entry in saved["state"].values() for k in ("ema_pending", "ema_tmp_cpu", "ema_event"))


def test_ema_checkpoint_moves_between_devices() -> None:
    """tests/test_ema.py:383-437: a GPU-EMA checkpoint loads into a CPU-EMA optimizer and back."""
    net_a, opt_a = _make(0, EMAConfig(decay=0.9, device=EMADevice.GPU))
    for _ in range(2):
        for p in net_a.parameters():
            p.grad = torch.randn_like(p)
        opt_a.step()
    net_b, opt_b = _make(0, EMAConfig(decay=0.9, device=EMADevice.CPU))
    opt_b.load_state_dict(opt_a.state_dict())
    for pa, pb in zip(net_a.parameters(), net_b.parameters()):
        sa, sb = opt_a.state[pa]["ema_shadow"], opt_b.state[pb]["ema_shadow"]
        assert sb.device.type == "cpu" and torch.equal(sa.cpu(), sb)
    assert opt_b.ema.step_count == 2


def test_mixin_on_a_stock_optimizer_with_bf16_parameters() -> None:
    """tests/test_ema.py:469-508."""
    class AdamWWithEMA(dionw.IntegratedEMAOptimizer, torch.optim.AdamW):
        def __init__(self, params, ema, **kw):
            super().__init__(params, **kw)
            self._init_integrated_ema(ema, dionw.ema.no_profile)

    net = nn.Linear(16, 8).to(DEV).bfloat16()
    opt = AdamWWithEMA(net.parameters(), EMAConfig(decay=0.5), lr=1e-2)
    for _ in range(2):
        for p in net.parameters():
            p.grad = torch.randn_like(p)
        opt.step()
    shadow = opt.state[net.weight]["ema_shadow"]
    assert shadow.dtype == torch.float32 and shadow.is_cuda
    assert opt.swap_ema_weights() and opt.restore_non_ema_weights()


def test_remaining_refusals_carry_the_reference_messages() -> None:
    """The refusals no other test reaches: a non-float32 CUDA parameter (src/dionw/optimizer.py:201-209),
    a run holding a parameter without a gradient (src/dionw/_matrix_step.py:129-130), and the two
    partial EMA swaps (src/dionw/ema/_swap.py:43-101)."""
    half = nn.Linear(32, 16).to(DEV).half()
    with pytest.raises(TypeError, match="float32 parameters"):
        dionw.Dion(dionw.param_groups(half).groups, lr=1e-3)

    net = nn.Linear(32, 16).to(DEV)
    opt = dionw.Dion(dionw.param_groups(net).groups, lr=1e-2, ema=EMAConfig(decay=0.5))
    from dionw_b200 import _matrix_step

    net.weight.grad = None
    bucket = opt._ensure_buckets()[0]
    with pytest.raises(RuntimeError, match="a Dion run holds a parameter without a gradient"):
        _matrix_step.step_run(bucket, [0], opt.param_groups[bucket.group_index], opt.state)

    for p in net.parameters():
        p.grad = torch.randn_like(p)
    opt.step()
    frozen = nn.Linear(4, 4).to(DEV).requires_grad_(False)
    with pytest.raises(ValueError, match="no optimizer-managed parameters"):
        opt.swap_ema_weights(frozen)
    del opt.state[net.bias]["ema_shadow"]
    with pytest.raises(RuntimeError, match="Refusing to mix live and EMA weights"):
        opt.swap_ema_weights()
    assert not opt.ema_weights_swapped
