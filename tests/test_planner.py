"""FormatPlanner / FormatRegistry: budgets are hard, importance decides who gets the precise tier."""
import numpy as np
import pytest
import torch

from transformers_fusion_b200.quant import codec
from transformers_fusion_b200.quant.planner import FormatPlanner, FormatRegistry, ImportanceMetric


@pytest.mark.parametrize("bpw", [1.0, 1.5, 2.5, 3.3, 4.0, 5.0, 7.1, 9.0, 20.0, 32.0])
def test_plan_meets_budget(bpw):
    plan = FormatPlanner(bpw).plan_for_model(256 * 200 + 77)
    assert plan.achieved_bpw <= max(bpw, 1.0) + 1e-3
    if bpw >= 2:
        assert plan.achieved_bpw > 0.7 * bpw
    assert len(plan.blocks) == 201 and plan.blocks[-1].num_weights == 77


def test_importance_orders_tiers():
    torch.manual_seed(0)
    w = torch.randn(64 * 256)
    w[: 8 * 256] *= 20
    p = FormatPlanner(5.0)
    s = p.score_importance(w)
    assert s.shape == (64,) and s[:8].min() > s[8:].max()
    plan = p.allocate(64)
    fm = plan.formats()
    hi = max(set(fm.tolist()), key=codec.format_bpw)
    assert plan.uses_mix and (fm[:8] == hi).all()
    g = torch.zeros_like(w)
    g[-256:] = 5.0
    s2 = p.score_importance(w, g, metric=ImportanceMetric.FISHER_DIAG)
    assert int(np.argmax(s2)) == 63


def test_mix_allocation_budget_and_quality():
    rng = np.random.default_rng(0)
    d = rng.standard_normal(256 * 64).astype(np.float32)
    d[: 256 * 4] *= 30
    for mix in (FormatRegistry.get_twi_mix(3.5), FormatRegistry.get_four_mix(4.0)):
        fm = FormatRegistry.allocate_mix_blocks(mix, d)
        by = sum(codec.claimed_bytes(int(f), 256) for f in fm)
        assert by <= int(np.ceil(mix.effective_bpw * d.size / 8))
        best = max(mix.tiers, key=codec.format_bpw)
        assert (fm[:4] == best).all()          # the loud blocks are promoted first
    # measured selection never exceeds the target
    f = FormatRegistry.select_best_format(4.6, d)
    assert f.bpw <= 4.6 + 1e-6
    m = FormatRegistry.select_best_mix(4.6, d)
    assert m.effective_bpw <= 4.6 + 1e-6


def test_table_and_parse():
    t = FormatRegistry.get_format_table()
    assert "Q_4" in t and "Q_G_8_K_M" in t and t.count("\n") > 105
    assert FormatRegistry.parse_format_name("q8").name == "Q_8"
    assert FormatRegistry.parse_format_name("nonsense") is None
    mix = FormatPlanner.compute_format_mix(100, 5.0)
    assert mix == {6: 50, 4: 50}


def test_mixed_tensor_roundtrip(tmp_path):
    torch.manual_seed(1)
    w = torch.randn(256 * 10 + 5)
    plan = FormatPlanner(6.0).plan_for_model(w.numel())
    wr = codec.QuantWriter(tmp_path / "m.quant")
    wr.add_tensor_mixed("w", w, plan.formats())
    wr.close()
    r = codec.QuantReader(tmp_path / "m.quant")
    assert (r.block_formats("w") == plan.formats()).all()
    back = r.read_tensor("w")
    # Q_6 is a 64-level normal-quantile codebook: outliers beyond its top level clip, so the check is on the energy of the error
    assert back.shape == w.shape and float(((back - w) ** 2).sum() / (w ** 2).sum()) < 5e-3


def test_registry_quantize_results():
    import numpy as np
    from transformers_fusion_b200.quant.planner import FormatRegistry as R
    rng = np.random.default_rng(0)
    w = rng.standard_normal(1000).astype(np.float32)
    q8 = R.quantize_q8(w)
    back = R.dequantize(q8)
    assert back.shape == (1000,) and R.measure_mse(w, back) < 1e-3 and len(q8.blocks) == 4
    assert 8.0 <= R.actual_bpw(q8) < 9.5 and R.serialized_size_bytes(q8) == sum(map(len, q8.blocks)) + 48
    errs = [R.measure_mse(w, R.dequantize(f(w))) for f in (R.quantize_q1, R.quantize_q2, R.quantize_q4, R.quantize_q8)]
    assert errs == sorted(errs, reverse=True)
    one = R.quantize_block(w[:100], R.parse_format_name("Q_4"))
    assert len(one.blocks) == 1 and R.dequantize(one).shape == (100,)
    scaled = np.concatenate([w[:256] * 10, w[256:512] * 0.1, w[512:768] * 5, w[768:] * 0.2])
    mix = R.quantize_q_twi_mix_1_5(scaled, 256)
    assert [R.parse_format_name("Q_2").id == m.format for m in mix] == [True, False, True, False]
    sp = R.quantize_q_sparse(w, 0.1)
    dense = R.dequantize_sparse(sp)
    assert sp["indices"].size == 100 and (dense != 0).sum() == 100 and abs(dense).max() == pytest.approx(abs(w).max(), rel=1e-3)
