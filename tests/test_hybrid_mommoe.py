"""Hybrid schedules and models, modality-routed MoE, expert placement, native low-bit MoE training."""
import math

import pytest
import torch

from transformers_fusion_b200.models import hybrid as HY, mommoe as MM
from transformers_fusion_b200.models.config import MoEConfig, TransformerConfig


def test_hybrid_schedule_and_model_matches_dense_forward():
    s = HY.build_hybrid_schedule(6)
    assert s.total() == 6 and s.num_std == 6 and HY.build_hybrid_schedule(0).total() == 0
    w = HY.build_hybrid_schedule(8, reserved=2, window_every=2)
    assert w.layers == ["std", "window", "std", "window", "std", "window", "std", "std"] and w.num_std == 5
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, ffn_hidden_size=48, max_seq_len=64, init_std=0.1)
    m = HY.HybridModel(cfg, dtype=torch.float32, seed=0)
    ids = torch.randint(0, 64, (2, 24))
    assert torch.allclose(m.forward_hybrid(ids), m(ids).float().view(2, 24, -1), atol=2e-4)
    mw = HY.HybridModel(cfg, HY.build_hybrid_schedule(2, 0, 1), window=4, dtype=torch.float32, seed=0)
    lw = mw.forward_hybrid(ids)
    assert not torch.allclose(lw, m.forward_hybrid(ids), atol=1e-3)            # the window changes late positions ...
    assert torch.allclose(lw[:, :4], m.forward_hybrid(ids)[:, :4], atol=2e-4)  # ... but not the first `window` ones
    assert m.param_count() == sum(p.numel() for p in m.parameters()) and mw.layer_kinds() == ["window", "window"]
    with pytest.raises(ValueError):
        HY.HybridModel(cfg, HY.build_hybrid_schedule(3), dtype=torch.float32)


def test_hybrid_moe_model_and_expert_shards():
    cfg = MoEConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, ffn_hidden_size=48, max_seq_len=32, num_experts=4,
                    top_k=2, init_std=0.1)
    m = HY.HybridMoeModel(cfg, dtype=torch.float32, seed=0)
    assert m(torch.randint(0, 64, (2, 8))).shape[-1] == 64 and m.schedule_state()["layers"] == ["std", "std"]
    assert m.stored_param_count() == m.param_count() > 0
    sh = HY.HybridExpertShard(3)
    plan = sh.assign_schedule(m.schedule, 4)
    assert [a.node_id for a in plan[0]] == [0, 1, 2, 0] and [a.node_id for a in plan[1]] == [1, 2, 0, 1]
    assert sum(sh.node_load(plan)) == 8 and max(sh.node_load(plan)) - min(sh.node_load(plan)) <= 1


def test_mommoe_routes_by_modality_and_trains():
    torch.manual_seed(0)
    cfg = MM.MoMMoEConfig(hidden_size=32, num_heads=2, ffn_hidden=48, num_layers=2, num_experts=8, top_k=2, vocab_size=50)
    m = MM.MoMMoE(cfg)
    ids = torch.randint(0, 50, (2, 12))
    logits = m(ids)
    assert logits.shape == (2, 12, 50) and abs(sum(m.expert_utilization()) - 1) < 1e-5
    assert m.active_parameters() < m.total_parameters() and MM.modality_name(2) == "AUDIO"
    # with a vision hint and a strong affinity the vision expert (index 4) is in every token's top-2
    blk = m.layers[0]
    with torch.no_grad():
        blk.router.affinity_scale.fill_(50.0)
    hints = torch.full((2, 12), int(MM.Modality.VISION))
    out = blk(m.embeddings(ids), hints)
    assert bool((out.routing.indices == 4).any(-1).all()) and out.routing.dominant_modality == MM.Modality.VISION
    assert torch.allclose(out.routing.weights.sum(-1), torch.ones(24)) and out.cross_modal_output.shape == (2, 12, 32)
    opt = torch.optim.AdamW(m.parameters(), 3e-3)
    losses = []
    for _ in range(25):
        lg = m(ids[:, :-1])
        loss = torch.nn.functional.cross_entropy(lg.reshape(-1, 50), ids[:, 1:].reshape(-1)) + m.aux_loss
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] - 0.3
    g = m.generate(ids[:, :4], 5, temperature=0.0)
    assert g.shape == (2, 9) and torch.equal(g[:, :4], ids[:, :4])
    with pytest.raises(ValueError):
        MM.MoMMoEConfig(num_experts=5).expert_modality()


def test_native_quant_moe_model_steps():
    from transformers_fusion_b200.trainer.native_quant import NativeMoEConfig, NativeQUANTMoEModel
    cfg = NativeMoEConfig(hidden_size=32, num_heads=2, ffn_hidden=48, num_layers=1, num_experts=4, top_k=2, vocab_size=64, max_seq_len=32,
                          block_size=64)
    nm = NativeQUANTMoEModel(cfg, seed=0)
    nm.init_from_fp32()
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, 64, (17,), generator=g)
    ids, labels = base[:-1].repeat(4, 1), base[1:].repeat(4, 1)
    mets = [nm.step(ids, labels, 1e-3, 5e-2) for _ in range(30)]
    assert all(math.isfinite(x.loss) for x in mets) and mets[-1].loss < mets[0].loss - 0.05, (mets[0].loss, mets[-1].loss)
    assert mets[-1].quant8 + mets[-1].quant + mets[-1].quant1 > 0 and 0 < mets[-1].active_params < mets[-1].total_params
    rep = nm.memory_report()
    assert rep["bytes"] < rep["fp32_bytes"] and rep["stored_bits_per_weight"] < 16
    # the step in its parts gives the same result as step()
    a, b = NativeQUANTMoEModel(cfg, seed=1), NativeQUANTMoEModel(cfg, seed=1)
    met = a.step(ids, labels, 1e-3, 5e-2)
    loss = b.backward(ids, labels)
    frozen = b.apply_update(1e-3, 5e-2)
    assert loss == pytest.approx(met.loss) and 100.0 * frozen == pytest.approx(met.frozen_pct)
    assert all(torch.equal(pa, pb) for pa, pb in zip(a.model.parameters(), b.model.parameters()))
    assert "x smaller" in b.print_memory_report()


def test_modality_router_stand_alone_losses_and_accessors():
    torch.manual_seed(0)
    cfg = MM.MoMMoEConfig(hidden_size=32, num_heads=2, ffn_hidden=48, num_layers=1, num_experts=8, top_k=2, vocab_size=50)
    model = MM.MoMMoE(cfg)
    assert model.config() is cfg
    r = model.layers[0].router if hasattr(model.layers[0], "router") else next(m for m in model.modules() if isinstance(m, MM.TopKRouter))
    x = torch.randn(24, 32)
    out = r(x)
    assert r.num_experts() == 8 and r.top_k() == 2 and r.gate_weight().shape == (8, 32) and r.modality_head_weight().shape[1] == 32
    assert float(r.load_balance_loss(out.gates, out.indices)) == pytest.approx(float(out.load_balance_loss), rel=1e-5)
    logits = torch.randn(5, 8)
    assert float(r.z_loss(logits)) == pytest.approx(float((torch.logsumexp(logits, -1) ** 2).mean()))
    assert r.classify_modality(x) == out.dominant_modality


def test_modality_block_projection_views_and_self_attention():
    torch.manual_seed(0)
    blk = MM.MoMBlock(32, 2, 48, 8, 2, MM.MoMMoEConfig(num_experts=8).expert_modality())
    ex = blk.experts[5]
    x = torch.randn(6, 32)
    want = (torch.nn.functional.silu(x @ ex.gate_proj().t()) * (x @ ex.up_proj().t())) @ ex.down_proj().t()
    assert torch.allclose(ex(x), want, atol=1e-5) and ex.specialization() == MM.Modality.AUDIO
    ca = blk.cross_modal_attn
    assert ca.q_proj().shape == ca.k_proj().shape == ca.v_proj().shape == ca.o_proj().shape == (32, 32)
    with torch.no_grad():
        ca.k_proj().zero_()
    assert float(ca.kv.weight[:32].abs().sum()) == 0.0 and float(ca.kv.weight[32:].abs().sum()) > 0      # a view: writes go through
    h = torch.randn(2, 5, 32)
    out = blk(h)
    # the first sub-layer of the block is exactly self_attention on the normalised input
    a = blk.self_attention(blk.attention_norm(h))
    assert a.shape == h.shape
    h2 = h.clone()
    h2[:, -1] += 1.0
    a2 = blk.self_attention(blk.attention_norm(h2))
    assert torch.allclose(a[:, :-1], a2[:, :-1], atol=1e-6) and not torch.allclose(a[:, -1], a2[:, -1])   # causal
    assert out.hidden.shape == h.shape
