import pytest
import torch

from transformers_fusion_b200.models import moe_extras as X


def test_dense_to_moe_reproduces_dense_with_all_experts():
    torch.manual_seed(0)
    H, F, E = 16, 32, 4
    gate_up, down = torch.randn(2 * F, H), torch.randn(H, F)
    gu, dn, router, assign = X.DenseToMoEPruner(E).convert(gate_up, down)
    assert gu.shape == (E, 2 * F // E, H) and dn.shape == (E, H, F // E) and router.shape == (E, H)
    assert torch.bincount(assign, minlength=E).tolist() == [F // E] * E
    x = torch.randn(5, H)
    dense = (torch.nn.functional.silu(x @ gate_up[:F].t()) * (x @ gate_up[F:].t())) @ down.t()
    per = F // E
    mix = sum((torch.nn.functional.silu(x @ gu[e, :per].t()) * (x @ gu[e, per:].t())) @ dn[e].t() for e in range(E))
    assert torch.allclose(mix, dense, atol=1e-4)


def test_routers():
    torch.manual_seed(1)
    logits = torch.randn(64, 4)
    idx, w, kept, aux = X.SwitchV2Router(4, capacity_factor=1.0).route(logits)
    assert idx.shape == (64,) and float(aux) > 0 and int(kept.sum()) <= 64 and torch.bincount(idx[kept], minlength=4).max() <= 16
    assert bool((w[~kept] == 0).all())
    ec = X.ExpertChoiceV2(4, capacity_factor=2.0)
    tok, wt = ec.route(logits)
    assert tok.shape == (4, 32) and wt.shape == (4, 32)                       # every expert serves exactly 32 tokens
    x = torch.randn(64, 8)
    y = ec.combine(x, tok, wt, lambda e, t: t * (e + 1))
    assert y.shape == x.shape
    d = X.ExpertDropout(0.9, keep_min=2)
    out = d(torch.zeros(3, 8), generator=torch.Generator().manual_seed(0))
    assert int(torch.isfinite(out[0]).sum()) >= 2 and torch.equal(d(torch.zeros(3, 8), training=False), torch.zeros(3, 8))


def test_merger_and_dynamic_pool():
    torch.manual_seed(2)
    a, b = torch.randn(1, 8, 4), torch.randn(1, 8, 4)
    gu = torch.cat([a, a + 0.01, b, b + 0.01])
    dn = torch.randn(1, 4, 4).repeat(4, 1, 1)
    g2, d2, mapping = X.ExpertMerger.merge(gu, dn, 2, usage=torch.tensor([3.0, 1.0, 1.0, 1.0]))
    assert g2.shape[0] == 2 and mapping[0] == mapping[1] and mapping[2] == mapping[3] and mapping[0] != mapping[2]
    assert torch.allclose(g2[mapping[0]], (3 * gu[0] + gu[1]) / 4, atol=1e-6)
    pool = X.DynamicExpertPool(torch.randn(4, 8, 4), torch.randn(4, 4, 4), torch.randn(4, 4), split_above=0.5, drop_below=0.02, momentum=0.0)
    pool.observe(torch.tensor([0] * 90 + [1] * 9 + [2] * 1))                   # expert 0 overloaded, expert 3 idle
    log = pool.adapt(torch.Generator().manual_seed(0))
    assert log["split"] == [0] and 3 in log["dropped"] and pool.num_experts == pool.gu.shape[0] == pool.router.shape[0]
    assert abs(float(pool.share.sum()) - 1) < 1e-6


def test_expert_prefetcher(tmp_path):
    pf = X.ExpertPrefetcher(str(tmp_path), host_slots=2, device_slots=1)
    for e in range(4):
        pf.store(e, {"w": torch.full((3,), float(e))})
    pf.prefetch([2])
    assert float(pf.get(2)["w"][0]) == 2.0
    assert float(pf.get(0)["w"][0]) == 0.0 and list(pf.dev) == [0] and pf.stats["disk_loads"] == 2
    assert float(pf.get(2)["w"][0]) == 2.0 and pf.stats["host_hits"] >= 1       # evicted from the device, still on the host
    with pytest.raises(TimeoutError):
        pf.get(99, timeout_s=0.2)                                                # missing file: bounded wait, clear error
    pf.close()


def test_reference_named_verbs(tmp_path):
    import torch
    from transformers_fusion_b200.models import moe_extras as X
    from transformers_fusion_b200.models.config import MoEConfig, TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.models.moe import MoEModel
    g = torch.Generator().manual_seed(0)
    H, Fd, E = 16, 32, 4
    gate, up, down = torch.randn(Fd, H, generator=g), torch.randn(Fd, H, generator=g), torch.randn(H, Fd, generator=g)
    pr = X.DenseToMoEPruner(E)
    a, b = pr.prune_ffn(gate, up, down), pr.convert(torch.cat([gate, up], 0), down)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    logits = torch.randn(12, E, generator=g)
    sw = X.SwitchV2Router(E, capacity_factor=1.0)
    d = sw.forward(logits, 12)
    idx, w, kept, _ = sw.route(logits)
    assert d.shape == (12, E) and (d > 0).sum(1).max() <= 1 and int((d > 0).sum()) == int(kept.sum())
    assert (d > 0).sum(0).max() <= 3                               # capacity 1.0 * 12 / 4
    x = torch.randn(12, H, generator=g)
    ec = X.ExpertChoiceV2(E, capacity_factor=2.0)
    tok, wt = ec.route(logits)
    want = torch.zeros(12, H)
    for e in range(E):
        want.index_add_(0, tok[e], x[tok[e]] * wt[e][:, None])
    assert torch.allclose(ec.forward(x, logits), want, atol=1e-6)
    dr = X.ExpertDropout(p=0.5, keep_min=2)
    assert dr.get_active_count(8) == 4 and dr.get_active_count(2) == 2
    masks = [dr.get_mask(8, generator=g) for _ in range(20)]
    assert all(sum(m) >= 2 and len(m) == 8 for m in masks) and any(sum(m) < 8 for m in masks)
    pool = X.DynamicExpertPool(torch.randn(2, 2 * Fd, H), torch.randn(2, H, Fd), torch.randn(2, H), min_experts=2, max_experts=3)
    assert pool.count() == 2 and pool.add_expert(torch.zeros(2 * Fd, H)) == 2 and pool.add_expert(torch.zeros(2 * Fd, H)) == -1
    assert abs(float(pool.share.sum()) - 1.0) < 1e-6 and pool.remove_expert(0) and pool.count() == 2 and not pool.remove_expert(0)
    assert not pool.remove_expert(7)
    # model accessors
    dm = DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=16,
                                      tie_embeddings=True, mtp_num_heads=1), dtype=torch.float32, seed=0)
    assert dm.vocab_size() == 64 and dm.param_count() == sum(p.numel() for p in dm.get_parameters())
    ids = torch.randint(0, 64, (2, 8), generator=g)
    assert dm.mtp_loss(ids, torch.roll(ids, -1, 1)) > 0
    mm = MoEModel(MoEConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, ffn_hidden_size=48, max_seq_len=32, num_experts=4,
                            top_k=2), dtype=torch.float32, seed=1)
    blk = mm.layers[0]
    experts = blk.gate_up.numel() + blk.down.numel()
    assert blk.num_stored_experts() == 4 and blk.activated_param_count() == blk.param_count() - experts // 2
    assert mm.stored_param_count() - mm.param_count() == 2 * (experts // 2) and mm.vocab_size() == 64
    pf = mm.init_prefetcher(str(tmp_path / "experts"), host_slots=4, device_slots=2)
    mm.wire_prefetcher_sources()
    pf.schedule_prefetch(1, [0, 3])
    wts = pf.get_expert_weights(1, 3)
    assert torch.equal(wts["gate_up"], mm.layers[1].gate_up.data[3]) and torch.equal(wts["down"], mm.layers[1].down.data[3])
    assert torch.equal(pf.get_expert_weights(0, 2)["down"], mm.layers[0].down.data[2])
    pf.release_expert(1, 3)
    st = pf.get_stats()
    assert st["evictions"] == 1 and st["disk_loads"] >= 3 and st["avg_wait_ms"] >= 0
    pf.set_expert_source(0, 0, torch.arange(4.0))
    assert pf.get_expert_weights(0, 0)["packed"].tolist() == [0.0, 1.0, 2.0, 3.0]
    pf.close()
