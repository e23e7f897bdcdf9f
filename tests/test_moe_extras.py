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
