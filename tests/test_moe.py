"""MoE routing / permutation / grouped GEMM / combine: CPU path against a dense PyTorch autograd
statement; GPU kernels against the CPU path."""
import pytest
import torch

from transformers_fusion_b200.ops import _lib, moe


def dense_ref(x, logits, gate_up, down, k, renorm, lb, zw):
    T, H = x.shape
    E, F2, _ = gate_up.shape
    Fh = F2 // 2
    probs = torch.softmax(logits.float(), -1)
    w, idx = torch.topk(probs, k, -1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    y = torch.zeros(T, H, dtype=torch.float32)
    for e in range(E):
        gu = x.float() @ gate_up[e].float().t()
        h = torch.nn.functional.silu(gu[:, :Fh]) * gu[:, Fh:]
        out = h @ down[e].float().t()
        we = (w * (idx == e)).sum(-1, keepdim=True)
        y = y + we * out
    f = torch.bincount(idx.reshape(-1), minlength=E).float() / (T * k)
    lse = torch.logsumexp(logits.float(), -1)
    aux = lb * E * (f * probs.mean(0)).sum() + zw * (lse * lse).mean()
    return y, aux


@pytest.mark.parametrize("renorm", [True, False])
def test_moe_cpu_matches_dense_autograd(renorm):
    T, H, Fh, E, k = 37, 16, 24, 4, 2
    x = torch.randn(T, H, requires_grad=True)
    logits = torch.randn(T, E, requires_grad=True)
    gu = torch.nn.Parameter(torch.randn(E, 2 * Fh, H) * 0.3)
    dn = torch.nn.Parameter(torch.randn(E, H, Fh) * 0.3)
    y, aux, idx = moe.moe_ffn(x, logits, gu, dn, k, renorm, "silu", 0.01, 0.001)
    g = torch.randn_like(y)
    ((y * g).sum() + aux).backward()
    x2 = x.detach().clone().requires_grad_(True)
    l2 = logits.detach().clone().requires_grad_(True)
    gu2 = gu.detach().clone().requires_grad_(True)
    dn2 = dn.detach().clone().requires_grad_(True)
    yr, auxr = dense_ref(x2, l2, gu2, dn2, k, renorm, 0.01, 0.001)
    ((yr * g).sum() + auxr).backward()
    assert torch.allclose(y, yr, atol=1e-4)
    assert torch.allclose(aux, auxr, atol=1e-6)
    assert torch.allclose(x.grad, x2.grad, atol=1e-4)
    assert torch.allclose(logits.grad, l2.grad, atol=1e-4)
    assert torch.allclose(gu.main_grad, gu2.grad, atol=1e-4)
    assert torch.allclose(dn.main_grad, dn2.grad, atol=1e-4)


@pytest.mark.gpu
def test_moe_gpu_matches_cpu():
    T, H, Fh, E, k = 1000, 256, 384, 8, 2
    x = (torch.randn(T, H) * 0.5).bfloat16()
    logits = torch.randn(T, E)
    gu = (torch.randn(E, 2 * Fh, H) * 0.05).bfloat16()
    dn = (torch.randn(E, H, Fh) * 0.05).bfloat16()
    g = torch.randn(T, H).bfloat16()
    outs = []
    for dev in ("cpu", "cuda"):
        xx = x.detach().clone().to(dev).requires_grad_(True)
        ll = logits.detach().clone().to(dev).requires_grad_(True)
        gup, dnp = torch.nn.Parameter(gu.to(dev)), torch.nn.Parameter(dn.to(dev))
        y, aux, idx = moe.moe_ffn(xx, ll, gup, dnp, k, True, "silu", 0.01, 0.001)
        ((y.float() * g.to(dev).float()).sum() + aux).backward()
        outs.append([t.float().cpu() for t in (y, aux, xx.grad, ll.grad, gup.main_grad, dnp.main_grad)])
    torch.cuda.synchronize()
    _lib.check_status()
    for a, b, name in zip(outs[0], outs[1], ("y", "aux", "dx", "dlogits", "dgate_up", "ddown")):
        tol = 3e-2 * a.abs().max().item() + 1e-3
        assert (a - b).abs().max().item() < tol, (name, (a - b).abs().max().item(), a.abs().max().item())


@pytest.mark.gpu
def test_router_stats_and_pad_zeroing_gpu():
    """The router kernel's block-aggregated reductions equal the torch reductions; permute leaves every unassigned row of
    the expert buffer zero (padding behind each segment and the tail) without a whole-buffer fill."""
    from transformers_fusion_b200.ops import moe as M
    torch.manual_seed(0)
    T, E, k, H = 3000, 16, 2, 64
    logits = torch.randn(T, E, device="cuda").bfloat16()
    idx, w, probs, counts, lse, psum, lsq = M.router_topk_stats(logits, k, True)
    assert int(counts.sum()) == T * k
    assert torch.equal(counts.cpu(), torch.bincount(idx.reshape(-1).long().cpu(), minlength=E).int())
    assert torch.allclose(psum, probs.sum(0), rtol=1e-4, atol=1e-3)
    assert torch.allclose(lsq[0], (lse * lse).sum(), rtol=1e-4)
    plan = M.Plan(idx, counts, E)
    x = torch.randn(T, H, device="cuda").bfloat16()
    xp = M.permute(x, idx, plan)
    rows = plan.row_of.reshape(-1).long()
    assert rows.unique().numel() == T * k                                  # every assignment has its own row
    assert torch.equal(xp[rows], x.repeat_interleave(k, 0))
    mask = torch.ones(plan.max_rows, dtype=torch.bool, device="cuda")
    mask[rows] = False
    assert float(xp[mask].abs().sum()) == 0.0
    seg = plan.seg_start.cpu().tolist()
    for e in range(E):                                                     # rows of expert e lie inside its segment
        r = rows[(idx.reshape(-1) == e)]
        assert r.numel() == int(counts[e]) and (r.numel() == 0 or (int(r.min()) >= seg[e] and int(r.max()) < seg[e] + int(counts[e])))


def test_routing_rules_of_the_non_topk_variants():
    """Expert choice, hierarchical and BASE-layer selections and the three capacity policies (models/moe_routing.py)."""
    import torch
    from transformers_fusion_b200.models import moe_routing as R
    g = torch.Generator().manual_seed(0)
    T, E = 64, 8
    logits = torch.randn(T, E, generator=g) * 2
    # expert choice: every expert holds exactly its capacity before the per-token cap, never more after it
    sel = R.expert_choice(logits, 2.0, E)
    C = R.expert_choice_capacity(T, E, 2.0)
    assert C == 16 and bool((sel.sum(0) == C).all())
    sel2 = R.expert_choice(logits, 2.0, 2)
    assert bool((sel2.sum(1) <= 2).all()) and bool((sel2.sum(0) <= C).all()) and bool((sel2 <= sel).all())
    # hierarchical: 4 groups of 2, two groups per token, one expert per chosen group
    sel = R.hierarchical(logits, 4, 2, 1)
    assert bool((sel.sum(1) == 2).all())
    grp = sel.view(T, 4, 2).any(-1)
    assert bool((grp.sum(1) == 2).all())
    score = torch.logsumexp(logits.view(T, 4, 2), -1)
    assert bool((grp == torch.zeros_like(grp).scatter(1, score.topk(2, 1).indices, True)).all())
    # BASE layer: balanced, one expert per token
    sel = R.base_layer(logits)
    assert bool((sel.sum(1) == 1).all()) and int(sel.sum(0).max()) <= 8 and int(sel.sum(0).min()) >= 8
    # capacity policies on skewed logits: expert 0 is everybody's favourite
    skew = logits.clone()
    skew[:, 0] += 6.0
    cap = R.capacity_limit(T, E, 2, 1.0)
    for pol in ("fixed", "token_drop", "token_pass"):
        sel, pt = R.apply_capacity(skew, 2, 1.0, pol)
        assert int(sel.sum(0).max()) <= cap, pol
        assert bool((sel.sum(1) <= 2).all())
        if pol == "fixed":
            assert float(sel.sum()) > float(R.apply_capacity(skew, 2, 1.0, "token_drop")[0].sum())   # lost pairs were re-routed
        if pol == "token_pass":
            assert float(pt.max()) > 0 and float(pt.max()) <= 1.0
        else:
            assert float(pt.abs().max()) == 0


def test_variant_models_route_by_their_rule():
    import torch
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.moe import MoEAllConfig, create_moe_variant
    base = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(1))
    outs = {}
    for name, kw in (("EXPERT_CHOICE", {}), ("HIERARCHICAL", dict(num_groups=4, top_groups=2)), ("BASE_LAYER", {}),
                     ("SPARSE_TOPK", dict(capacity_policy="token_drop", capacity_factor=0.5)), ("SPARSE_TOPK", {})):
        m = create_moe_variant(name, base, MoEAllConfig(num_experts=8, top_k=2, expert_hidden=32, **kw), device="cpu",
                               dtype=torch.float32, seed=0)
        m.flatten()
        loss, ce, aux = m.loss(ids, torch.roll(ids, -1, 1))
        loss.backward()
        assert torch.isfinite(loss) and m.layers[0].router.grad is not None
        blk = m.layers[0]
        outs[(name, tuple(kw))] = float(ce.detach())
        if name == "EXPERT_CHOICE":
            assert int(blk.last_sel.sum(0).max()) <= 8           # capacity 2.0 * 32 / 8
        if name == "HIERARCHICAL":
            assert bool((blk.last_sel.sum(1) == 2).all())
        if name == "BASE_LAYER":
            assert int(blk.last_sel.sum(0).max()) == 4 and bool((blk.last_sel.sum(1) == 1).all())
        if kw.get("capacity_policy"):
            assert int(blk.last_sel.sum(0).max()) <= 4            # ceil(0.5 * 32 * 2 / 8)
    assert len(set(round(v, 5) for v in outs.values())) == len(outs)     # the rules really differ from plain top-k


def test_structural_and_quantised_output_variants():
    """PRODUCT_KEY (two independently routed halves), ATTENTION_MOE (product of two projections as routing score),
    LOWRANK_MOE (bottleneck in front of router and experts), DOMAIN_MOE (classifier-weighted expert groups) and the
    variants that snap the mixture to fixed levels: each trains (finite loss, gradients on its own parameters and on the
    experts of every group) and differs from plain top-k."""
    import torch
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.moe import MoEAllConfig, create_moe_variant
    base = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(1))
    ces = {}
    for name in ("SPARSE_TOPK", "PRODUCT_KEY", "ATTENTION_MOE", "LOWRANK_MOE", "DOMAIN_MOE", "QUANT_MOE", "Q1_MOE", "Q8_MOE",
                 "Q4_MOE", "QUANTIZED_INT8_MOE"):
        m = create_moe_variant(name, base, MoEAllConfig(num_experts=8, top_k=2, expert_hidden=32), device="cpu",
                               dtype=torch.float32, seed=0)
        m.flatten()
        loss, ce, aux = m.loss(ids, torch.roll(ids, -1, 1))
        loss.backward()
        blk = m.layers[0]
        assert torch.isfinite(loss), name
        ces[name] = round(float(ce.detach()), 6)
        g = blk.gate_up.main_grad.abs().sum((1, 2))
        if name == "PRODUCT_KEY":
            assert blk.last_idx.shape[1] == 4 and bool((blk.last_idx[:, :2] < 4).all()) and bool((blk.last_idx[:, 2:] >= 4).all())
            assert bool((g[:4] > 0).any()) and bool((g[4:] > 0).any())
        if name == "DOMAIN_MOE":
            assert blk.last_idx.shape[1] == 8 and blk.domain_classifier.grad is not None and bool((g > 0).all())
        if name == "ATTENTION_MOE":
            assert blk.router_k.grad is not None and float(blk.router_k.grad.abs().sum()) > 0
        if name == "LOWRANK_MOE":
            assert blk.lowrank_down.grad is not None and blk.lowrank_up.grad is not None
            names = [n for n, _ in m.named_tensors()]
            assert "layers.0.moe.lowrank_down.weight" in names
        if name in ("QUANT_MOE", "Q1_MOE", "Q8_MOE", "Q4_MOE"):
            assert float(g.sum()) > 0            # straight-through: the experts still get gradients
    assert ces["QUANTIZED_INT8_MOE"] == ces["SPARSE_TOPK"]          # all scales are one until calibrated
    # the structural variants really route / mix differently from plain top-k; the level-snapping ones change the output
    # wherever it does not already sit on a level (small mixtures may all snap to the same level at initialisation)
    for name in ("PRODUCT_KEY", "ATTENTION_MOE", "LOWRANK_MOE", "DOMAIN_MOE", "Q1_MOE", "Q8_MOE"):
        assert ces[name] != ces["SPARSE_TOPK"], (name, ces)


def test_cross_layer_multi_gate_and_state_variants():
    """CROSS_LAYER: every layer routes into one shared pool of experts (routers cycle over num_shared_layers); MMOE: the
    gate of the selected task routes; MAMBA_MOE: a tiled state projection is added in front of router and experts."""
    import torch
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.moe import MoEAllConfig, create_moe_variant
    base = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=3, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(1))
    lab = torch.roll(ids, -1, 1)

    def make(name, **kw):
        return create_moe_variant(name, base, MoEAllConfig(num_experts=8, top_k=2, expert_hidden=32, **kw), device="cpu",
                                  dtype=torch.float32, seed=0)
    plain = make("SPARSE_TOPK")
    cross = make("CROSS_LAYER", num_shared_layers=2)
    assert cross.layers[1].gate_up is cross.layers[0].gate_up and cross.layers[2].down is cross.layers[0].down
    assert cross.layers[2].router is cross.layers[0].router and cross.layers[1].router is not cross.layers[0].router
    n_plain = sum(p.numel() for p in plain.parameters())
    n_cross = sum(p.numel() for p in cross.parameters())
    assert n_cross < n_plain - 2 * cross.layers[0].gate_up.numel()            # two layers' experts (and one router) are gone
    cross.flatten()
    loss, _, _ = cross.loss(ids, lab)
    loss.backward()
    assert torch.isfinite(loss) and float(cross.layers[0].gate_up.main_grad.abs().sum()) > 0
    assert len([n for n, _ in cross.named_tensors() if "expert.0.gate_proj" in n]) == 3   # the file still lists every layer

    mm = make("MMOE", num_tasks=3)
    mm.flatten()
    outs = []
    for tid in (0, 1):
        for blk in mm.layers:
            blk.task_id = tid
        outs.append(mm(ids).detach())
    assert not torch.allclose(outs[0], outs[1])                               # another task, another gate
    loss, _, _ = mm.loss(ids, lab)
    loss.backward()
    g = mm.layers[0].task_gates.grad.view(3, 8, -1).abs().sum((1, 2))
    assert float(g[1]) > 0 and float(g[0]) == 0 and float(g[2]) == 0          # only the selected task's gate learns

    mb = make("MAMBA_MOE")
    mb.flatten()
    loss, ce, _ = mb.loss(ids, lab)
    loss.backward()
    assert torch.isfinite(loss) and mb.layers[0].ssm_proj.grad is not None and float(mb.layers[0].ssm_proj.grad.abs().sum()) > 0
    _, ce_plain, _ = plain.loss(ids, lab)
    assert float(ce.detach()) != float(ce_plain.detach())
