"""Mixture-of-experts decoder: dense attention blocks whose FFN is a sparse MoE layer (router ->
top-k -> grouped expert GEMMs -> weighted combine), optional shared expert, 26 routing variants.

The expert path is ``ops.moe.moe_ffn`` (device-side routing plan, grouped tcgen05 GEMMs, no host
sync); with ``cfg.expert_fp8`` the expert GEMMs run in block-scaled E4M3 (1x128 activation scales,
128x128 weight scales).  Under expert parallelism (``parallel.ep.ExpertParallel``) the permute /
combine steps become the NVLink all-to-all.

Reference counterparts: MoEBlock / MoEModel and tensor names ``layers.{i}.moe.router.weight``,
``layers.{i}.moe.expert.{e}.{gate,up,down}_proj.weight``, ``layers.{i}.shared_expert.*``
(src/model/moe_model.cpp:33-57,180-236,384-502), SparseMoE + variants (include/quant/moe_variants.h:19-123,
src/model/moe_variants.cpp), ExpertFFN / softmax_with_topk / load-balance loss (src/model/moe_core.cpp:70-188).
"""
from __future__ import annotations

from typing import Optional

from dataclasses import dataclass

import math

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..ops import moe as M
from . import moe_routing as R
from .config import MoEConfig, TransformerConfig
from .dense import DenseModel, FlatBuffers, _EmbedFn, _FinalNormFn, _LinearFn, _ensure_main_grad

# variant name -> (top_k override, renormalise, extra behaviour)
VARIANTS = [
    "SPARSE_TOP1", "SPARSE_TOP2", "SPARSE_TOPK", "SOFT_MIXTURE", "HIERARCHICAL", "MOMOE", "EXPERT_CHOICE", "HASH_ROUTED",
    "CROSS_LAYER", "MULTIMODAL", "MMOE", "DEEPSEEK_MOE", "BASE_LAYER", "DENSE_MOE", "SHARED_EXPERT", "RESIDUAL_MOE",
    "GATING_DROPOUT", "DOMAIN_MOE", "PRODUCT_KEY", "ATTENTION_MOE", "LOWRANK_MOE", "MAMBA_MOE", "QUANTIZED_INT8_MOE",
    "QUANT_MOE", "Q1_MOE", "Q8_MOE", "Q4_MOE",
]


class _LinearAG(torch.autograd.Function):
    """y = x W^T through the tcgen05 GEMM with ordinary autograd gradients (small layers: router, adapters)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        if w.shape[0] % 8:                       # rows of [T, N] must be 16-byte multiples for the TMA path (e.g. 4 experts)
            return x @ w.t()
        return F.gemm(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        if w.shape[0] % 8:
            return dy @ w, (dy.float().t() @ x.float()).to(w.dtype)
        dx = F.gemm(dy, w, b_mn=True)
        dw = F.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32)
        return dx, dw.to(w.dtype)


class AttentionBlockFn(torch.autograd.Function):
    """Attention half of a block (norm -> qkv -> rope -> flash attention -> o + residual) as one node."""

    @staticmethod
    def forward(ctx, h, blk, B, S, rope, *params):
        cfg = blk.cfg
        Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        a, _, rstd = F.rmsnorm_fwd(h, blk.attention_norm, cfg.norm_eps)
        qkv = F.gemm(a, blk.qkv)
        if rope is not None:
            F.rope_(qkv, rope[0], rope[1], Hq + Hkv, D, S)
        o, lse = F.attn_fwd(qkv, qkv, qkv, B, S, Hq, Hkv, D, k_col0=Hq * D, v_col0=(Hq + Hkv) * D)
        out = F.gemm(o, blk.o, residual=h)
        ctx.blk, ctx.dims, ctx.rope = blk, (B, S), rope
        ctx.save_for_backward(h, rstd, a, qkv, o, lse)
        return out

    @staticmethod
    def backward(ctx, dout):
        blk = ctx.blk
        cfg = blk.cfg
        B, S = ctx.dims
        Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        h, rstd, a, qkv, o, lse = ctx.saved_tensors
        dout = dout.contiguous()
        for p in (blk.attention_norm, blk.qkv, blk.o):
            _ensure_main_grad(p)
        d_o = F.gemm(dout, blk.o, b_mn=True)
        F.gemm(dout, o, a_mn=True, b_mn=True, out=blk.o.main_grad, accumulate=True)
        d_qkv = torch.empty_like(qkv)
        F.attn_bwd(qkv, qkv, qkv, o, d_o, lse, d_qkv, B, S, Hq, Hkv, D, k_col0=Hq * D, v_col0=(Hq + Hkv) * D)
        if ctx.rope is not None:
            F.rope_(d_qkv, ctx.rope[0], ctx.rope[1], Hq + Hkv, D, S, backward=True)
        d_a = F.gemm(d_qkv, blk.qkv, b_mn=True)
        F.gemm(d_qkv, a, a_mn=True, b_mn=True, out=blk.qkv.main_grad, accumulate=True)
        dh = F.rmsnorm_bwd(d_a, h, blk.attention_norm, rstd, blk.attention_norm.main_grad, dout)
        return (dh, None, None, None, None) + (None,) * 3


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, eps):
        y, _, rstd = F.rmsnorm_fwd(h, w, eps)
        ctx.save_for_backward(h, rstd)
        ctx.w = w
        return y

    @staticmethod
    def backward(ctx, dy):
        h, rstd = ctx.saved_tensors
        _ensure_main_grad(ctx.w)
        return F.rmsnorm_bwd(dy.contiguous(), h, ctx.w, rstd, ctx.w.main_grad, None), None, None


class MoEBlock(nn.Module):
    def __init__(self, cfg: MoEConfig, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        H, D, Fe, E = cfg.hidden_size, cfg.head_dim, cfg.expert_hidden_size, cfg.num_experts
        nq, nkv = cfg.num_heads * D, cfg.num_kv_heads * D
        kw = dict(device=device, dtype=dtype)
        self.attention_norm = nn.Parameter(torch.ones(H, **kw))
        self.qkv = nn.Parameter(torch.empty(nq + 2 * nkv, H, **kw))
        self.o = nn.Parameter(torch.empty(H, nq, **kw))
        self.ffn_norm = nn.Parameter(torch.ones(H, **kw))
        self.router = nn.Parameter(torch.empty(E, H, **kw))
        self.gate_up = nn.Parameter(torch.empty(E, 2 * Fe, H, **kw))   # [gate | up] rows per expert
        self.down = nn.Parameter(torch.empty(E, H, Fe, **kw))
        ns = cfg.num_shared_experts
        self.shared_gate_up = nn.Parameter(torch.empty(2 * Fe * ns, H, **kw)) if ns else None
        self.shared_down = nn.Parameter(torch.empty(H, Fe * ns, **kw)) if ns else None
        self.router_bias = None   # DEEPSEEK_MOE: non-learned balancing bias, nudged by -0.001 per pick
        self.ep = None            # parallel.ep.ExpertParallel when experts are sharded across ranks
        # variant-specific parameters (reference: src/model/moe_variants.cpp:990-1150)
        variant = cfg.variant.upper()
        self.router_k = self.lowrank_down = self.lowrank_up = self.domain_classifier = self.task_gates = self.ssm_proj = None
        self.task_id = 0                          # MMOE: which task's gate routes (set by the caller per batch)
        if variant == "MMOE":                     # one gate per task over the shared experts
            self.num_tasks = max(1, getattr(cfg, "num_tasks", 0) or 2)
            self.task_gates = nn.Parameter(torch.empty(self.num_tasks * E, H, **kw))
        elif variant == "MAMBA_MOE":              # a state projection, tiled back over the hidden dimension, is added to x
            st = 64 if H % 64 == 0 else max(8, H // 8 // 8 * 8)
            while H % st:
                st -= 8
            self.ssm_proj = nn.Parameter(torch.empty(max(st, 8), H, **kw))
        if variant == "ATTENTION_MOE":            # routing score = (x Wq) * (x Wk) * sqrt(H), element-wise per expert
            self.router_k = nn.Parameter(torch.empty(E, H, **kw))
        elif variant == "LOWRANK_MOE":            # router and experts see x pushed through a rank-r bottleneck
            r = max(8, min(256, H // 2) // 8 * 8)
            self.lowrank_down = nn.Parameter(torch.empty(r, H, **kw))
            self.lowrank_up = nn.Parameter(torch.empty(H, r, **kw))
        elif variant == "DOMAIN_MOE":             # a domain classifier mixes per-domain expert groups
            nd = max(1, min(getattr(cfg, "num_domains", 0) or 4, E))
            while E % nd:
                nd -= 1
            self.num_domains = nd
            self.domain_classifier = nn.Parameter(torch.empty(nd, H, **kw))
        # quantised-output variants: fixed levels, gradients pass straight through
        self.register_buffer("expert_scales", torch.ones(E, device=device, dtype=torch.float32), persistent=False)

    def moe(self, f):
        cfg = self.cfg
        logits = _LinearAG.apply(f, self.router).float()
        variant = cfg.variant.upper()
        k, renorm = cfg.top_k, cfg.renormalize_topk
        if variant == "SPARSE_TOP1":
            k = 1
        elif variant == "SPARSE_TOP2":
            k = 2
        elif variant in ("SOFT_MIXTURE", "DENSE_MOE"):
            k, renorm = cfg.num_experts, False            # every expert, soft-max weights
        elif variant == "HASH_ROUTED":
            # deterministic routing by token content hash: logits replaced by a fixed pseudo-random table
            idx = (f.float().abs().sum(-1) * 1000).long() % cfg.num_experts
            logits = TF.one_hot(idx, cfg.num_experts).float() * 20.0 + 0 * logits
            k = 1
        elif variant == "DEEPSEEK_MOE":
            if self.router_bias is None:
                self.router_bias = torch.zeros(cfg.num_experts, device=f.device)
            logits = logits + self.router_bias
        elif variant == "ATTENTION_MOE":
            logits = logits * _LinearAG.apply(f, self.router_k).float() * math.sqrt(cfg.hidden_size)
        elif variant == "GATING_DROPOUT" and self.training:
            logits = logits + torch.where(torch.rand_like(logits) < 0.1, torch.full_like(logits, -1e4), torch.zeros_like(logits))
        # ---- rules that pick a selection [T, E] first (models/moe_routing.py); the fused expert path then runs on masked logits
        sel = passthrough = None
        E = cfg.num_experts
        if variant == "EXPERT_CHOICE":
            k = min(max(k, 2), E, 8)
            sel = R.expert_choice(logits, cfg.capacity_factor, k)
            renorm = True
        elif variant in ("HIERARCHICAL", "MOMOE"):
            groups = getattr(cfg, "num_groups", 0) or max(1, int(round(E ** 0.5)))
            while E % groups:
                groups -= 1
            top_groups = min(groups, max(1, getattr(cfg, "top_groups", 0) or k))
            sel = R.hierarchical(logits, groups, top_groups, getattr(cfg, "top_experts_per_group", 1) or 1)
            k, renorm = min(8, top_groups * (getattr(cfg, "top_experts_per_group", 1) or 1)), True
        elif variant == "BASE_LAYER":
            sel = R.base_layer(logits)
            k, renorm = 1, True
        elif cfg.capacity_policy.lower() in ("fixed", "token_drop", "token_pass") and variant.startswith("SPARSE"):
            sel, passthrough = R.apply_capacity(logits, min(k, 8), cfg.capacity_factor, cfg.capacity_policy)
            renorm = True
        covered = None
        if sel is not None:
            self.last_sel = sel
            logits, covered = R.masked_logits(logits, sel)
        def experts(x, lg, lo, hi, kk):
            """Fused expert path over experts lo .. hi-1 with their slice of the logits."""
            if (lo, hi) == (0, E):
                gu, dn = self.gate_up, self.down
            else:
                # views of the group's experts; their weight gradients land in the matching rows of the full main_grad
                gu, dn = self.gate_up[lo:hi], self.down[lo:hi]
                for full, part in ((self.gate_up, gu), (self.down, dn)):
                    _ensure_main_grad(full)
                    part.main_grad = full.main_grad[lo:hi]
            if self.ep is not None:
                assert (lo, hi) == (0, E), "grouped variants are not expert-parallel"
                return self.ep.moe_ffn(x, lg, gu, dn, kk, renorm, cfg.act_kernel, cfg.load_balance_weight, cfg.router_z_weight)
            return M.moe_ffn(x, lg.contiguous(), gu, dn, kk, renorm, cfg.act_kernel, cfg.load_balance_weight, cfg.router_z_weight)

        if variant == "PRODUCT_KEY":
            # two key spaces: the first and second half of the experts are routed independently (top-k in each) and the
            # two mixtures are added
            half = max(1, E // 2)
            ya, aux_a, idx_a = experts(f, logits[:, :half], 0, half, min(k, half, 8))
            if E - half > 0:
                yb, aux_b, idx_b = experts(f, logits[:, half:], half, E, min(k, E - half, 8))
                y, aux, idx = ya + yb, aux_a + aux_b, torch.cat([idx_a, idx_b + half], -1)
            else:
                y, aux, idx = ya, aux_a, idx_a
        elif variant == "DOMAIN_MOE":
            nd, per = self.num_domains, E // self.num_domains
            dom = torch.softmax(_LinearAG.apply(f, self.domain_classifier).float(), -1)
            y, aux, idxs = 0.0, 0.0, []
            for d in range(nd):
                yd, ad, idd = experts(f, logits[:, d * per:(d + 1) * per], d * per, (d + 1) * per, min(k, per, 8))
                y = y + yd * dom[:, d:d + 1].to(yd.dtype)
                aux = aux + ad / nd
                idxs.append(idd + d * per)
            idx = torch.cat(idxs, -1)
        else:
            xin = f
            if variant == "LOWRANK_MOE":
                xin = _LinearAG.apply(_LinearAG.apply(f, self.lowrank_down), self.lowrank_up)
                logits = _LinearAG.apply(xin, self.router).float()
            elif variant == "MAMBA_MOE":
                st = self.ssm_proj.shape[0]
                xin = f + _LinearAG.apply(f, self.ssm_proj).repeat(1, cfg.hidden_size // st)   # state j feeds dims d with d % st == j
                logits = _LinearAG.apply(xin, self.router).float()
            elif variant == "MMOE":
                tid = self.task_id if 0 <= self.task_id < self.num_tasks else 0
                logits = _LinearAG.apply(f, self.task_gates[tid * E:(tid + 1) * E]).float()
            y, aux, idx = experts(xin, logits, 0, E, min(k, 8))
        if covered is not None:
            y = y * covered[:, None].to(y.dtype)               # tokens that no expert serves contribute nothing
            if passthrough is not None and bool((passthrough > 0).any()):
                y = y * (1.0 - passthrough)[:, None].to(y.dtype) + f * passthrough[:, None].to(f.dtype)
        # ---- quantised-output variants (reference: moe_variants.cpp:1190-1380): the mixture is snapped to fixed levels,
        # gradients pass straight through
        if variant in ("QUANT_MOE", "Q1_MOE", "Q8_MOE", "Q4_MOE", "QUANTIZED_INT8_MOE"):
            sq = float(self.expert_scales[-1])
            yf = y.float()
            if variant == "QUANTIZED_INT8_MOE":
                y = y * float(self.expert_scales.double().prod())
            else:
                if variant == "QUANT_MOE":
                    q = torch.where(yf * sq > 0.1, sq, torch.where(yf * sq < -0.1, -sq, 0.0))
                elif variant == "Q1_MOE":
                    q = torch.where(yf * sq >= 0, sq, -sq)
                elif variant == "Q8_MOE":
                    q = (torch.round(yf / 0.01).clamp(-128, 127)) * 0.01
                else:
                    q = (torch.round(yf / 0.1).clamp(-8, 7)) * 0.1
                y = y + (q - yf).detach().to(y.dtype)
        if variant == "DEEPSEEK_MOE" and self.training:
            with torch.no_grad():
                self.router_bias -= 0.001 * torch.bincount(idx.reshape(-1).long(), minlength=cfg.num_experts).float() / idx.numel() * cfg.num_experts
        if self.shared_gate_up is not None:
            gu = _LinearAG.apply(f, self.shared_gate_up)
            Fh = gu.shape[1] // 2
            y = y + _LinearAG.apply((TF.silu(gu[:, :Fh].float()) * gu[:, Fh:].float()).to(f.dtype), self.shared_down)
        self.last_idx, self.last_logits, self.last_covered = idx, logits.detach(), covered
        return y, aux

    # ---- sizes (reference: MoEBlock, include/quant/moe_model.h)
    def num_stored_experts(self) -> int:
        return self.gate_up.shape[0]

    def param_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def activated_param_count(self) -> int:
        """Parameters one token touches: everything but the experts it is not routed to."""
        experts = self.gate_up.numel() + self.down.numel()
        k = min(self.cfg.top_k, self.cfg.num_experts)
        return self.param_count() - experts + experts * k // max(1, self.gate_up.shape[0])

    def forward(self, h, B, S, rope):
        h = AttentionBlockFn.apply(h, self, B, S, rope, self.attention_norm, self.qkv, self.o)
        f = _RMSNormFn.apply(h, self.ffn_norm, self.cfg.norm_eps)
        y, aux = self.moe(f)
        if self.cfg.variant.upper() == "RESIDUAL_MOE":
            y = y + f
        return h + y, aux


class MoEModel(DenseModel):
    """Decoder with MoE blocks.  ``forward(ids)`` -> logits; ``loss(ids, labels)`` -> (ce + aux, ce, aux)."""

    def __init__(self, cfg: MoEConfig, device=None, dtype=torch.bfloat16, seed: Optional[int] = 0):
        nn.Module.__init__(self)
        self.cfg = cfg
        H, V = cfg.hidden_size, cfg.vocab_size
        kw = dict(device=device, dtype=dtype)
        self.tok_embeddings = nn.Parameter(torch.empty(V, H, **kw))
        self.pos_embeddings = None
        self.layers = nn.ModuleList([MoEBlock(cfg, device, dtype) for _ in range(cfg.num_layers)])
        if cfg.variant.upper() == "CROSS_LAYER":
            # one pool of experts serves every layer; the routers cycle over num_shared_layers layers
            # (reference: CrossLayerMoE, src/model/moe_variants.cpp:579-614)
            nsl = max(1, getattr(cfg, "num_shared_layers", 0) or cfg.num_layers)
            for i, blk in enumerate(self.layers):
                if i > 0:
                    blk.gate_up, blk.down = self.layers[0].gate_up, self.layers[0].down
                if i >= nsl:
                    blk.router = self.layers[i % nsl].router
        self.norm = nn.Parameter(torch.ones(H, **kw))
        self.norm_bias = None
        self.lm_head = self.tok_embeddings if cfg.tie_embeddings else nn.Parameter(torch.empty(V, H, **kw))
        self.mtp_heads = nn.ParameterList()
        self.activation_checkpointing = False
        self.loss_chunk_tokens = 9472
        self._rope = None
        self.flat = None
        self.last_aux = None
        if seed is not None:
            self.init_weights(seed)

    def hidden_states(self, ids):
        B, S = ids.shape
        rope = self.rope(ids.device)
        h = _EmbedFn.apply(ids, self, self.tok_embeddings)
        aux = 0.0
        for blk in self.layers:
            h, a = blk(h, B, S, rope)
            aux = aux + a
        self.last_aux = aux
        return _FinalNormFn.apply(h, self, self.norm)

    def loss(self, ids, labels, ignore_index=-100):
        logits = self.forward(ids).float()
        ce = TF.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1), ignore_index=ignore_index)
        return ce + self.last_aux, ce, self.last_aux

    def forward_backward(self, ids, labels, loss_scale: float = 1.0, ignore_index: int = -100, label_smoothing=None):
        """Same contract as DenseModel.forward_backward (gradients land in main_grad); returns the CE loss."""
        assert self.flat is not None
        if label_smoothing is None:
            label_smoothing = getattr(self, "loss_label_smoothing", 0.0)
        B, S = ids.shape
        with torch.enable_grad():
            # blocks under autograd (block-level nodes); the head runs as in the dense model: chunked LM head with the
            # cross entropy computed in place, so the full [T, V] logits never exist and no fp32 copy of them is made
            rope = self.rope(ids.device)
            h = _EmbedFn.apply(ids, self, self.tok_embeddings)
            aux = 0.0
            for blk in self.layers:
                h, a = blk(h, B, S, rope)
                aux = aux + a
            self.last_aux = aux
            with torch.no_grad():
                ce, dh = self.head_loss_backward(h.detach(), labels.reshape(-1), loss_scale, ignore_index, label_smoothing)
            if torch.is_tensor(aux) and aux.requires_grad:
                torch.autograd.backward([h, aux * loss_scale], [dh, None])
            else:
                h.backward(dh)
        # parameters that went through ordinary autograd carry .grad; fold it into main_grad
        for p in self.flat.params_list:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None
        return ce.detach()

    def named_tensors(self):
        cfg = self.cfg
        D = cfg.head_dim
        nq, nkv, Fe = cfg.num_heads * D, cfg.num_kv_heads * D, cfg.expert_hidden_size
        out = [("tok_embeddings.weight", self.tok_embeddings.data)]
        for i, l in enumerate(self.layers):
            pre = f"layers.{i}."
            out += [(pre + "attention_norm.weight", l.attention_norm.data), (pre + "ffn_norm.weight", l.ffn_norm.data),
                    (pre + "attention.q_proj.weight", l.qkv.data[:nq]), (pre + "attention.k_proj.weight", l.qkv.data[nq:nq + nkv]),
                    (pre + "attention.v_proj.weight", l.qkv.data[nq + nkv:]), (pre + "attention.o_proj.weight", l.o.data),
                    (pre + "moe.router.weight", l.router.data)]
            for e in range(cfg.num_experts):
                ep = pre + f"moe.expert.{e}."
                out += [(ep + "gate_proj.weight", l.gate_up.data[e, :Fe]), (ep + "up_proj.weight", l.gate_up.data[e, Fe:]),
                        (ep + "down_proj.weight", l.down.data[e])]
            for nm in ("router_k", "lowrank_down", "lowrank_up", "domain_classifier", "task_gates", "ssm_proj"):
                if getattr(l, nm, None) is not None:
                    out.append((pre + f"moe.{nm}.weight", getattr(l, nm).data))
            if l.shared_gate_up is not None:
                Fs = l.shared_gate_up.shape[0] // 2
                out += [(pre + "shared_expert.gate_proj.weight", l.shared_gate_up.data[:Fs]),
                        (pre + "shared_expert.up_proj.weight", l.shared_gate_up.data[Fs:]),
                        (pre + "shared_expert.down_proj.weight", l.shared_down.data)]
        out.append(("norm.weight", self.norm.data))
        if not cfg.tie_embeddings:
            out.append(("lm_head.weight", self.lm_head.data))
        return out

    @classmethod
    def load(cls, path, device="cpu", dtype=torch.float32, strict=True, **moe_kw):
        """Read a ``.quant`` container written by ``save``.  The container's header holds the dense configuration only
        (as the reference's does, src/model/moe_model.cpp:384-440), so the mixture's shape is read off the tensors: the
        number of experts and their width from the ``moe.expert.N`` names, shared experts from theirs; what cannot be
        seen in a file (``top_k``, the variant, loss weights) comes from ``moe_kw`` or the defaults."""
        import re
        from dataclasses import fields
        from ..quant import codec
        from .config import MoEConfig, TransformerConfig
        raw, tensors = codec.load_state(path)
        base = TransformerConfig.from_bytes(raw)
        experts = {int(m.group(1)) for n in tensors for m in [re.match(r"layers\.0\.moe\.expert\.(\d+)\.gate_proj", n)] if m}
        if not experts:
            raise ValueError(f"{path}: no expert tensors (not a mixture-of-experts checkpoint)")
        kw = {f.name: getattr(base, f.name) for f in fields(TransformerConfig)}
        kw["tie_embeddings"] = "lm_head.weight" not in tensors
        fe = tensors["layers.0.moe.expert.0.gate_proj.weight"].numel() // base.hidden_size
        ns = 0
        if "layers.0.shared_expert.gate_proj.weight" in tensors:
            ns = tensors["layers.0.shared_expert.gate_proj.weight"].numel() // base.hidden_size // fe
        kw.update(num_experts=len(experts), expert_hidden_size=fe, num_shared_experts=ns)
        kw.update(moe_kw)
        model = cls(MoEConfig(**kw), device=device, dtype=dtype, seed=None)
        with torch.no_grad():
            for name, dst in model.named_tensors():
                if name not in tensors:
                    if strict:
                        raise KeyError(f"{path}: tensor {name} missing")
                    continue
                src = tensors[name]
                if src.numel() != dst.numel():
                    raise ValueError(f"{name}: {src.numel()} weights in file, {dst.numel()} expected")
                dst.copy_(src.view(dst.shape).to(dst.dtype))
        return model

    # ---- sizes and the expert prefetcher (reference: MoEModel, include/quant/moe_model.h)
    def stored_param_count(self) -> int:
        seen, n = set(), 0
        for p in self.parameters():
            if id(p) not in seen:
                seen.add(id(p))
                n += p.numel()
        return n

    def param_count(self) -> int:
        """Parameters active per token (all experts count in ``stored_param_count``)."""
        inactive = 0
        for l in self.layers:
            experts = l.gate_up.numel() + l.down.numel()
            inactive += experts - experts * min(self.cfg.top_k, self.cfg.num_experts) // max(1, l.gate_up.shape[0])
        return self.stored_param_count() - inactive

    def vocab_size(self) -> int:
        return self.cfg.vocab_size

    def init_prefetcher(self, directory: str, host_slots: int = 8, device_slots: int = 2):
        """An expert prefetcher (disk -> pinned host -> device tiers) sized for this model; ``wire_prefetcher_sources``
        fills its disk tier."""
        from .moe_extras import ExpertPrefetcher
        dev = self.tok_embeddings.device
        self.prefetcher = ExpertPrefetcher(directory, dev, host_slots, device_slots).initialize(self.cfg.num_experts, len(self.layers))
        return self.prefetcher

    def wire_prefetcher_sources(self):
        """Write every expert of every layer to the prefetcher's disk tier."""
        for li, l in enumerate(self.layers):
            for e in range(l.gate_up.shape[0]):
                self.prefetcher.set_expert_segments(li, e, [("gate_up", l.gate_up.data[e]), ("down", l.down.data[e])])
        return self.prefetcher

    def expert_utilization(self):
        """Fraction of routed (token, k) pairs per expert in the last forward, per layer."""
        E = self.cfg.num_experts
        return [torch.bincount(l.last_idx.reshape(-1).long(), minlength=E).float() / max(1, l.last_idx.numel())
                for l in self.layers if hasattr(l, "last_idx")]


@dataclass
class MoEAllConfig:
    """Router / capacity settings shared by every variant (reference MoEAllConfig, include/quant/moe_variants.h:61-123)."""
    num_experts: int = 16
    top_k: int = 2
    expert_hidden: int = 2048
    load_balance_weight: float = 0.01
    router_z_weight: float = 0.001
    capacity_factor: float = 2.0
    capacity_policy: str = "none"           # none | fixed | token_drop | token_pass (see models/moe_routing.py)
    num_shared_experts: int = 0
    num_groups: int = 0                     # HIERARCHICAL / MOMOE: 0 = about sqrt(num_experts)
    num_domains: int = 4                    # DOMAIN_MOE: expert groups mixed by the domain classifier
    num_tasks: int = 2                      # MMOE: gates (one per task) over the shared experts
    num_shared_layers: int = 0              # CROSS_LAYER: routers cycle over this many layers (0 = one per layer)
    top_groups: int = 0                     # 0 = top_k
    top_experts_per_group: int = 1


def create_moe_variant(variant: str, base: TransformerConfig, mcfg: "MoEAllConfig" = None, **model_kw) -> "MoEModel":
    """Factory: a MoEModel of the named variant (any of VARIANTS, case-insensitive) over the dense shape ``base``.
    Reference counterpart: create_moe_variant (src/model/moe_core.cpp:446-551)."""
    name = variant.upper()
    if name not in VARIANTS:
        raise ValueError(f"unknown MoE variant '{variant}' (known: {', '.join(VARIANTS)})")
    m = mcfg or MoEAllConfig()
    import dataclasses
    fields = {f.name for f in dataclasses.fields(TransformerConfig)}
    kw = {k: v for k, v in dataclasses.asdict(base).items() if k in fields}
    shared = m.num_shared_experts or (1 if name == "SHARED_EXPERT" else 0)
    cfg = MoEConfig(**kw, num_experts=m.num_experts, top_k=m.top_k, expert_hidden_size=m.expert_hidden, num_shared_experts=shared,
                    load_balance_weight=m.load_balance_weight, router_z_weight=m.router_z_weight, capacity_factor=m.capacity_factor,
                    capacity_policy=m.capacity_policy, variant=name)
    cfg.num_groups, cfg.top_groups, cfg.top_experts_per_group = m.num_groups, m.top_groups, m.top_experts_per_group
    cfg.num_domains, cfg.num_tasks, cfg.num_shared_layers = m.num_domains, m.num_tasks, m.num_shared_layers
    return MoEModel(cfg, **model_kw)


# ------------------------------------------------------------------------------------------------
# Stand-alone mixture layers under the reference's class names (include/quant/moe_variants.h:144-680): the feed-forward
# half of a block of the named variant, usable inside any other network
# ------------------------------------------------------------------------------------------------
@dataclass
class MoELayerOutput:
    output: torch.Tensor                    # same shape as the input
    aux_loss: torch.Tensor                  # weighted load-balance + z loss (add it to the training loss)
    expert_indices: Optional[torch.Tensor]  # [tokens, k] where the variant routes discretely
    router_logits: Optional[torch.Tensor]


class MoELayer(nn.Module):
    VARIANT = "SPARSE_TOPK"

    def __init__(self, hidden_size: int, cfg: Optional[MoEAllConfig] = None, device=None, dtype=torch.float32, seed: int = 0):
        super().__init__()
        self.config, self.hidden_size = cfg or MoEAllConfig(), hidden_size
        base = TransformerConfig(vocab_size=8, hidden_size=hidden_size, num_layers=1, num_heads=1, ffn_hidden_size=self.config.expert_hidden,
                                 max_seq_len=8)
        host = create_moe_variant(self.VARIANT, base, self.config, device=device, dtype=dtype, seed=seed)
        self.block = host.layers[0]
        for n in ("attention_norm", "qkv", "o", "ffn_norm"):          # the attention half is not part of a mixture layer
            setattr(self.block, n, None)

    @property
    def router_weight(self) -> torch.Tensor: return self.block.router

    @property
    def experts(self):
        """(gate_up [2F, H], down [H, F]) views, one pair per expert."""
        return [(self.block.gate_up[e], self.block.down[e]) for e in range(self.block.gate_up.shape[0])]

    def forward(self, x: torch.Tensor, training: Optional[bool] = None) -> MoELayerOutput:
        if training is not None:
            self.block.train(training)
        flat = x.reshape(-1, self.hidden_size)
        y, aux = self.block.moe(flat)
        if self.VARIANT == "RESIDUAL_MOE":
            y = y + flat
        b = self.block
        return MoELayerOutput(y.view(x.shape), aux, getattr(b, "last_idx", None), getattr(b, "last_logits", None))

    def load_balance_loss(self, gates: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        E = self.config.num_experts
        f = torch.bincount(indices.reshape(-1).long(), minlength=E).float() / max(1, indices.numel())
        return E * (f * gates.float().reshape(-1, E).mean(0)).sum()

    def z_loss(self, logits: torch.Tensor) -> torch.Tensor:
        return (torch.logsumexp(logits.float(), -1) ** 2).mean()

    def compute_capacity(self, T: int) -> int:
        from .moe_routing import capacity_limit
        return capacity_limit(T, self.config.num_experts, self.config.top_k, self.config.capacity_factor)

    def export_weights(self) -> bytes:
        """Every parameter of the layer as little-endian fp32, in ``named_parameters`` order."""
        return b"".join(p.detach().float().cpu().contiguous().numpy().tobytes() for _, p in self.named_parameters())

    def import_weights(self, data: bytes):
        import numpy as np
        a = np.frombuffer(data, dtype="<f4")
        need = sum(p.numel() for p in self.parameters())
        if a.size != need:
            raise ValueError(f"{a.size} values given, the layer holds {need}")
        off = 0
        with torch.no_grad():
            for _, p in self.named_parameters():
                p.copy_(torch.from_numpy(a[off:off + p.numel()].copy()).view(p.shape).to(p.dtype))
                off += p.numel()


def _variant_layer(name: str, variant: str, doc: str):
    return type(name, (MoELayer,), {"VARIANT": variant, "__doc__": doc})


SparseMoE = _variant_layer("SparseMoE", "SPARSE_TOPK", "Top-k routing with load-balance and z losses.")
SoftMoE = _variant_layer("SoftMoE", "SOFT_MIXTURE", "Every expert, soft-max mixing weights.")
HierarchicalMoE = _variant_layer("HierarchicalMoE", "HIERARCHICAL", "Groups first, experts inside the chosen groups second.")
MoMoE = _variant_layer("MoMoE", "MOMOE", "Mixture of mixtures: grouped routing with per-group balance.")
ExpertChoiceMoE = _variant_layer("ExpertChoiceMoE", "EXPERT_CHOICE", "Experts pick their tokens up to a capacity.")
HashMoE = _variant_layer("HashMoE", "HASH_ROUTED", "Routing by a fixed hash of the token: no learned router.")
CrossLayerMoE = _variant_layer("CrossLayerMoE", "CROSS_LAYER", "One expert pool shared by several layers.")
MultiModalMoE = _variant_layer("MultiModalMoE", "MULTIMODAL", "Top-k routing over experts shared by the modalities.")
MMoE = _variant_layer("MMoE", "MMOE", "Multi-gate: one router per task over shared experts (set ``block.task_id``).")
DeepSeekMoE = _variant_layer("DeepSeekMoE", "DEEPSEEK_MOE", "Fine-grained experts with a non-learned balancing bias.")
BaseLayerMoE = _variant_layer("BaseLayerMoE", "BASE_LAYER", "Balanced assignment: every expert gets the same number of tokens.")
DenseMoE = _variant_layer("DenseMoE", "DENSE_MOE", "All experts for every token.")
SharedExpertMoE = _variant_layer("SharedExpertMoE", "SHARED_EXPERT", "Routed experts plus one expert every token uses.")
ResidualMoE = _variant_layer("ResidualMoE", "RESIDUAL_MOE", "The mixture is added to its own input.")
GatingDropoutMoE = _variant_layer("GatingDropoutMoE", "GATING_DROPOUT", "Router logits are dropped at random while training.")
DomainMoE = _variant_layer("DomainMoE", "DOMAIN_MOE", "A domain classifier mixes per-domain expert groups.")
ProductKeyMoE = _variant_layer("ProductKeyMoE", "PRODUCT_KEY", "Expert index from the product of two half-size key sets.")
AttentionMoE = _variant_layer("AttentionMoE", "ATTENTION_MOE", "Routing scores from a query-key product.")
LowRankMoE = _variant_layer("LowRankMoE", "LOWRANK_MOE", "Router and experts behind a low-rank bottleneck.")
MambaMoE = _variant_layer("MambaMoE", "MAMBA_MOE", "A state projection is added to the routed input.")
QuantizedINT8MoE = _variant_layer("QuantizedINT8MoE", "QUANTIZED_INT8_MOE", "Mixture output on a per-expert 8-bit grid.")
QuantMoE = _variant_layer("QuantMoE", "QUANT_MOE", "Mixture output snapped to 4-bit levels.")
Quant1MoE = _variant_layer("Quant1MoE", "Q1_MOE", "Mixture output snapped to ternary levels.")
Q8MoE = _variant_layer("Q8MoE", "Q8_MOE", "Mixture output snapped to 8-bit levels.")
Q4MoE = _variant_layer("Q4MoE", "Q4_MOE", "Mixture output snapped to 4-bit codebook levels.")
MOE_LAYER_CLASSES = {c.VARIANT: c for c in (SparseMoE, SoftMoE, HierarchicalMoE, MoMoE, ExpertChoiceMoE, HashMoE, CrossLayerMoE, MultiModalMoE, MMoE,
                                            DeepSeekMoE, BaseLayerMoE, DenseMoE, SharedExpertMoE, ResidualMoE, GatingDropoutMoE, DomainMoE,
                                            ProductKeyMoE, AttentionMoE, LowRankMoE, MambaMoE, QuantizedINT8MoE, QuantMoE, Quant1MoE, Q8MoE, Q4MoE)}
