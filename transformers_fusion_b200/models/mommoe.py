"""Mixture-of-modality MoE: a router that also classifies the modality of every token, experts reserved per modality,
and a cross-modal attention step in every block.

Reference counterparts: Modality, RouterOutput, TopKRouter, CrossModalAttention, ModalityExpertFFN, MoMBlock, MoMMoEConfig,
MoMMoE (include/quant/mommoe_block.h:41-300, src/model/mommoe_block.cpp)."""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as TF
from torch import nn


class Modality(enum.IntEnum):
    TEXT = 0
    VISION = 1
    AUDIO = 2
    IMAGE_GEN = 3
    VIDEO_GEN = 4
    OCR = 5
    EMBEDDING = 6
    CROSS_MODAL = 7
    META_COGNITION = 8


NUM_MODALITIES = len(Modality)


def modality_name(m) -> str:
    return Modality(int(m)).name


@dataclass
class RouterOutput:
    gates: torch.Tensor              # [T, E] softmax probabilities
    indices: torch.Tensor            # [T, k]
    weights: torch.Tensor            # [T, k], rows sum to 1
    modality_probs: torch.Tensor     # [T, M]
    dominant_modality: Modality
    load_balance_loss: torch.Tensor
    z_loss: torch.Tensor
    num_activated_experts: int


class TopKRouter(nn.Module):
    """Expert logits = learned gate + a bias from the token's modality towards the experts reserved for it."""

    def __init__(self, hidden: int, num_experts: int, top_k: int, expert_modality: List[int], num_modalities: int = NUM_MODALITIES):
        super().__init__()
        self.k, self.E = top_k, num_experts
        self.gate = nn.Linear(hidden, num_experts, bias=False)
        self.modality_head = nn.Linear(hidden, num_modalities, bias=False)
        affinity = torch.zeros(num_modalities, num_experts)
        for e, m in enumerate(expert_modality):
            affinity[m, e] = 1.0
        self.register_buffer("affinity", affinity)
        self.affinity_scale = nn.Parameter(torch.tensor(2.0))

    def forward(self, x: torch.Tensor, modality_hints: Optional[torch.Tensor] = None) -> RouterOutput:
        mp = torch.softmax(self.modality_head(x).float(), -1)
        if modality_hints is not None:                       # known modality: one-hot instead of the classifier
            mp = TF.one_hot(modality_hints.reshape(-1).long(), mp.shape[-1]).float()
        logits = self.gate(x).float() + self.affinity_scale * (mp @ self.affinity)
        gates = torch.softmax(logits, -1)
        w, idx = gates.topk(self.k, -1)
        w = w / w.sum(-1, keepdim=True)
        T = x.shape[0]
        f = torch.bincount(idx.reshape(-1), minlength=self.E).float() / max(1, T * self.k)
        lb = self.E * (f * gates.mean(0)).sum()
        z = (torch.logsumexp(logits, -1) ** 2).mean()
        dom = Modality(int(mp.mean(0).argmax()))
        return RouterOutput(gates, idx, w, mp, dom, lb, z, int((f > 0).sum()))


def _router_api():
    """The reference's stand-alone pieces of the router (include/quant/mommoe_block.h:88-106): the two auxiliary losses as
    functions of given routing results, the modality classifier, and plain accessors."""
    def load_balance_loss(self, gates: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        f = torch.bincount(indices.reshape(-1), minlength=self.E).float() / max(1, indices.numel())
        return self.E * (f * gates.float().reshape(-1, self.E).mean(0)).sum()

    def z_loss(self, logits: torch.Tensor) -> torch.Tensor:
        return (torch.logsumexp(logits.float(), -1) ** 2).mean()

    def classify_modality(self, hidden: torch.Tensor) -> Modality:
        """The modality the classifier head gives the highest mean probability over the given tokens."""
        mp = torch.softmax(self.modality_head(hidden.reshape(-1, hidden.shape[-1])).float(), -1)
        return Modality(int(mp.mean(0).argmax()))

    TopKRouter.load_balance_loss, TopKRouter.z_loss, TopKRouter.classify_modality = load_balance_loss, z_loss, classify_modality
    TopKRouter.gate_weight = lambda self: self.gate.weight
    TopKRouter.modality_head_weight = lambda self: self.modality_head.weight
    TopKRouter.num_experts = lambda self: self.E
    TopKRouter.top_k = lambda self: self.k


_router_api()


class CrossModalAttention(nn.Module):
    """Tokens attend to per-modality summaries of the sequence (mean of the tokens weighted by their modality
    probability): M keys per sequence, so the cost is linear in the sequence length."""

    def __init__(self, hidden: int, num_heads: int, num_modalities: int = NUM_MODALITIES):
        super().__init__()
        self.h, self.d = num_heads, hidden // num_heads
        self.q, self.kv, self.o = nn.Linear(hidden, hidden, bias=False), nn.Linear(hidden, 2 * hidden, bias=False), nn.Linear(hidden, hidden, bias=False)
        self.M = num_modalities

    def forward(self, x: torch.Tensor, modality_probs: torch.Tensor) -> torch.Tensor:
        B, S, H = x.shape
        mp = modality_probs.view(B, S, self.M).to(x.dtype)
        summ = torch.einsum("bsm,bsh->bmh", mp, x) / mp.sum(1).clamp(min=1e-6)[..., None]        # [B, M, H]
        q = self.q(x).view(B, S, self.h, self.d).transpose(1, 2)
        k, v = self.kv(summ).chunk(2, -1)
        k, v = k.view(B, self.M, self.h, self.d).transpose(1, 2), v.view(B, self.M, self.h, self.d).transpose(1, 2)
        a = torch.softmax((q @ k.transpose(-1, -2)).float() / math.sqrt(self.d), -1).to(x.dtype)
        return self.o((a @ v).transpose(1, 2).reshape(B, S, H))


class ModalityExpertFFN(nn.Module):
    def __init__(self, hidden: int, ffn_hidden: int, modality: Modality):
        super().__init__()
        self.modality = modality
        self.gate_up, self.down = nn.Linear(hidden, 2 * ffn_hidden, bias=False), nn.Linear(ffn_hidden, hidden, bias=False)

    def forward(self, x):
        g, u = self.gate_up(x).chunk(2, -1)
        return self.down(TF.silu(g) * u)


def _projection_views():
    """The reference names the projections one by one (include/quant/mommoe_block.h:140-180); here gate / up and key / value
    are stored fused for one GEMM each, so these return views of the fused weights (writes go through)."""
    ModalityExpertFFN.gate_proj = lambda self: self.gate_up.weight[: self.gate_up.out_features // 2]
    ModalityExpertFFN.up_proj = lambda self: self.gate_up.weight[self.gate_up.out_features // 2:]
    ModalityExpertFFN.down_proj = lambda self: self.down.weight
    ModalityExpertFFN.specialization = lambda self: self.modality
    CrossModalAttention.q_proj = lambda self: self.q.weight
    CrossModalAttention.k_proj = lambda self: self.kv.weight[: self.kv.out_features // 2]
    CrossModalAttention.v_proj = lambda self: self.kv.weight[self.kv.out_features // 2:]
    CrossModalAttention.o_proj = lambda self: self.o.weight


_projection_views()


class _RMS(nn.Module):
    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(d)), eps

    def forward(self, x):
        f = x.float()
        return (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


@dataclass
class MoMOutput:
    hidden: torch.Tensor
    routing: RouterOutput
    cross_modal_output: torch.Tensor


class MoMBlock(nn.Module):
    def __init__(self, hidden, num_heads, ffn_hidden, num_experts, top_k, expert_modality, num_modalities=NUM_MODALITIES):
        super().__init__()
        self.h = num_heads
        self.attention_norm, self.moe_norm = _RMS(hidden), _RMS(hidden)
        self.qkv, self.o = nn.Linear(hidden, 3 * hidden, bias=False), nn.Linear(hidden, hidden, bias=False)
        self.cross_modal_attn = CrossModalAttention(hidden, num_heads, num_modalities)
        self.router = TopKRouter(hidden, num_experts, top_k, expert_modality, num_modalities)
        self.experts = nn.ModuleList(ModalityExpertFFN(hidden, ffn_hidden, Modality(m)) for m in expert_modality)

    def self_attention(self, a: torch.Tensor) -> torch.Tensor:
        """Causal multi-head self-attention of already normalised states [B, S, H] (the block's first sub-layer, without
        the residual)."""
        B, S, H = a.shape
        q, k, v = self.qkv(a).view(B, S, 3, self.h, H // self.h).permute(2, 0, 3, 1, 4)
        return self.o(TF.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, H))

    def forward(self, x, modality_hints=None) -> MoMOutput:
        B, S, H = x.shape
        x = x + self.self_attention(self.attention_norm(x))
        f = self.moe_norm(x)
        r = self.router(f.reshape(B * S, H), modality_hints)
        cross = self.cross_modal_attn(f, r.modality_probs)
        x = x + cross
        flat, out = f.reshape(B * S, H), torch.zeros(B * S, H, dtype=x.dtype, device=x.device)
        for e, expert in enumerate(self.experts):
            tok, slot = (r.indices == e).nonzero(as_tuple=True)
            if tok.numel():
                out.index_add_(0, tok, expert(flat[tok]) * r.weights[tok, slot].to(x.dtype)[:, None])
        return MoMOutput(x + out.view(B, S, H), r, cross)


@dataclass
class MoMMoEConfig:
    hidden_size: int = 2048
    num_heads: int = 16
    ffn_hidden: int = 8192
    num_layers: int = 24
    num_experts: int = 8
    top_k: int = 2
    vocab_size: int = 32000
    max_seq_len: int = 1 << 20
    num_modalities: int = NUM_MODALITIES
    text_experts: int = 4
    vision_experts: int = 1
    audio_experts: int = 1
    image_gen_experts: int = 1
    video_gen_experts: int = 1

    def expert_modality(self) -> List[int]:
        m = ([Modality.TEXT] * self.text_experts + [Modality.VISION] * self.vision_experts + [Modality.AUDIO] * self.audio_experts +
             [Modality.IMAGE_GEN] * self.image_gen_experts + [Modality.VIDEO_GEN] * self.video_gen_experts)
        if len(m) != self.num_experts:
            raise ValueError(f"per-modality expert counts sum to {len(m)}, num_experts is {self.num_experts}")
        return [int(x) for x in m]


class MoMMoE(nn.Module):
    def __init__(self, cfg: Optional[MoMMoEConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or MoMMoEConfig()
        em = cfg.expert_modality()
        self.embeddings = nn.Embedding(cfg.vocab_size, cfg.hidden_size)          # LM head tied to it
        self.layers = nn.ModuleList(MoMBlock(cfg.hidden_size, cfg.num_heads, cfg.ffn_hidden, cfg.num_experts, cfg.top_k, em,
                                             cfg.num_modalities) for _ in range(cfg.num_layers))
        self.final_norm = _RMS(cfg.hidden_size)
        self._util = torch.zeros(cfg.num_experts)
        self.aux_loss = torch.zeros(())

    def forward(self, input_ids, modality_hints=None):
        x = self.embeddings(input_ids)
        aux, util = 0.0, torch.zeros(self.cfg.num_experts, device=x.device)
        for blk in self.layers:
            out = blk(x, modality_hints)
            x = out.hidden
            aux = aux + 0.01 * out.routing.load_balance_loss + 0.001 * out.routing.z_loss
            util += torch.bincount(out.routing.indices.reshape(-1), minlength=self.cfg.num_experts).float()
        self.aux_loss, self._util = aux, (util / util.sum().clamp(min=1)).detach().cpu()
        return self.final_norm(x) @ self.embeddings.weight.t()

    @torch.no_grad()
    def generate(self, prompt_ids, max_new_tokens: int, temperature: float = 1.0, top_k: int = 50, generator=None):
        ids = prompt_ids.clone()
        for _ in range(max_new_tokens):
            lg = self(ids)[:, -1].float()
            if temperature <= 0:
                nxt = lg.argmax(-1, keepdim=True)
            else:
                v, i = (lg / temperature).topk(min(top_k, lg.shape[-1]), -1)
                nxt = i.gather(1, torch.multinomial(torch.softmax(v, -1), 1, generator=generator))
            ids = torch.cat([ids, nxt], 1)
        return ids

    def config(self) -> MoMMoEConfig: return self.cfg

    def total_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def active_parameters(self) -> int:
        per_expert = sum(p.numel() for p in self.layers[0].experts[0].parameters())
        return self.total_parameters() - self.cfg.num_layers * (self.cfg.num_experts - self.cfg.top_k) * per_expert

    def expert_utilization(self) -> List[float]:
        return self._util.tolist()
