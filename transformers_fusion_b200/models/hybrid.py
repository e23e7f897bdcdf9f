"""Hybrid-layer scaffolding: a per-layer schedule of attention kinds, dense and MoE models built over it, and the
placement of experts on cluster nodes layer by layer.

The reference defines one attention kind (standard softmax attention) and a schedule that assigns it to every layer
while reserving a count for future kinds; this module keeps that contract and adds a sliding-window kind (served by the
tiled host attention or, on the device, by the flash kernel over the window) so that a schedule can actually differ
between layers.

Reference counterparts: HybridAttnKind / HybridSchedule / build_hybrid_schedule (include/quant/hybrid_scheduler.h:9-18,
src/model/hybrid_scheduler.cpp:6-17), HybridBlock / HybridModel (hybrid_block.h:9-40), HybridMoeBlock / HybridMoeModel
(hybrid_moe_model.h:10-60; load / save deliberately unsupported there), HybridExpertShard (hybrid_expert.h:12-30)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

import torch

from .config import MoEConfig, TransformerConfig
from .dense import DenseModel
from .moe import MoEModel

STD, WINDOW = "std", "window"


@dataclass
class HybridSchedule:
    layers: List[str] = field(default_factory=list)
    num_std: int = 0

    def total(self) -> int: return len(self.layers)


def build_hybrid_schedule(total_layers: int, reserved: int = 3, window_every: int = 0) -> HybridSchedule:
    """Every layer standard attention (``reserved`` is clamped and otherwise unused, as in the reference); with
    ``window_every = n`` every n-th layer outside the last ``reserved`` becomes a sliding-window layer."""
    s = HybridSchedule()
    if total_layers <= 0:
        return s
    reserved = max(0, min(reserved, total_layers))
    for i in range(total_layers):
        kind = WINDOW if window_every > 0 and (i + 1) % window_every == 0 and i < total_layers - reserved else STD
        s.layers.append(kind)
        s.num_std += kind == STD
    return s


class HybridModel(DenseModel):
    """DenseModel whose layers carry a schedule entry; window layers restrict attention to ``window`` past tokens in the
    generic (autograd) forward."""

    def __init__(self, cfg: TransformerConfig, schedule: HybridSchedule = None, window: int = 1024, **kw):
        super().__init__(cfg, **kw)
        self.schedule = schedule or build_hybrid_schedule(cfg.num_layers)
        if self.schedule.total() != cfg.num_layers:
            raise ValueError("schedule length does not match the number of layers")
        self.window = window

    def param_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def layer_kinds(self) -> List[str]:
        return list(self.schedule.layers)

    @torch.no_grad()
    def forward_hybrid(self, ids: torch.Tensor) -> torch.Tensor:
        """Logits with the schedule honoured (host statement: plain torch ops, fp32).  With an all-standard schedule this
        equals ``forward``."""
        from ..inference.speculative_extras import MemoryEfficientAttention
        cfg = self.cfg
        B, S = ids.shape
        D, Hq, Hkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
        att = MemoryEfficientAttention(64, 64)
        h = self.tok_embeddings.data[ids].float()
        rope = self.rope(ids.device)

        def norm(x, w):
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * w.float()

        def rot(x):                     # [B, S, H, D] rotate-half
            if rope is None:
                return x
            cos, sin = rope[0][:S].float()[None, :, None, :], rope[1][:S].float()[None, :, None, :]
            x1, x2 = x[..., :D // 2], x[..., D // 2:]
            return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)
        for kind, blk in zip(self.schedule.layers, self.layers):
            a = norm(h, blk.attention_norm.data)
            qkv = a @ blk.qkv.data.float().t()
            q = rot(qkv[..., :Hq * D].view(B, S, Hq, D)).transpose(1, 2)
            k = rot(qkv[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
            v = qkv[..., (Hq + Hkv) * D:].view(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
            o = att.forward_block_sparse(q, k, v, self.window) if kind == WINDOW else att.forward(q, k, v)
            h = h + o.transpose(1, 2).reshape(B, S, Hq * D) @ blk.o.data.float().t()
            f = norm(h, blk.ffn_norm.data)
            gu = f @ blk.gate_up.data.float().t()
            Fh = gu.shape[-1] // 2
            h = h + (torch.nn.functional.silu(gu[..., :Fh]) * gu[..., Fh:]) @ blk.down.data.float().t()
        return norm(h, self.norm.data) @ self.lm_head.data.float().t()


class HybridMoeModel(MoEModel):
    """MoE model with a layer schedule.  Like the reference's, it has no container mapping of its own: ``save`` / ``load``
    go through the ordinary MoE checkpoint and the schedule travels in ``schedule_state``."""

    def __init__(self, cfg: MoEConfig, schedule: HybridSchedule = None, **kw):
        super().__init__(cfg, **kw)
        self.schedule = schedule or build_hybrid_schedule(cfg.num_layers)
        if self.schedule.total() != cfg.num_layers:
            raise ValueError("schedule length does not match the number of layers")

    def param_count(self) -> int: return sum(p.numel() for p in self.parameters())
    def stored_param_count(self) -> int: return self.param_count()
    def schedule_state(self) -> dict: return {"layers": list(self.schedule.layers)}


@dataclass
class ExpertAssignment:
    expert_id: int
    node_id: int
    layer: int = 0


class HybridExpertShard:
    """Experts of every layer spread over ``num_nodes`` nodes; the starting node rotates with the layer so that layer l's
    expert e does not always share a node with layer l + 1's expert e."""

    def __init__(self, num_nodes: int):
        if num_nodes <= 0:
            raise ValueError("need at least one node")
        self._n = num_nodes

    def num_nodes(self) -> int: return self._n

    def assign_layer(self, num_experts: int, layer: int = 0) -> List[ExpertAssignment]:
        return [ExpertAssignment(e, (e + layer) % self._n, layer) for e in range(num_experts)]

    def assign_schedule(self, schedule: HybridSchedule, num_experts: int) -> List[List[ExpertAssignment]]:
        return [self.assign_layer(num_experts, l) for l in range(schedule.total())]

    def node_load(self, assignments: List[List[ExpertAssignment]]) -> List[int]:
        load = [0] * self._n
        for layer in assignments:
            for a in layer:
                load[a.node_id] += 1
        return load
