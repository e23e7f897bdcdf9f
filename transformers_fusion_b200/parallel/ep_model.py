"""Expert-parallel training of the MoE model: every rank keeps the attention / norm / router / embedding weights
(replicated, data parallel) and E / W of the experts of every layer; tokens travel to the experts' owners and back
through the fused dispatch / combine kernels over NVLink peer memory (``parallel.ep.ExpertParallel``).

Gradients: replicated tensors are averaged over the ranks; an expert's weights see the tokens of all ranks already, so
their gradients are only divided by the world size (each rank's loss is the mean over its own tokens, the objective is
the mean over ranks).

Reference counterparts: ExpertParallel (round-robin experts, replicated tokens, all-reduce combine;
src/model/moe_model.cpp:508-700), ExpertParallelManager / assign_experts_to_nodes (src/model/expert_parallel.cpp:319)."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
from torch import nn

from .ep import ExpertParallel


def attach_expert_parallel(model, symm, rank: int, world: int, max_tokens: int, resident: bool = True,
                           capacity_factor: Optional[float] = None) -> List[nn.Parameter]:
    """Cuts every MoE block's expert tensors down to this rank's contiguous block of experts, attaches the dispatch /
    combine object, and rebuilds the flat parameter buffer.  Returns the expert parameters (the rest is replicated).
    ``resident`` (every layer owns its buffers and each forward is followed by its backward): dispatched rows and expert
    outputs stay in the symmetric buffers between forward and backward; pass False for schedules that run a layer's
    forward twice before its backward (recomputation, interleaved micro-batches).  ``capacity_factor`` sizes the
    per-rank expert buffers as a multiple of the balanced load (max_tokens * top_k rows); the default provisions for
    every token of every rank landing on one rank."""
    cfg = model.cfg
    E = cfg.num_experts
    if E % world:
        raise ValueError("the number of experts must divide by the expert-parallel degree")
    El = E // world
    experts = []
    for blk in model.layers:
        if not hasattr(blk, "router"):
            continue
        blk.gate_up = nn.Parameter(blk.gate_up.data[rank * El:(rank + 1) * El].clone())
        blk.down = nn.Parameter(blk.down.data[rank * El:(rank + 1) * El].clone())
        blk.ep = ExpertParallel(symm, rank, world, E, cfg.hidden_size, max_tokens, min(cfg.top_k, 8),
                                capacity_factor=capacity_factor, resident=resident)
        experts += [blk.gate_up, blk.down]
    model.flat = None
    model.flatten()
    return experts


class EPTrainer:
    """Fused AdamW (fp32 masters, one kernel over the flat buffer) over the replicated tensors and this rank's experts.
    The clipping norm is global: the replicated part once plus every rank's expert part."""

    def __init__(self, model, expert_params: List[nn.Parameter], lr=3e-4, weight_decay=0.01, max_grad_norm=1.0, group=None,
                 replica_group=None, replicas: int = 1):
        """``group``: every rank of the job (the replicated tensors are averaged over it).  When the expert-parallel
        degree is smaller than the job (``replicas`` = world / ep copies of every expert), ``replica_group`` holds the
        ranks that own the same experts as this one: their expert gradients are summed over it."""
        from ..trainer.fused_optim import FlatAdamW
        self.model, self.group = model, group
        self.replica_group, self.replicas = replica_group, max(1, int(replicas))
        ids = {id(p) for p in expert_params}
        self.experts = list(expert_params)
        self.shared = [p for p in model.parameters() if id(p) not in ids]
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._runs = None
        self.opt = FlatAdamW(model.flat, lr=lr, weight_decay=weight_decay, max_grad_norm=max_grad_norm,
                             norm_reduce=self._norm_reduce if self.world > 1 else None)

    def _shared_runs(self):
        """The replicated tensors' gradients as maximal contiguous slices of the flat gradient buffer, so that the
        all-reduce count is the number of runs between expert tensors, not the number of tensors."""
        if self._runs is None:
            flat = self.model.flat.grads
            base, esz = flat.data_ptr(), flat.element_size()
            spans = sorted(((p.main_grad.data_ptr() - base) // esz, p.main_grad.numel()) for p in self.shared)
            taken = sorted((p.main_grad.data_ptr() - base) // esz for p in self.experts)
            runs = []
            for off, n in spans:
                assert 0 <= off and off + n <= flat.numel()
                end = runs[-1][0] + runs[-1][1] if runs else -1
                # alignment padding between two replicated tensors is zero on every rank: the run may span it
                if runs and off >= end and not any(end <= t < off for t in taken) and off - end < 4096:
                    runs[-1][1] = off + n - runs[-1][0]
                else:
                    runs.append([off, n])
            self._runs = [flat[o:o + n] for o, n in runs]
        return self._runs

    def _norm_reduce(self, sumsq):
        """sumsq holds this rank's total (replicated + own experts); the result is replicated + every rank's experts.
        Both terms come out of one all-reduce, so every rank gets the same bits and hence the same clipping factor
        (a rank-local sum would differ in rounding and let the replicated weights drift apart)."""
        own = torch.stack([p.main_grad.pow(2).sum() for p in self.experts]).sum().reshape(1)
        v = torch.cat([sumsq.reshape(1) - own, own])
        dist.all_reduce(v, group=self.group)
        # the replicated part was counted by every rank, each distinct expert by each of its `replicas` owners
        sumsq.copy_((v[0] / self.world + v[1] / self.replicas).reshape(sumsq.shape))

    @property
    def grad_norm(self) -> float:
        return float(self.opt.grad_norm)

    def train_step(self, ids, labels, lr: Optional[float] = None) -> float:
        m, W = self.model, self.world
        loss = m.forward_backward(ids, labels)
        lt = loss.detach().float().reshape(1).clone()
        if W > 1:
            for g in self._shared_runs():
                dist.all_reduce(g, group=self.group)
            if self.replicas > 1:
                for p in self.experts:
                    dist.all_reduce(p.main_grad, group=self.replica_group)
            m.flat.grads.div_(W)
            dist.all_reduce(lt, group=self.group)
        self.opt.step(lr)                                   # clips, updates, refreshes the bf16 weights, zeroes the gradients
        return float(lt) / W
