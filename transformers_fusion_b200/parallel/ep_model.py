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


# =====================================================================================================================
# Replicated-token expert parallelism: the reference's algorithm, on library collectives
# =====================================================================================================================
class _SumOverRanks(torch.autograd.Function):
    """y = sum over ranks of the partial outputs.  Every rank holds the same tokens and computes the same loss from the
    same y, so the gradient of each partial output is the gradient of y itself."""

    @staticmethod
    def forward(ctx, y, group):
        y = y.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, dy):
        return dy, None


class _GradSumOverRanks(torch.autograd.Function):
    """Identity whose gradient is summed over the ranks: the input feeds every rank's partial mixture."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dx):
        dx = dx.contiguous().clone()
        dist.all_reduce(dx, group=ctx.group)
        return dx, None


class _ReplicatedTokenFFN:
    """Stand-in for the device dispatch / combine object of a block (``blk.ep``): every rank routes ALL tokens, runs the
    experts it holds on the rows routed to them and the partial mixtures are summed over the ranks."""

    def __init__(self, rank: int, world: int, num_experts: int, group=None):
        self.rank, self.world, self.E, self.group = rank, world, num_experts, group
        self.El = num_experts // world

    def moe_ffn(self, x, logits, gate_up, down, k, renorm, act, lb_weight, z_weight):
        from ..ops import moe as M
        T, H = x.shape
        E, lo = self.E, self.rank * self.El
        idx, w, probs, counts, lse, prob_sums, lse_sq = M.router_topk_stats(logits.detach(), k, renorm)
        multi = self.world > 1 and dist.is_initialized()
        p = torch.softmax(logits.float(), -1)                  # for the auxiliary losses: replicated, not summed
        # the expert path: x and the mixture weights feed every rank's partial output, so their gradients are summed
        lg_e = _GradSumOverRanks.apply(logits, self.group) if multi and logits.requires_grad else logits
        x = _GradSumOverRanks.apply(x, self.group) if multi and x.requires_grad else x
        wsel = torch.softmax(lg_e.float(), -1).gather(1, idx.long())
        if renorm:
            wsel = wsel / wsel.sum(-1, keepdim=True)
        holds_all = gate_up.shape[0] == E                      # un-cut model: use this rank's block of the full tensors
        y = torch.zeros((T, H), dtype=torch.float32, device=x.device)
        for j in range(self.El):
            e = lo + j
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            wg, wd = (gate_up[e], down[e]) if holds_all else (gate_up[j], down[j])
            gu = x[tok].float() @ wg.float().t()
            Fh = gu.shape[1] // 2
            g = gu[:, :Fh]
            a = {"gelu": torch.nn.functional.gelu(g, approximate="tanh"), "relu": torch.relu(g)}.get(str(act), torch.nn.functional.silu(g)) * gu[:, Fh:]
            y = y.index_add(0, tok, (a @ wd.float().t()) * wsel[tok, slot][:, None])
        if multi:
            y = _SumOverRanks.apply(y, self.group)
        f = counts.float() / float(T * k)
        aux = lb_weight * E * (f * p.mean(0)).sum() + z_weight * torch.logsumexp(logits.float(), -1).pow(2).mean()
        return y.to(x.dtype), aux, idx


class ModelExpertParallel:
    """Model-level expert parallelism with the reference's interface (``ExpertParallel`` of include/quant/moe_model.h:
    96-120; algorithm of src/model/moe_model.cpp:537-665): tokens are replicated, every rank runs the experts it holds,
    the partial mixtures meet in one all-reduce per layer, and ``sync_gradients`` averages what is replicated.  It runs
    on any ``torch.distributed`` backend, CPU included; the NVLink dispatch / combine path (``attach_expert_parallel`` +
    ``EPTrainer``) is the fast form of the same layer on GPUs and is tested against this one."""

    def __init__(self, num_experts: int, num_ranks: int = 1, rank: int = 0, ctx=None):
        if num_experts % max(1, num_ranks):
            raise ValueError("the number of experts must divide by the number of ranks")
        self._E, self._W, self._rank = num_experts, max(1, num_ranks), rank
        self.group = getattr(ctx, "group", None)

    def num_experts(self) -> int: return self._E
    def num_ranks(self) -> int: return self._W
    def rank(self) -> int: return self._rank
    def num_local_experts(self) -> int: return self._E // self._W

    def local_experts(self) -> List[int]:
        per = self._E // self._W
        return list(range(self._rank * per, (self._rank + 1) * per))

    def alltoall_experts(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Every rank's rows, concatenated in rank order (the reference's exchange is an all-gather: tokens are
        replicated, nothing is routed at this point)."""
        if self._W == 1 or not dist.is_initialized():
            res = x.clone()
        else:
            parts = [torch.empty_like(x) for _ in range(self._W)]
            dist.all_gather(parts, x.contiguous(), group=self.group)
            res = torch.cat(parts, 0)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def attach(self, model):
        for blk in model.layers:
            if hasattr(blk, "router"):
                blk.ep = _ReplicatedTokenFFN(self._rank, self._W, self._E, self.group)
        return model

    def detach(self, model):
        for blk in model.layers:
            if isinstance(getattr(blk, "ep", None), _ReplicatedTokenFFN):
                blk.ep = None
        return model

    def forward_with_parallel(self, model, ids: torch.Tensor) -> torch.Tensor:
        """Logits of ``model`` with every MoE layer computed across the ranks (all ranks pass the same ``ids``)."""
        self.attach(model)
        try:
            return model.forward(ids)
        finally:
            self.detach(model)

    def forward_backward(self, model, ids, labels):
        """Training form of ``forward_with_parallel``: loss and gradients (in ``main_grad``), expert layers across ranks."""
        self.attach(model)
        try:
            return model.forward_backward(ids, labels)
        finally:
            self.detach(model)

    def sync_gradients(self, model):
        """After ``forward_backward`` on replicated tokens: the replicated tensors already hold identical gradients on
        every rank and an expert's gradient lives on its owner only, so the owners' expert gradients are summed into every
        rank's copy (each rank then holds the full model's gradient).  With a model cut to its local experts there is
        nothing to exchange."""
        if self._W == 1 or not dist.is_initialized():
            return
        for blk in model.layers:
            if hasattr(blk, "router") and blk.gate_up.shape[0] == self._E:
                for p in (blk.gate_up, blk.down):
                    if getattr(p, "main_grad", None) is not None:
                        dist.all_reduce(p.main_grad, group=self.group)
