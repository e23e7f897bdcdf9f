"""MoE training engine facade and the host-side routing planners.  The planners take plain tensors and return plain
Python structures; they are the CPU oracles of the device router, the permute / combine kernels and the expert-parallel
dispatch.

Reference counterparts: engines/trainer/moe/moe.h:17-118 (MoETrainerEngine, route_topk, plan_capacity, build_ep_map,
balance_stats, MoEPipeline), engines/trainer/moe/dispatch.h:11-56 (plan_dispatch, gather_expert_inputs,
combine_expert_outputs, drop_stats)."""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..trainer.moe_trainer import MoETrainConfig, MoETrainer
from ..trainer.trainer import DataLoader


@dataclass
class MoEStats:
    steps: int = 0
    tokens: int = 0
    tok_per_sec: float = 0.0
    last_loss: float = 0.0
    expert_util: float = 0.0
    aux_loss: float = 0.0


class MoETrainerEngine:
    def __init__(self, model, tokenizer=None, ep=None):
        self.model, self.tok, self.ep = model, tokenizer, ep
        self.trainer = MoETrainer(model, tokenizer)
        self.cfg = MoETrainConfig()
        self._stats = MoEStats()
        self._t0 = time.perf_counter()

    def compile(self, optimizer=None, cfg: Optional[MoETrainConfig] = None):
        self.cfg = cfg or self.cfg
        self.trainer.compile(optimizer, self.cfg)
        self._t0 = time.perf_counter()
        return self

    def train_step(self, ids, labels) -> float:
        loss = self.trainer.train_step(ids, labels)
        s, m = self._stats, self.trainer.metrics()
        s.steps += 1
        s.tokens += ids.numel()
        s.last_loss, s.aux_loss = float(loss), m.aux_loss
        s.expert_util = self.expert_utilization()
        s.tok_per_sec = s.tokens / max(1e-9, time.perf_counter() - self._t0)
        return loss

    def micro_step(self, ids, labels, loss_scale: float = 1.0) -> float:
        return self.trainer.micro_step(ids, labels, loss_scale)

    def fit(self, dl, cfg: Optional[MoETrainConfig] = None, val_dl=None):
        return self.trainer.fit(dl, cfg, val_dl)

    def eval_loss(self, val_dl, max_batches: int = 20) -> float:
        return self.trainer.eval_loss(val_dl, max_batches)

    def save_checkpoint(self, path): self.trainer.save_checkpoint(path)
    def load_checkpoint(self, path): self.trainer.load_checkpoint(path)

    def expert_utilization(self) -> float:
        """Fraction of experts that received at least half of their fair share of tokens in the last step."""
        u = self.trainer.compute_expert_utilization()
        return float((u >= 0.5 / max(1, u.numel())).float().mean()) if u.numel() else 0.0

    def metrics(self): return self.trainer.metrics()
    def stats(self) -> MoEStats: return self._stats


# ----------------------------------------------------------------------------------------------- routing planners
@dataclass
class RouterOut:
    weights: torch.Tensor          # [T, k] renormalised to sum 1 per token
    indices: torch.Tensor          # [T, k]
    aux_loss: float = 0.0


def route_topk(router_logits: torch.Tensor, top_k: int, load_balance_coef: float = 0.01) -> RouterOut:
    """Softmax over all experts, top-k, weights renormalised over the chosen k; aux = coef * E * sum_e f_e * P_e with f_e
    the fraction of assignments routed to e and P_e its mean probability."""
    T, E = router_logits.shape
    if not 0 < top_k <= E:
        raise ValueError("bad top_k")
    p = torch.softmax(router_logits.float(), -1)
    w, idx = p.topk(top_k, -1)
    w = w / w.sum(-1, keepdim=True)
    f = torch.bincount(idx.reshape(-1), minlength=E).float() / max(1, T * top_k)
    return RouterOut(w, idx, float(load_balance_coef * E * (f * p.mean(0)).sum()))


@dataclass
class CapacityPlan:
    experts: int = 8
    top_k: int = 2
    capacity_factor: float = 2.0
    tokens: int = 0
    slots_per_expert: int = 0
    dropped: int = 0


def plan_capacity(tokens: int, experts: int, top_k: int, capacity_factor: float) -> CapacityPlan:
    """slots = ceil(tokens * top_k / experts * factor); ``dropped`` is the lower bound on drops (assignments beyond all slots)."""
    if experts <= 0:
        raise ValueError("bad experts")
    slots = math.ceil(tokens * top_k / experts * capacity_factor)
    return CapacityPlan(experts, top_k, capacity_factor, tokens, slots, max(0, tokens * top_k - slots * experts))


def z_loss(router_logits: torch.Tensor) -> float:
    if router_logits.dim() != 2:
        raise ValueError("z_loss needs a 2-D tensor")
    return float((torch.logsumexp(router_logits.float(), -1) ** 2).mean())


@dataclass
class EPMap:
    ranks: int = 1
    expert_rank: List[int] = field(default_factory=list)
    rank_counts: List[int] = field(default_factory=list)


def build_ep_map(experts: int, ranks: int, contiguous: bool = True) -> EPMap:
    """Expert -> rank.  ``contiguous`` (the layout of the fused dispatch kernels: rank r owns a block of E / W experts);
    otherwise round-robin."""
    if ranks <= 0:
        raise ValueError("bad ranks")
    per = -(-experts // ranks)
    er = [min(ranks - 1, e // per) if contiguous else e % ranks for e in range(experts)]
    return EPMap(ranks, er, [er.count(r) for r in range(ranks)])


@dataclass
class BalanceOut:
    cv: float = 0.0
    min_share: float = 0.0
    max_share: float = 0.0


def balance_stats(importance: Sequence[float], rows: int) -> BalanceOut:
    if not len(importance) or rows <= 0:
        return BalanceOut()
    v = torch.as_tensor(importance, dtype=torch.float64)
    mean = float(v.mean())
    return BalanceOut(float(v.std(unbiased=False) / (mean if mean > 0 else 1.0)), float(v.min()) / rows, float(v.max()) / rows)


@dataclass
class DispatchItem:
    token: int
    expert: int
    weight: float


@dataclass
class DispatchPlan:
    per_expert: List[List[DispatchItem]]
    dropped: List[DispatchItem]
    slots_per_expert: int = 0


def plan_dispatch(indices: torch.Tensor, weights: torch.Tensor, num_experts: int, slots_per_expert: int) -> DispatchPlan:
    """Tokens in order, choices in order; an assignment to a full expert is dropped (slots_per_expert <= 0: unlimited)."""
    plan = DispatchPlan([[] for _ in range(num_experts)], [], slots_per_expert)
    idx, w = indices.tolist(), weights.tolist()
    for t, (ei, wi) in enumerate(zip(idx, w)):
        for e, x in zip(ei, wi):
            it = DispatchItem(t, e, float(x))
            if slots_per_expert > 0 and len(plan.per_expert[e]) >= slots_per_expert:
                plan.dropped.append(it)
            else:
                plan.per_expert[e].append(it)
    return plan


@dataclass
class ExpertInputs:
    bufs: List[torch.Tensor]
    counts: List[int]


def gather_expert_inputs(hidden: torch.Tensor, plan: DispatchPlan, num_experts: int) -> ExpertInputs:
    bufs = [hidden[[it.token for it in plan.per_expert[e]]] if plan.per_expert[e] else hidden.new_zeros((0, hidden.shape[-1]))
            for e in range(num_experts)]
    return ExpertInputs(bufs, [b.shape[0] for b in bufs])


@dataclass
class CombineOut:
    hidden: torch.Tensor
    dropped: int = 0


def combine_expert_outputs(expert_outs: Sequence[torch.Tensor], plan: DispatchPlan, tokens: int, dim: int) -> CombineOut:
    out = torch.zeros((tokens, dim), dtype=torch.float32)
    for e, items in enumerate(plan.per_expert):
        if items:
            tok = torch.tensor([it.token for it in items])
            wt = torch.tensor([it.weight for it in items])
            out.index_add_(0, tok, expert_outs[e].float().cpu() * wt[:, None])
    return CombineOut(out, len(plan.dropped))


@dataclass
class DropStats:
    assigned: int = 0
    kept: int = 0
    dropped: int = 0
    drop_rate: float = 0.0
    per_expert_kept: List[int] = field(default_factory=list)


def drop_stats(plan: DispatchPlan, num_experts: int) -> DropStats:
    kept = [len(plan.per_expert[e]) for e in range(num_experts)]
    k, d = sum(kept), len(plan.dropped)
    return DropStats(k + d, k, d, d / (k + d) if k + d else 0.0, kept)


# ----------------------------------------------------------------------------------------------- epoch pipeline
class MoEPipeline:
    """File-to-checkpoints loop: tokenise the training (and validation) text, run epochs, keep the best validation
    checkpoint, stop after ``patience`` epochs without improvement, append one JSON line per epoch to the log file."""

    def __init__(self, engine: MoETrainerEngine, tokenizer, train_path: str, val_path: str = ""):
        self.engine, self.tok, self.train_path, self.val_path = engine, tokenizer, train_path, val_path
        self.cfg = engine.cfg
        self.ckpt_dir, self.log_path = "", ""
        self._best_val, self._no_improve, self.patience = 1e30, 0, 3

    def configure(self, cfg: MoETrainConfig):
        self.cfg = cfg
        self.engine.compile(None, cfg)

    def set_checkpoint_dir(self, d: str):
        os.makedirs(d, exist_ok=True)
        self.ckpt_dir = d

    def set_log_file(self, path: str): self.log_path = path
    def best_val(self) -> float: return self._best_val

    def _loader(self, path):
        dev = self.engine.model.tok_embeddings.device
        return DataLoader(self.tok, path, self.cfg.batch_size, self.cfg.seq_length, device=dev)

    def run_epoch(self, epoch: int) -> float:
        dl = self._loader(self.train_path)
        n = min(len(dl), self.cfg.max_steps)
        tot = sum(self.engine.train_step(*dl.next_batch()) for _ in range(n)) / max(1, n)
        val = self.engine.eval_loss(self._loader(self.val_path)) if self.val_path else tot
        if val < self._best_val - 1e-6:
            self._best_val, self._no_improve = val, 0
            if self.ckpt_dir:
                self.engine.save_checkpoint(os.path.join(self.ckpt_dir, "best.quant"))
        else:
            self._no_improve += 1
        if self.ckpt_dir:
            self.engine.save_checkpoint(os.path.join(self.ckpt_dir, f"epoch{epoch}.quant"))
        if self.log_path:
            with open(self.log_path, "a") as f:
                s = self.engine.stats()
                f.write(json.dumps({"epoch": epoch, "train_loss": tot, "val_loss": val, "aux_loss": s.aux_loss,
                                    "expert_util": s.expert_util, "tok_per_sec": s.tok_per_sec}) + "\n")
        return tot

    def run(self, epochs: int = -1) -> float:
        epochs = self.cfg.epochs if epochs < 0 else epochs
        last = 0.0
        for e in range(epochs):
            last = self.run_epoch(e)
            if self._no_improve >= self.patience:
                break
        return last
