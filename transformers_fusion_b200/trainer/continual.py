"""Continual learning: elastic weight consolidation state (Fisher diagonal + anchor), a compressed replay buffer (8-bit
codebook-quantised samples with importance-weighted sampling), forgetting metrics, a learning-rate governor that trades
stability for plasticity, an experience replay ring, a weight-distribution watchdog with rollback, orthogonal projection of
updates and an entropy floor.

Reference counterparts: include/quant/continual_engine.h:29-320, src/trainer/continual_engine.cpp."""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class CompressedReplayEntry:
    q_input: torch.Tensor
    q_target: torch.Tensor
    in_lo: float
    in_scale: float
    tg_lo: float
    tg_scale: float
    fisher_importance: float = 1.0
    task_id: int = 0
    step_inserted: int = 0
    access_count: int = 0


class CompressedReplayBuffer:
    def __init__(self, capacity=65536, spill_threshold=0.8, seed=42):
        self.capacity, self.spill = capacity, spill_threshold
        self.entries: List[CompressedReplayEntry] = []
        self.rng = random.Random(seed)
        self.step = 0
        self.raw_bytes = 0

    @staticmethod
    def _q(x):
        x = x.detach().float().reshape(-1).cpu()
        lo, hi = float(x.min()), float(x.max())
        sc = (hi - lo) / 255.0 or 1.0
        return torch.clamp(torch.round((x - lo) / sc), 0, 255).to(torch.uint8), lo, sc

    def insert(self, inp, tgt, task_id=0, fisher_importance=1.0):
        qi, il, isc = self._q(inp)
        qt, tl, tsc = self._q(tgt)
        self.entries.append(CompressedReplayEntry(qi, qt, il, isc, tl, tsc, fisher_importance, task_id, self.step))
        self.raw_bytes += (qi.numel() + qt.numel()) * 4
        self.step += 1
        if len(self.entries) > self.capacity:
            self.compact()

    def at(self, idx: int) -> "CompressedReplayEntry":
        """The stored entry at a position (IndexError outside the buffer)."""
        if not 0 <= idx < len(self.entries):
            raise IndexError(f"replay entry {idx} of {len(self.entries)}")
        return self.entries[idx]

    def compact(self):
        """Drop the least important entries down to ``spill_threshold`` of the capacity."""
        keep = int(self.capacity * self.spill)
        self.entries.sort(key=lambda e: -e.fisher_importance)
        del self.entries[keep:]

    def sample_batch(self, batch_size):
        """(inputs, targets, weights): sampled proportionally to importance; weights are the inverse probabilities,
        normalised to mean 1."""
        if not self.entries:
            return None
        w = [max(e.fisher_importance, 1e-8) for e in self.entries]
        tot = sum(w)
        idx = self.rng.choices(range(len(self.entries)), weights=w, k=batch_size)
        ins, tgs, ws = [], [], []
        for i in idx:
            e = self.entries[i]
            e.access_count += 1
            ins.append(e.q_input.float() * e.in_scale + e.in_lo)
            tgs.append(e.q_target.float() * e.tg_scale + e.tg_lo)
            ws.append(tot / (len(self.entries) * w[i]))
        m = sum(ws) / len(ws)
        return ins, tgs, [x / m for x in ws]

    def importance_resample(self):
        self.entries = [self.entries[i] for i in self.rng.choices(range(len(self.entries)),
                                                                weights=[e.fisher_importance for e in self.entries], k=len(self.entries))]

    def set_fisher(self, idx, v):
        self.entries[idx].fisher_importance = v

    def update_importance(self, decay):
        for e in self.entries:
            e.fisher_importance *= decay

    def clear(self):
        self.entries, self.raw_bytes = [], 0

    def size(self):
        return len(self.entries)

    def memory_bytes(self):
        return sum(e.q_input.numel() + e.q_target.numel() + 32 for e in self.entries)

    def compression_ratio(self):
        kept = sum((e.q_input.numel() + e.q_target.numel()) * 4 for e in self.entries)
        return kept / max(1, self.memory_bytes())


class ECCState:
    """Fisher diagonal (EMA of squared gradients) and anchor weights; ``regularize`` is lambda/2 * sum F (w - w*)^2."""

    def __init__(self):
        self.fisher = None
        self.anchor = None
        self.initialized = False

    def initialize(self, n, device="cpu"):
        self.fisher = torch.zeros(n, device=device)
        self.anchor = torch.zeros(n, device=device)
        self.initialized = True

    def update_fisher(self, grads, alpha):
        self.fisher.mul_(1 - alpha).add_(grads.float() ** 2, alpha=alpha)

    def update_anchor(self, weights):
        self.anchor.copy_(weights.float())

    def regularize(self, weights, lam) -> float:
        return float(0.5 * lam * (self.fisher * (weights.float() - self.anchor) ** 2).sum())

    def penalty_grad(self, weights, lam):
        return lam * self.fisher * (weights.float() - self.anchor)


@dataclass
class ForgettingMetrics:
    avg_forgetting: float = 0.0
    max_forgetting: float = 0.0
    backward_transfer: float = 0.0
    forward_transfer: float = 0.0
    stability_score: float = 0.0
    num_tasks: int = 0


class ForgettingBenchmark:
    def __init__(self):
        self.baseline: Dict[int, float] = {}
        self.current: Dict[int, float] = {}
        self.first_seen: Dict[int, float] = {}

    def register(self, task_id, baseline_loss, untrained_loss=None):
        self.baseline[task_id] = baseline_loss
        if untrained_loss is not None:
            self.first_seen[task_id] = untrained_loss

    def update(self, task_id, loss):
        self.current[task_id] = loss

    # ---- the reference's spelling (include/quant/continual_engine.h:124-144): tasks are numbered in registration order and
    # keep their held-out evaluation set, so a caller can re-measure them after every later task
    def register_task(self, eval_inputs, eval_targets, elem_count: Optional[int] = None) -> int:
        if not hasattr(self, "tasks"):
            self.tasks = []
        n = elem_count if elem_count is not None else len(eval_inputs)
        self.tasks.append((eval_inputs[:n], eval_targets[:n]))
        return len(self.tasks) - 1

    def eval_set(self, task_id: int):
        return self.tasks[task_id]

    def record_baseline(self, task_id: int, loss: float):
        """Loss on the task right after training on it; the first value ever recorded for a task (normally before training) is
        kept as the untrained loss that forward transfer is measured from."""
        self.first_seen.setdefault(task_id, float(loss))
        self.baseline[task_id] = float(loss)

    def record_current(self, task_id: int, loss: float):
        self.first_seen.setdefault(task_id, float(loss))
        self.current[task_id] = float(loss)

    def forgetting(self, task_id: int) -> float:
        if task_id not in self.baseline or task_id not in self.current:
            return 0.0
        return max(0.0, self.current[task_id] - self.baseline[task_id])

    def backward_transfer(self) -> float: return self.compute().backward_transfer
    def forward_transfer(self) -> float: return self.compute().forward_transfer

    def num_tasks(self) -> int:
        return max(len(getattr(self, "tasks", ())), len(self.baseline))

    def compute(self) -> ForgettingMetrics:
        ts = [t for t in self.baseline if t in self.current]
        if not ts:
            return ForgettingMetrics()
        f = [max(0.0, self.current[t] - self.baseline[t]) for t in ts]
        bwt = sum(self.baseline[t] - self.current[t] for t in ts) / len(ts)
        fwt = sum(self.first_seen[t] - self.baseline[t] for t in ts if t in self.first_seen) / max(1, sum(t in self.first_seen for t in ts))
        avg = sum(f) / len(f)
        return ForgettingMetrics(avg, max(f), bwt, fwt, 1.0 / (1.0 + avg), len(ts))


@dataclass
class ContinualEngineConfig:
    replay_capacity: int = 65536
    ecc_lambda: float = 1.0
    ecc_alpha: float = 0.01
    forgetting_temperature: float = 100.0
    importance_decay: float = 0.99
    forgetting_check_interval: int = 100
    stability_lr_factor: float = 0.5
    plasticity_lr_factor: float = 2.0
    forgetting_threshold: float = 0.1


class ContinualEngine:
    def __init__(self, cfg: Optional[ContinualEngineConfig] = None):
        self.cfg = cfg or ContinualEngineConfig()
        self.replay = CompressedReplayBuffer(self.cfg.replay_capacity)
        self.ecc = ECCState()
        self.benchmark = ForgettingBenchmark()
        self.current_task, self.current_step = 0, 0

    def on_step(self, grads, weights, base_lr, task_id):
        if not self.ecc.initialized:
            self.ecc.initialize(weights.numel(), weights.device)
            self.ecc.update_anchor(weights)
        self.ecc.update_fisher(grads, self.cfg.ecc_alpha)
        self.current_task = task_id
        self.current_step += 1
        if self.current_step % 10 == 0:
            self.replay.update_importance(self.cfg.importance_decay)
        return self.effective_lr(base_lr)

    def on_task_boundary(self, new_task_id, weights, baseline_loss=None, untrained_loss=None):
        """The finished task's weights become the anchor; its evaluation loss the forgetting baseline."""
        self.ecc.update_anchor(weights)
        if baseline_loss is not None:
            self.benchmark.register(self.current_task, baseline_loss, untrained_loss)
        self.current_task = new_task_id

    def register_eval(self, task_id, loss):
        self.benchmark.update(task_id, loss)

    def effective_lr(self, base_lr):
        m = self.benchmark.compute()
        if m.num_tasks and m.avg_forgetting > self.cfg.forgetting_threshold:
            return base_lr * self.cfg.stability_lr_factor
        if m.num_tasks and m.avg_forgetting < 0.1 * self.cfg.forgetting_threshold:
            return base_lr * self.cfg.plasticity_lr_factor
        return base_lr

    def should_check_forgetting(self):
        return self.current_step > 0 and self.current_step % self.cfg.forgetting_check_interval == 0

    def regularized_grads(self, grads, weights):
        return grads + self.ecc.penalty_grad(weights, self.cfg.ecc_lambda).to(grads.dtype)

    def forgetting_metrics(self):
        return self.benchmark.compute()


def apply_orthogonal_projection(update: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Remove from ``update`` its component along ``weights`` (keeps the weight norm to first order); in place."""
    w = weights.float().reshape(-1)
    u = update.reshape(-1)
    u.sub_((u.float() @ w) / (w @ w).clamp(min=1e-30) * w.to(u.dtype))
    return update


class ExperienceReplayBuffer:
    def __init__(self, max_size, replay_interval):
        self.max, self.interval = max_size, replay_interval
        self.buf: List = []
        self.head = 0

    def add(self, inp, tgt, generation=0):
        item = (inp, tgt, generation)
        if len(self.buf) < self.max:
            self.buf.append(item)
        else:
            self.buf[self.head] = item
        self.head = (self.head + 1) % self.max

    def sample_batch(self, batch_size, rng=random):
        if not self.buf:
            return None
        items = [rng.choice(self.buf) for _ in range(batch_size)]
        return [i[0] for i in items], [i[1] for i in items]

    def should_replay(self, current_batch):
        return self.interval > 0 and current_batch > 0 and current_batch % self.interval == 0

    def size(self):
        return len(self.buf)


@dataclass
class LayerStatus:
    mean: float
    variance: float
    kurtosis: float
    is_healthy: bool = True


class DistributionWatchdog:
    """Tracks mean / variance / kurtosis of each layer's weights; a layer whose variance leaves ``threshold`` x its
    baseline (either way) or whose values stop being finite is unhealthy and can be rolled back to the last good copy."""

    def __init__(self, threshold=2.0):
        self.threshold = threshold
        self.good: Dict[int, torch.Tensor] = {}
        self.base: Dict[int, LayerStatus] = {}
        self.cur: Dict[int, LayerStatus] = {}

    @staticmethod
    def _stats(w):
        f = w.detach().float().reshape(-1)
        m, v = float(f.mean()), float(f.var(unbiased=False))
        k = float(((f - m) ** 4).mean() / max(v * v, 1e-30))
        return LayerStatus(m, v, k)

    def track_layer(self, layer_id, w):
        st = self._stats(w)
        if layer_id not in self.base:
            self.base[layer_id] = st
            self.good[layer_id] = w.detach().clone()
        b = self.base[layer_id]
        finite = bool(torch.isfinite(w).all())
        ratio = st.variance / max(b.variance, 1e-30)
        st.is_healthy = finite and (1.0 / self.threshold) <= ratio <= self.threshold
        self.cur[layer_id] = st
        if st.is_healthy:
            self.good[layer_id] = w.detach().clone()

    def check_health(self):
        return dict(self.cur)

    def rollback(self, layer_id, w):
        w.data.copy_(self.good[layer_id])


def apply_entropy_floor(output_entropy, weights, importance, floor=0.5, noise_scale=0.01, generator=None):
    """When the output distribution has collapsed (entropy below the floor), perturb the least important weights."""
    if output_entropy >= floor:
        return False
    imp = importance.float().reshape(-1)
    mask = imp <= imp.median()
    noise = torch.randn(weights.numel(), generator=generator).to(weights.device) * noise_scale * float(weights.float().std())
    weights.reshape(-1).add_((noise * mask).to(weights.dtype))
    return True
