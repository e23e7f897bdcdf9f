"""Small training-loop utilities with the reference's names: loss scaling and mixed-precision master weights, EMA weight
averaging, progress / metric trackers, snapshots, early stopping, learning-rate warm-up, gradient accumulation, and the
extra loss functions (cross entropy with ignore_index / label smoothing, focal, R-Drop, InfoNCE, MSE, z-loss).

Reference counterparts: include/quant/training_utils.h:10-230, engines/trainer/dense losses."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn.functional as TF


@dataclass
class MoEAuxLosses:
    load_balance: float = 0.0
    z_loss: float = 0.0
    aux: float = 0.0

    def total(self, lb_w=0.01, z_w=0.001, aux_w=0.01):
        return lb_w * self.load_balance + z_w * self.z_loss + aux_w * self.aux


class MixedPrecisionScaler:
    """Dynamic loss scale: halve on overflow, double after ``interval`` clean steps."""

    def __init__(self, init_scale=128.0, interval=2000, min_scale=1.0, max_scale=65536.0):
        self.scale, self.interval, self.min, self.max = init_scale, interval, min_scale, max_scale
        self.good = 0

    def update(self, overflow: bool):
        if overflow:
            self.scale, self.good = max(self.min, self.scale / 2), 0
        else:
            self.good += 1
            if self.good >= self.interval:
                self.scale, self.good = min(self.max, self.scale * 2), 0
        return self.scale

    @staticmethod
    def has_overflow(grads: torch.Tensor) -> bool:
        return not bool(torch.isfinite(grads).all())


class MixedPrecisionManager:
    """fp32 master copies of low-precision parameters: ``quantize_forward`` refreshes the compute copy from the master,
    ``restore_master`` puts the fp32 values back (for optimizers that step the parameter tensors themselves)."""

    def __init__(self, params, compute_dtype=torch.bfloat16):
        self.params = list(params)
        self.dtype = compute_dtype
        self.master = [p.detach().float().clone() for p in self.params]

    def quantize_forward(self):
        for p, m in zip(self.params, self.master):
            p.data.copy_(m.to(self.dtype).to(p.dtype))

    def restore_master(self):
        for p, m in zip(self.params, self.master):
            p.data.copy_(m.to(p.dtype))

    def step_master(self, lr, grads):
        for m, g in zip(self.master, grads):
            m.add_(g.float(), alpha=-lr)


class EMAWeightAveraging:
    def __init__(self, params, decay=0.999):
        self.params, self.decay = list(params), decay
        self.shadow = [p.detach().float().clone() for p in self.params]
        self.backup = None

    def update(self):
        for s, p in zip(self.shadow, self.params):
            s.mul_(self.decay).add_(p.detach().float(), alpha=1 - self.decay)

    def apply(self):
        self.backup = [p.detach().clone() for p in self.params]
        for s, p in zip(self.shadow, self.params):
            p.data.copy_(s.to(p.dtype))

    def restore(self):
        if self.backup is not None:
            for b, p in zip(self.backup, self.params):
                p.data.copy_(b)
            self.backup = None


class ProgressTracker:
    def __init__(self, total_steps):
        self.total, self.step, self.t0 = total_steps, 0, time.time()

    def update(self, n=1):
        self.step += n

    def fraction(self):
        return min(1.0, self.step / max(1, self.total))

    def eta_seconds(self):
        el = time.time() - self.t0
        return el / max(1, self.step) * max(0, self.total - self.step)

    def render(self, width=30):
        k = int(self.fraction() * width)
        return "[" + "#" * k + "." * (width - k) + f"] {self.step}/{self.total}"


class MetricTracker:
    def __init__(self, window=100):
        self.window = window
        self.hist: Dict[str, List[float]] = {}

    def add(self, name, v):
        self.hist.setdefault(name, []).append(float(v))

    def mean(self, name, last=None):
        h = self.hist.get(name, [])[-(last or self.window):]
        return sum(h) / len(h) if h else 0.0

    def best(self, name, lower_is_better=True):
        h = self.hist.get(name, [])
        return (min(h) if lower_is_better else max(h)) if h else None


class ModelSnapshot:
    """In-memory copy of a model's flat parameters (best-so-far restore)."""

    def __init__(self):
        self.data, self.metric = None, None

    def capture(self, model, metric=None):
        self.data, self.metric = model.flat.params.detach().clone(), metric

    def restore(self, model):
        if self.data is not None:
            model.flat.params.copy_(self.data)


class EarlyStopping:
    def __init__(self, patience=5, min_delta=0.0, lower_is_better=True):
        self.patience, self.min_delta, self.lower = patience, min_delta, lower_is_better
        self.best, self.bad = None, 0

    def step(self, value) -> bool:
        """True when training should stop."""
        better = self.best is None or (value < self.best - self.min_delta if self.lower else value > self.best + self.min_delta)
        if better:
            self.best, self.bad = value, 0
        else:
            self.bad += 1
        return self.bad >= self.patience


class LearningRateWarmup:
    LINEAR, EXPONENTIAL = "linear", "exponential"

    def __init__(self, base_lr, warmup_steps, mode="linear"):
        self.base, self.n, self.mode = base_lr, warmup_steps, mode

    def lr(self, step):
        if step >= self.n or self.n <= 0:
            return self.base
        f = (step + 1) / self.n
        return self.base * (f if self.mode == self.LINEAR else 1 - math.exp(-5 * f)) / (1.0 if self.mode == self.LINEAR else 1 - math.exp(-5))


class GradientAccumulator:
    def __init__(self, steps):
        self.steps, self.count = max(1, steps), 0

    def accumulate(self) -> bool:
        """Call once per micro-batch; True when the optimizer should step (gradients hold the sum of ``steps`` batches)."""
        self.count += 1
        if self.count >= self.steps:
            self.count = 0
            return True
        return False

    def scale(self):
        return 1.0 / self.steps


# ---- losses -------------------------------------------------------------------------------------------------------------
def cross_entropy_loss(logits, labels, ignore_index=-100, label_smoothing=0.0):
    return TF.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.reshape(-1), ignore_index=ignore_index,
                            label_smoothing=label_smoothing)


def focal_loss(logits, labels, gamma=2.0, ignore_index=-100):
    lp = torch.log_softmax(logits.float().view(-1, logits.shape[-1]), -1)
    lab = labels.reshape(-1)
    keep = lab != ignore_index
    lpt = lp[keep].gather(1, lab[keep][:, None])[:, 0]
    return (-(1 - lpt.exp()) ** gamma * lpt).mean() if keep.any() else lp.sum() * 0


def rdrop_loss(logits1, logits2, labels, alpha=1.0, ignore_index=-100):
    """Mean CE of two stochastic passes + alpha * symmetric KL between them."""
    ce = 0.5 * (cross_entropy_loss(logits1, labels, ignore_index) + cross_entropy_loss(logits2, labels, ignore_index))
    p, q = torch.log_softmax(logits1.float(), -1), torch.log_softmax(logits2.float(), -1)
    kl = 0.5 * ((p.exp() * (p - q)).sum(-1) + (q.exp() * (q - p)).sum(-1)).mean()
    return ce + alpha * kl


def infonce_loss(a, b, temperature=0.07):
    """Symmetric InfoNCE over matching rows of two embedding batches."""
    a, b = TF.normalize(a.float(), dim=-1), TF.normalize(b.float(), dim=-1)
    logits = a @ b.t() / temperature
    tgt = torch.arange(a.shape[0], device=a.device)
    return 0.5 * (TF.cross_entropy(logits, tgt) + TF.cross_entropy(logits.t(), tgt))


def mse_loss(a, b):
    return ((a.float() - b.float()) ** 2).mean()


def z_loss(logits, weight=1e-4):
    return weight * (torch.logsumexp(logits.float(), -1) ** 2).mean()


def mtp_loss(hidden, heads, labels, weights=None):
    """Multi-token prediction: head k predicts the token k + 2 positions ahead of each position from hidden [B, S, H]."""
    total, n = 0.0, 0
    for k, w in enumerate(heads):
        shift = k + 1
        if hidden.shape[1] <= shift:
            break
        lg = hidden[:, :-shift].float() @ w.float().t()
        total = total + (weights[k] if weights else 1.0) * cross_entropy_loss(lg, labels[:, shift:])
        n += 1
    return total / max(1, n)
