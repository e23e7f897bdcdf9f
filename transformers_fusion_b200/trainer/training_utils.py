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
        self.good, self._init = 0, init_scale

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

    # ---- the reference's names (include/quant/training_utils.h: MixedPrecisionScaler)
    def scale_loss(self, loss):
        return loss * self.scale

    def check_gradients(self, grads) -> bool:
        """True when any gradient holds inf / nan (``grads``: tensors, or parameters whose ``.grad`` / ``.main_grad`` is read)."""
        for g in grads:
            t = g if torch.is_tensor(g) and not isinstance(g, torch.nn.Parameter) else (getattr(g, "main_grad", None) if getattr(g, "main_grad", None) is not None else g.grad)
            if t is not None and self.has_overflow(t):
                return True
        return False

    update_scale = update

    def current_scale(self) -> float: return self.scale
    def good_steps(self) -> int: return self.good

    def reset(self, init_scale=None):
        self.scale, self.good = (init_scale if init_scale is not None else getattr(self, "_init", self.scale)), 0


class MixedPrecisionManager:
    """fp32 master copies of low-precision parameters: ``quantize_forward`` refreshes the compute copy from the master,
    ``restore_master`` puts the fp32 values back (for optimizers that step the parameter tensors themselves)."""

    def __init__(self, params=(), compute_dtype=torch.bfloat16, enabled: bool = True, init_loss_scale: float = 65536.0,
                 growth_interval: int = 2000):
        self.params = list(params)
        self.dtype, self.enabled = compute_dtype, enabled
        self.master = [p.detach().float().clone() for p in self.params]
        self.scaler = MixedPrecisionScaler(init_loss_scale if enabled else 1.0, growth_interval)

    # ---- the reference's names (include/quant/training_utils.h: MixedPrecisionManager)
    def is_enabled(self) -> bool: return self.enabled
    def current_loss_scale(self) -> float: return self.scaler.scale

    def to_fp16(self, t): return t.to(self.dtype)
    @staticmethod
    def to_fp32(t): return t.float()

    def create_master_weights(self, model_params):
        self.params = list(model_params)
        self.master = [p.detach().float().clone() for p in self.params]

    def sync_weights_to_model(self, model_params=None):
        """master -> model, rounded to the compute precision."""
        for p, m in zip(model_params or self.params, self.master):
            p.data.copy_(m.to(self.dtype).to(p.dtype))

    def sync_weights_from_model(self, model_params=None):
        for p, m in zip(model_params or self.params, self.master):
            m.copy_(p.detach().float())

    def scale_loss(self, loss):
        return loss * self.scaler.scale if self.enabled else loss

    def check_gradients(self, grads=None) -> bool:
        return self.scaler.check_gradients(grads if grads is not None else self.params)

    def unscale_gradients(self, params=None):
        inv = 1.0 / self.scaler.scale
        for p in params or self.params:
            g = getattr(p, "main_grad", None) if getattr(p, "main_grad", None) is not None else p.grad
            if g is not None:
                g.mul_(inv)

    def update_loss_scale(self, has_overflow: bool):
        return self.scaler.update(has_overflow) if self.enabled else 1.0

    def cast_gradients_to_fp32(self, params=None):
        """Low-precision ``.grad`` tensors become fp32 ``.main_grad`` tensors (this framework's place for fp32 gradients;
        ``.grad`` itself must keep the parameter's dtype)."""
        for p in params or self.params:
            if p.grad is not None and p.grad.dtype != torch.float32:
                p.main_grad = p.grad.float()
                p.grad = None

    def reset(self):
        self.scaler.reset()
        self.sync_weights_from_model()

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
    def __init__(self, params=(), decay=0.999):
        if isinstance(params, (int, float)):                  # the reference's order: EMAWeightAveraging(decay); init(params)
            params, decay = (), float(params)
        self.params, self.decay = list(params), decay
        self.shadow = [p.detach().float().clone() for p in self.params]
        self.backup = None

    def init(self, params):
        self.params = list(params)
        self.shadow = [p.detach().float().clone() for p in self.params]
        return self

    def update(self, params=None):
        for s, p in zip(self.shadow, params or self.params):
            s.mul_(self.decay).add_(p.detach().float(), alpha=1 - self.decay)

    def apply_to_model(self, model_params=None):
        """Averaged weights into the model, keeping a backup for ``restore``."""
        if model_params is not None:
            self.params = list(model_params)
        self.apply()

    def copy_to_model(self, model_params=None):
        """Averaged weights into the model for good (no backup)."""
        for s, p in zip(self.shadow, model_params or self.params):
            p.data.copy_(s.to(p.dtype))

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
    def __init__(self, total_steps, log_interval: int = 100):
        self.total, self.count, self.t0, self.log_interval = total_steps, 0, time.time(), log_interval

    def update(self, n=1):
        self.count += n

    def step(self):
        self.count += 1
        return self.log_interval > 0 and self.count % self.log_interval == 0       # True when a log line is due

    def reset(self):
        self.count, self.t0 = 0, time.time()

    def is_done(self) -> bool: return self.count >= self.total
    def current_step(self) -> int: return self.count
    def total_steps(self) -> int: return self.total
    def progress(self) -> float: return self.fraction()
    def elapsed_sec(self) -> float: return time.time() - self.t0
    def eta_sec(self) -> float: return self.eta_seconds()

    def fraction(self):
        return min(1.0, self.count / max(1, self.total))

    def eta_seconds(self):
        el = time.time() - self.t0
        return el / max(1, self.count) * max(0, self.total - self.count)

    def render(self, width=30):
        k = int(self.fraction() * width)
        return "[" + "#" * k + "." * (width - k) + f"] {self.count}/{self.total}"


class MetricTracker:
    """Named metric histories (``add / mean / best``) and, for one metric, the reference's exponential running average
    with best-so-far tracking (``update / value / improved``; include/quant/training_utils.h: MetricTracker)."""

    def __init__(self, window=100, alpha: float = 0.9, minimize: bool = True):
        if isinstance(window, float):                         # MetricTracker(alpha, minimize)
            window, alpha = 100, window
        self.window = window
        self.hist: Dict[str, List[float]] = {}
        self._alpha, self.minimize = alpha, minimize
        self.reset()

    def reset(self):
        self._avg, self._best, self._steps, self._improved = 0.0, None, 0, False

    def update(self, value: float):
        self._steps += 1
        self._avg = float(value) if self._steps == 1 else self._alpha * self._avg + (1 - self._alpha) * float(value)
        self._improved = self._best is None or (self._avg < self._best if self.minimize else self._avg > self._best)
        if self._improved:
            self._best = self._avg
        return self._avg

    def value(self) -> float: return self._avg
    def steps(self) -> int: return self._steps
    def improved(self) -> bool: return self._improved
    def alpha(self) -> float: return self._alpha

    def add(self, name, v):
        self.hist.setdefault(name, []).append(float(v))

    def mean(self, name, last=None):
        h = self.hist.get(name, [])[-(last or self.window):]
        return sum(h) / len(h) if h else 0.0

    def best(self, name=None, lower_is_better=True):
        if name is None:
            return self._best
        h = self.hist.get(name, [])
        return (min(h) if lower_is_better else max(h)) if h else None


class ModelSnapshot:
    """In-memory copy of a model's flat parameters (best-so-far restore)."""

    def __init__(self, path: str = "snapshot"):
        self.data, self.metric, self._path = None, None, path

    def path(self) -> str: return self._path

    def save(self, opt, step: int, current_lr: float, params):
        """Write parameters + optimizer state + step / rate to ``path`` (atomic: written aside, then renamed)."""
        import os
        st = {"step": int(step), "lr": float(current_lr), "params": [p.detach().cpu().clone() for p in params]}
        if opt is not None:
            st["opt"] = opt.state_dict() if hasattr(opt, "state_dict") else {k: v.detach().cpu().clone() for k, v in vars(opt).items() if torch.is_tensor(v)}
        tmp = self._path + ".tmp"
        torch.save(st, tmp)
        os.replace(tmp, self._path)

    def load(self, opt, params):
        """Restore what ``save`` wrote; returns (step, lr), or None when there is no usable snapshot."""
        import os
        if not os.path.exists(self._path):
            return None
        st = torch.load(self._path, map_location="cpu", weights_only=False)
        if len(st["params"]) != len(list(params)):
            return None
        for p, q in zip(params, st["params"]):
            p.data.copy_(q.to(p.dtype))
        if opt is not None and "opt" in st:
            if hasattr(opt, "load_state_dict"):
                opt.load_state_dict(st["opt"])
            else:
                for k, v in st["opt"].items():
                    getattr(opt, k).copy_(v)
        return st["step"], st["lr"]

    def capture(self, model, metric=None):
        self.data, self.metric = model.flat.params.detach().clone(), metric

    def restore(self, model):
        if self.data is not None:
            model.flat.params.copy_(self.data)


class EarlyStopping:
    def __init__(self, patience=5, min_delta=0.0, lower_is_better=True):
        self.patience, self.min_delta, self.lower = patience, min_delta, lower_is_better
        self.reset()

    def reset(self):
        self.best, self.bad, self._epoch, self._best_epoch, self._stopped = None, 0, 0, -1, False

    def step(self, value) -> bool:
        """True when training should stop."""
        better = self.best is None or (value < self.best - self.min_delta if self.lower else value > self.best + self.min_delta)
        if better:
            self.best, self.bad, self._best_epoch = value, 0, self._epoch
        else:
            self.bad += 1
        self._epoch += 1
        self._stopped = self.bad >= self.patience
        return self._stopped

    def stopped(self) -> bool: return self._stopped
    def best_epoch(self) -> int: return self._best_epoch
    def best_metric(self): return self.best


class LearningRateWarmup:
    LINEAR, EXPONENTIAL = "linear", "exponential"

    def __init__(self, base_lr, warmup_steps, mode="linear"):
        self.base, self.n, self.mode = base_lr, warmup_steps, mode

    def get_lr(self, step): return self.lr(step)
    def warmup_steps(self) -> int: return self.n
    def target_lr(self) -> float: return self.base

    def lr(self, step):
        if step >= self.n or self.n <= 0:
            return self.base
        f = (step + 1) / self.n
        return self.base * (f if self.mode == self.LINEAR else 1 - math.exp(-5 * f)) / (1.0 if self.mode == self.LINEAR else 1 - math.exp(-5))


class GradientAccumulator:
    def __init__(self, steps):
        self.steps, self.count = max(1, steps), 0

    def accumulate(self, params=None) -> bool:
        """Call once per micro-batch; True when the optimizer should step (gradients hold the sum of ``steps`` batches).
        With ``params`` their current ``.grad`` is added into the accumulator's own buffers (see ``apply_grads``)."""
        if params is not None:
            self.accumulate_grads(params)
            return self.ready()
        self.count += 1
        if self.count >= self.steps:
            self.count = 0
            return True
        return False

    def scale(self):
        return 1.0 / self.steps

    # ---- explicit buffers (reference: GradientAccumulator, include/quant/training_utils.h): for parameters whose
    # gradients are overwritten by each backward pass
    def accumulation_steps(self) -> int: return self.steps
    def current_step(self) -> int: return self.count
    def ready(self) -> bool: return self.count >= self.steps

    def accumulate_grads(self, params):
        """Add every parameter's current ``.grad`` into the accumulator's own buffers."""
        bufs = self.__dict__.setdefault("_bufs", {})
        for p in params:
            if p.grad is not None:
                bufs[id(p)] = bufs[id(p)] + p.grad.detach().float() if id(p) in bufs else p.grad.detach().float().clone()
        self.count += 1

    def apply_grads(self, params, opt=None):
        """Write the mean of the accumulated gradients into ``.grad``, step ``opt`` when given, and start over."""
        bufs = self.__dict__.setdefault("_bufs", {})
        for p in params:
            if id(p) in bufs:
                p.grad = (bufs[id(p)] / max(1, self.count)).to(p.dtype)
        if opt is not None:
            opt.step()
        self.reset()

    def reset(self):
        self.count, self._bufs = 0, {}


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
