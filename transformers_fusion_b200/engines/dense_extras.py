"""Dense training engine facades for fine-tuning, quantisation-aware training, mixed precision and continual learning: small
objects that hold statistics and drive the trainer's own machinery (``Trainer.enable_qat``, ``Trainer.enable_continual``,
``trainer.finetune.FineTuner``).

Reference counterparts: engines/trainer/dense/finetune.h:10-66 (FinetuneRunner, LoRAEngine), qat.h:10-58 (QATEngine,
MixedPrecision), continual.h:10-55 (ContinualRunner, EWCProbe)."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..quant.qat import STEQuantizer
from ..trainer import training_utils as TU
from ..trainer.continual import ContinualEngineConfig, ECCState
from ..trainer.finetune import FineTuner


# ----------------------------------------------------------------------------------------------- fine-tuning
@dataclass
class FinetuneStats:
    steps: int = 0
    tokens: int = 0
    tok_per_sec: float = 0.0
    last_loss: float = 0.0
    trainable_blocks: int = 0


class FinetuneRunner:
    """Runs a ``FineTuner`` and keeps throughput statistics."""

    def __init__(self, tuner: FineTuner, trainer=None):
        self.tuner, self.trainer = tuner, trainer
        self._stats = FinetuneStats()
        self._t0 = time.perf_counter()

    def configure(self, **cfg):
        self.tuner.configure(**cfg)
        return self

    def stats(self) -> FinetuneStats: return self._stats

    def train_step(self, ids: torch.Tensor, labels: torch.Tensor) -> float:
        loss = float(self.tuner.train_step(ids, labels))
        s = self._stats
        s.steps, s.tokens, s.last_loss = s.steps + 1, s.tokens + ids.numel(), loss
        s.tok_per_sec = s.tokens / max(time.perf_counter() - self._t0, 1e-9)
        return loss

    def fine_tune(self, dl, max_batches: Optional[int] = None) -> FinetuneStats:
        n = 0
        while (max_batches is None or n < max_batches) and (not hasattr(dl, "has_next") or dl.has_next()):
            self.train_step(*dl.next_batch())
            n += 1
        return self._stats

    def trainable_blocks(self, grads: torch.Tensor, threshold: float = 1e-6, block: int = 256) -> List[int]:
        out = FineTuner.find_trainable_blocks(grads, threshold, block)
        self._stats.trainable_blocks = len(out)
        return out

    def quant_update(self, fp32_grad: torch.Tensor, quant_weight: torch.Tensor, fmt=None, lr: Optional[float] = None):
        return self.tuner.apply_quant_update(fp32_grad, quant_weight, fmt, lr)


@dataclass
class LoRAConfig:
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    targets: List[str] = field(default_factory=list)


@dataclass
class LoRALayer:
    A: torch.Tensor            # [rank, in], Xavier
    B: torch.Tensor            # [out, rank], zero: the adapter starts as the identity
    scale: float = 1.0


class LoRAEngine:
    """Named low-rank adapters kept apart from the weights they adapt: ``forward`` is the adapter's own contribution
    (x A^T B^T scale), ``merge_into`` folds it into a weight matrix [out, in].  The model-level engine that trains adapters
    through the fused training path is ``trainer.finetune.RankAdapterEngine``."""

    def __init__(self, cfg: Optional[LoRAConfig] = None, seed: int = 0):
        self.cfg = cfg or LoRAConfig()
        self.layers: Dict[str, LoRALayer] = {}
        self._gen = torch.Generator().manual_seed(seed)

    def config(self) -> LoRAConfig: return self.cfg

    def attach(self, name: str, in_dim: int, out_dim: int) -> LoRALayer:
        r = self.cfg.rank
        bound = math.sqrt(6.0 / (in_dim + r))
        A = ((torch.rand(r, in_dim, generator=self._gen) * 2 - 1) * bound).requires_grad_()
        B = torch.zeros(out_dim, r, requires_grad=True)
        self.layers[name] = LoRALayer(A, B, self.cfg.alpha / r)
        return self.layers[name]

    def _get(self, name: str) -> LoRALayer:
        if name not in self.layers:
            raise KeyError(f"no adapter named {name!r}")
        return self.layers[name]

    def forward(self, name: str, x: torch.Tensor, training: bool = False) -> torch.Tensor:
        l = self._get(name)
        if training and self.cfg.dropout > 0:
            x = torch.nn.functional.dropout(x, self.cfg.dropout)
        return (x.float() @ l.A.t() @ l.B.t() * l.scale).to(x.dtype)

    @torch.no_grad()
    def merge_into(self, weight: torch.Tensor, name: str, merge_scale: float = 1.0):
        l = self._get(name)
        weight.add_((l.B @ l.A * (l.scale * merge_scale)).to(weight.dtype))
        return weight

    @torch.no_grad()
    def zero(self, name: str):
        self._get(name).B.zero_()

    def parameters(self) -> List[torch.Tensor]:
        return [t for l in self.layers.values() for t in (l.A, l.B)]

    def trainable_params(self) -> int:
        return sum(t.numel() for t in self.parameters())


# ----------------------------------------------------------------------------------------------- QAT / mixed precision
@dataclass
class QATStats:
    steps: int = 0
    mean_scale: float = 0.0
    mean_sqnr_db: float = 0.0


class QATEngine:
    """Quantisation-aware training on a schedule: attached to a trainer it switches the trainer's fake quantisation on for
    steps in [start, end) (``sync(step)``, called once per step); stand-alone it fake-quantises tensors and reports the
    signal-to-quantisation-noise ratio."""

    def __init__(self, bits: int = 8, symmetric: bool = True, use_lsq: bool = False, init_scale: float = 0.1):
        self.bits, self.symmetric, self.use_lsq, self.init_scale = bits, symmetric, use_lsq, init_scale
        self.trainer = None
        self._stats = QATStats()
        self._start, self._end = 0, 1 << 30
        self._ste = STEQuantizer("Q_8" if bits >= 8 else "Q_4" if bits >= 4 else "Q_2")
        self._scales: List[float] = []

    def stats(self) -> QATStats: return self._stats
    def inner(self) -> STEQuantizer: return self._ste

    def attach(self, trainer):
        self.trainer = trainer
        return self

    def set_bits(self, bits: int):
        self.bits = int(bits)
        if self.trainer is not None and self.trainer.qat_enabled():
            self.trainer.enable_qat(self.bits, self.symmetric, self.use_lsq, self.init_scale)

    def set_schedule(self, start_step: int, end_step: int):
        self._start, self._end = int(start_step), int(end_step)

    def active_at(self, step: int) -> bool:
        return self._start <= step < self._end

    def sync(self, step: Optional[int] = None) -> bool:
        """Bring the attached trainer's fake quantisation in line with the schedule; returns whether it is on."""
        t = self.trainer
        step = t.global_step if step is None else step
        on = self.active_at(step)
        if on and not t.qat_enabled():
            t.enable_qat(self.bits, self.symmetric, self.use_lsq, self.init_scale)
        elif not on and t.qat_enabled():
            t.disable_qat()
        self._stats.steps += int(on)
        return on

    def _qrange(self):
        return (-(1 << (self.bits - 1)) + 1, (1 << (self.bits - 1)) - 1) if self.symmetric else (0, (1 << self.bits) - 1)

    def fake_quantize(self, weight: torch.Tensor) -> torch.Tensor:
        """Per-tensor absmax grid of the configured width (straight-through gradient)."""
        from ..quant.qat import ste_fake_quantize
        qmin, qmax = self._qrange()
        amax = float(weight.detach().abs().max())
        scale = amax / qmax if amax > 0 else self.init_scale
        self._scales.append(scale)
        return ste_fake_quantize(weight, scale, qmin, qmax)

    def sqnr_db(self, fp32: torch.Tensor, fq: torch.Tensor) -> float:
        sig = float(fp32.float().pow(2).sum())
        noise = float((fp32.float() - fq.float()).pow(2).sum())
        return 10.0 * math.log10(sig / noise) if noise > 0 and sig > 0 else float("inf")

    def calibrate(self, params: Sequence[torch.Tensor], batches: int = 8) -> QATStats:
        """Scale and SQNR statistics of the given tensors at the current width."""
        self._scales = []
        db = []
        for p in params:
            q = self.fake_quantize(p.detach())
            v = self.sqnr_db(p.detach(), q)
            if math.isfinite(v):
                db.append(v)
        self._stats.mean_scale = sum(self._scales) / max(1, len(self._scales))
        self._stats.mean_sqnr_db = sum(db) / max(1, len(db))
        return self._stats

    def step_scales(self, lr: float = 1e-4) -> float:
        """Mean learned step size of the attached trainer's matrices (they are trained by the trainer's own step when
        ``use_lsq`` is on); without a trainer, the mean scale of the last ``calibrate``."""
        t = self.trainer
        steps = getattr(t, "_qat_steps", None) if t is not None else None
        if steps:
            vals = [float(s) for s in (steps.values() if isinstance(steps, dict) else steps)]
            self._stats.mean_scale = sum(vals) / len(vals)
        return self._stats.mean_scale


@dataclass
class MPStats:
    loss_scale: float = 128.0
    overflows: int = 0
    steps: int = 0


class MixedPrecision:
    """Dynamic loss scaling over a list of parameters' gradients (``p.grad`` or ``p.main_grad``): unscale, skip the step on
    overflow and halve the scale, double it after ``interval`` clean steps."""

    def __init__(self, init_scale: float = 128.0, interval: int = 2000):
        self._sc = TU.MixedPrecisionScaler(init_scale, interval)
        self._stats = MPStats(loss_scale=init_scale)

    def scale(self) -> float: return float(self._sc.scale)
    def stats(self) -> MPStats: return self._stats

    @staticmethod
    def _grads(params):
        for p in params:
            g = getattr(p, "main_grad", None)
            g = p.grad if g is None else g
            if g is not None:
                yield g

    @torch.no_grad()
    def unscale(self, params):
        inv = 1.0 / self.scale()
        for g in self._grads(params):
            g.mul_(inv)

    def check_overflow(self, params) -> bool:
        return any(not bool(torch.isfinite(g).all()) for g in self._grads(params))

    def step(self, params) -> bool:
        """Call after backward: returns True when the optimizer step may go ahead (gradients are unscaled then)."""
        bad = self.check_overflow(params)
        if not bad:
            self.unscale(params)
        self._sc.update(bad)
        s = self._stats
        s.steps, s.overflows, s.loss_scale = s.steps + 1, s.overflows + int(bad), self.scale()
        return not bad


# ----------------------------------------------------------------------------------------------- continual learning
@dataclass
class ContinualStats:
    task_id: int = 0
    steps: int = 0
    ewc_penalty: float = 0.0
    replay_loss: float = 0.0
    forgetting: float = 0.0
    stability: float = 0.0


class EWCProbe:
    """The consolidation state's three operations on plain tensors."""

    @staticmethod
    def penalty(ecc: ECCState, weights: torch.Tensor, lam: float) -> float:
        return float(ecc.regularize(weights, lam))

    @staticmethod
    def accumulate_fisher(ecc: ECCState, grads: torch.Tensor, alpha: float):
        if not ecc.initialized:
            ecc.initialize(grads.numel(), grads.device)
        ecc.update_fisher(grads, alpha)

    @staticmethod
    def anchor(ecc: ECCState, weights: torch.Tensor):
        if not ecc.initialized:
            ecc.initialize(weights.numel(), weights.device)
        ecc.update_anchor(weights)


class ContinualRunner:
    """Continual learning through the trainer: the consolidation penalty and replay run inside ``Trainer.train_step``; this
    object names the task boundaries, sets the two knobs and reports the statistics."""

    def __init__(self, trainer, cfg: Optional[ContinualEngineConfig] = None):
        self.trainer = trainer
        trainer.enable_continual(cfg)
        self._stats = ContinualStats()

    def engine(self): return self.trainer.continual_engine()
    def stats(self) -> ContinualStats: return self._stats
    def set_ewc_lambda(self, lam: float): self.trainer.set_ewc_lambda(lam)
    def set_replay_ratio(self, r: float): self.trainer.set_replay_ratio(r)

    def on_task_boundary(self, new_task_id: int, eval_dl=None, max_batches: int = 4):
        self.trainer.on_task_boundary(new_task_id, eval_dl, max_batches)
        self._stats.task_id = int(new_task_id)

    def ewc_penalty(self, lam: Optional[float] = None) -> float:
        e = self.engine()
        if not e.ecc.initialized:
            return 0.0
        w = self.trainer.model.flat.params.float()
        self._stats.ewc_penalty = float(e.ecc.regularize(w, e.cfg.ecc_lambda if lam is None else lam))
        return self._stats.ewc_penalty

    def replay_mix(self, ids: torch.Tensor, labels: torch.Tensor, ratio: Optional[float] = None):
        if ratio is not None:
            self.trainer.set_replay_ratio(ratio)
        return self.trainer._mix_replay(ids, labels)

    def train_step_mixed(self, ids: torch.Tensor, labels: torch.Tensor, replay_ratio: Optional[float] = None) -> float:
        if replay_ratio is not None:
            self.trainer.set_replay_ratio(replay_ratio)
        loss = float(self.trainer.train_step(ids, labels))
        self._stats.steps += 1
        self._stats.replay_loss = loss
        self.ewc_penalty()
        return loss

    def eval_forgetting(self) -> float:
        m = self.engine().benchmark.compute()
        self._stats.forgetting, self._stats.stability = m.avg_forgetting, m.stability_score
        return m.avg_forgetting
