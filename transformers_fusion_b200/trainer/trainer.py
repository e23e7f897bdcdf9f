"""Trainer / UnifiedTrainer / DataLoader: the public training API.

Field-for-field counterpart of the reference's ``TrainConfig`` (include/quant/trainer.h:24-69) and the
``Trainer`` surface (``compile``, ``fit``, ``micro_step``, ``train_step``, ``clip_gradients``,
``eval_loss``, ``save_checkpoint`` / ``load_checkpoint``, log / epoch / step callbacks, ``metrics``,
EMA, dynamic loss scale, gradient noise, label smoothing: include/quant/trainer.h:240-342,
src/trainer/trainer_core.cpp:201-1069).  Checkpoints are the reference's pair: ``<path>`` (.quant
container, Q_32 blocks) and ``<path>.opt`` ({step, lr, n, per parameter m and v}); ``--resume`` state
(step, loader offset, RNG) goes to ``<path>.state.json``.
"""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, List, Optional

import torch

from ..quant import codec
from .fused_optim import FlatAdamW
from .optimizers import FlatOptimizer, build_optimizer
from .schedulers import schedule_lr


@dataclass
class TrainConfig:
    batch_size: int = 8
    seq_length: int = 512
    epochs: int = 3
    max_steps: int = 10000
    learning_rate: float = 3e-4
    weight_decay: float = 1e-2
    warmup_steps: int = 100
    log_interval: int = 10
    save_interval: int = 1000
    val_interval: int = 500
    max_grad_norm: float = 1.0
    grad_accum_steps: int = 1
    lr_schedule: str = "WARMUP_COSINE"
    loss_scale: float = 128.0
    loss_scale_interval: int = 2000
    dynamic_loss_scale: bool = False
    label_smoothing: float = 0.0
    rdrop_alpha: float = 0.0
    grad_noise_eta: float = 0.0
    grad_noise_gamma: float = 0.55
    ema_decay: float = 0.0
    qat_bits: int = 0
    qat_symmetric: bool = True
    moe_lb_weight: float = 0.01
    moe_z_weight: float = 0.001
    mtp_loss_weight: float = 0.0
    optimizer: str = "adamw"
    seed: int = 42
    checkpoint_path: str = "model.quant"
    activation_checkpointing: bool = False
    zero_stage: int = 2
    cuda_graph: bool = False


@dataclass
class TrainMetrics:
    loss: float = 0.0
    perplexity: float = 0.0
    val_loss: float = 0.0
    learning_rate: float = 0.0
    grad_norm: float = 0.0
    tokens_per_sec: float = 0.0
    step: int = 0
    epoch: int = 0


@dataclass
class DataLoaderConfig:
    """The reference's loader description (include/quant/dataloader.h:16-27)."""
    data_path: str = ""
    batch_size: int = 8
    seq_length: int = 2048
    shuffle_buffer: int = 10000
    num_epochs: int = 1
    num_workers: int = 1
    seed: int = 42
    drop_last: bool = True
    world_size: int = 1
    rank: int = 0


class DataLoader:
    """Token stream -> (ids, labels) batches of [batch, seq]; labels are ids shifted left by one.
    Source: a text file tokenised with ``tokenizer`` (reference DataLoader, include/quant/trainer.h:78-159),
    a 1-D tensor of token ids, or ``synthetic=(vocab, seed)``."""

    def __init__(self, tokenizer=None, path: Optional[str] = None, batch_size=8, seq_length=512, tokens=None,
                 synthetic=None, device="cpu", rank=0, world=1, pin=False):
        self.B, self.S, self.device, self.rank, self.world = batch_size, seq_length, device, rank, world
        self.offset = 0
        self.synthetic = synthetic
        self.pin = pin
        if synthetic is not None:
            self.tokens = None
            self._gen = torch.Generator().manual_seed(synthetic[1] * 9973 + rank)
        elif tokens is not None:
            self.tokens = tokens.long()
        else:
            text = open(path, "r", encoding="utf-8", errors="ignore").read()
            self.tokens = torch.tensor(tokenizer.encode(text), dtype=torch.long)

    def __len__(self):
        if self.tokens is None:
            return 1 << 30
        return max(0, (self.tokens.numel() - 1) // (self.B * self.S * self.world))

    def reset(self):
        self.offset = 0

    @classmethod
    def from_config(cls, cfg: DataLoaderConfig, tokenizer=None, device="cpu") -> "DataLoader":
        """A loader described by a ``DataLoaderConfig``: the text file at ``data_path`` tokenised with ``tokenizer`` (bytes
        when none is given), this rank's share of every global batch, shuffled per epoch when ``shuffle_buffer`` > 0."""
        if tokenizer is None:
            from ..tokenizer import ByteTokenizer
            tokenizer = ByteTokenizer()
        dl = cls(tokenizer, cfg.data_path, cfg.batch_size, cfg.seq_length, device=device, rank=cfg.rank, world=cfg.world_size)
        dl._config = cfg
        if cfg.shuffle_buffer > 0:
            dl._order = torch.randperm(max(len(dl), 1), generator=torch.Generator().manual_seed(cfg.seed)).tolist()
        return dl

    def config(self) -> DataLoaderConfig:
        """The loader's description; for a loader built directly it is filled in from the constructor's arguments."""
        if getattr(self, "_config", None) is None:
            self._config = DataLoaderConfig(batch_size=self.B, seq_length=self.S, shuffle_buffer=0, world_size=self.world, rank=self.rank)
        return self._config

    def next_batch_with_labels(self):
        return self.next_batch()

    # ---- the reference's verbs (include/quant/trainer.h:78-159)
    def num_batches(self) -> int: return len(self)
    def batch_size(self) -> int: return self.B
    def seq_length(self) -> int: return self.S
    def has_next(self) -> bool: return self.offset < len(self)

    def shuffle(self, epoch: int = 0):
        """Visit the batches of this epoch in a permuted order (the same order for the same epoch on every rank)."""
        n = len(self)
        if self.tokens is not None and n > 0:
            self._order = torch.randperm(n, generator=torch.Generator().manual_seed(1000003 * (epoch + 1))).tolist()
        self.offset = 0

    def set_augmentation(self, mask_prob: float = 0.0, replace_prob: float = 0.0, mask_id: int = 0, vocab_size: int = 0, seed: int = 0):
        """Token-level augmentation of the inputs: each position is masked with ``mask_prob`` (its label is kept, so the
        model must recover it) or replaced by a random id with ``replace_prob``."""
        self._aug = dict(mask_prob=mask_prob, replace_prob=replace_prob, mask_id=mask_id, vocab_size=vocab_size)
        self._aug_gen = torch.Generator().manual_seed(seed)

    def apply_augmentation(self, ids, labels):
        a = getattr(self, "_aug", None)
        if not a or (a["mask_prob"] <= 0 and a["replace_prob"] <= 0):
            return ids, labels
        r = torch.rand(ids.shape, generator=self._aug_gen).to(ids.device)
        out = ids.clone()
        out[r < a["mask_prob"]] = a["mask_id"]
        rep = (r >= a["mask_prob"]) & (r < a["mask_prob"] + a["replace_prob"])
        if a["vocab_size"] > 0 and bool(rep.any()):
            out[rep] = torch.randint(0, a["vocab_size"], (int(rep.sum()),), generator=self._aug_gen).to(ids.device)
        return out, labels

    def set_curriculum(self, total_epochs: int, min_seq_length: int = 64):
        """Sequence-length curriculum: batches start at ``min_seq_length`` tokens and grow linearly to the full length
        over ``total_epochs`` (the batch keeps its shape; positions past the current length get label -100)."""
        self._cur = dict(total=max(1, total_epochs), epoch=0, min_len=min_seq_length)

    def curriculum_step(self, epoch: int):
        if getattr(self, "_cur", None):
            self._cur["epoch"] = epoch

    def effective_seq_length(self) -> int:
        c = getattr(self, "_cur", None)
        if not c:
            return self.S
        t = min(1.0, c["epoch"] / c["total"])
        return int(min(self.S, max(c["min_len"], round(c["min_len"] + t * (self.S - c["min_len"])))))

    def next_batch(self):
        ids, labels = self._next_batch()
        if getattr(self, "_cur", None) and self.effective_seq_length() < self.S:
            labels = labels.clone()
            labels[:, self.effective_seq_length():] = -100
        if getattr(self, "_aug", None):
            ids, labels = self.apply_augmentation(ids, labels)
        return ids, labels

    next_batch_with_labels = next_batch

    def _next_batch(self):
        B, S = self.B, self.S
        if self.tokens is None:
            ids = torch.randint(0, self.synthetic[0], (B, S + 1), generator=self._gen)
        else:
            n = B * S
            order = getattr(self, "_order", None)
            slot = order[self.offset % len(order)] if order and self.offset < len(order) else self.offset
            start = (slot * self.world + self.rank) * n
            if start + n + 1 > self.tokens.numel():
                self.offset = 0
                start = self.rank * n
                if start + n + 1 > self.tokens.numel():
                    raise ValueError("dataset is smaller than one batch")
            chunk = self.tokens[start:start + n + 1]
            self.offset += 1
            return self._ship(chunk[:-1].view(B, S).contiguous()), self._ship(chunk[1:].view(B, S).contiguous())
        self.offset += 1
        return self._ship(ids[:, :-1].contiguous()), self._ship(ids[:, 1:].contiguous())

    def _ship(self, t):
        if self.pin and torch.cuda.is_available():
            t = t.pin_memory()
        return t.to(self.device, non_blocking=True)

    def __iter__(self):
        for _ in range(len(self)):
            yield self.next_batch()


class ModelEMA:
    def __init__(self, flat, decay):
        self.flat, self.decay = flat, decay
        self.shadow = flat.params.float().clone()

    def step(self):
        self.shadow.mul_(self.decay).add_(self.flat.params.float(), alpha=1 - self.decay)

    update = step

    def set_decay(self, d: float):
        self.decay = float(d)

    def swap(self):
        cur = self.flat.params.float().clone()
        self.flat.params.copy_(self.shadow.to(self.flat.params.dtype))
        self.shadow = cur

    def apply(self):
        """Overwrite the parameters with their average (the average is kept)."""
        self.flat.params.copy_(self.shadow.to(self.flat.params.dtype))


class Trainer:
    def __init__(self, model, tokenizer=None):
        self.model, self.tok = model, tokenizer
        self.cfg = TrainConfig()
        self.opt = None
        self.engine = None
        self._metrics = TrainMetrics()
        self.log_cb: Optional[Callable[[TrainMetrics], None]] = None
        self.epoch_cb = self.step_cb = None
        self.ema: Optional[ModelEMA] = None
        self.loss_scale = 1.0
        self._good_steps = 0
        self.global_step = 0
        self._qat = None                 # (bits, symmetric, use_lsq) when quantisation-aware training is on
        self._qat_steps = {}             # LSQ: learned step size per parameter (by position in the flat list)
        self.continual = None            # trainer.continual.ContinualEngine when continual learning is on
        self.current_task = 0
        self.replay_ratio = 0.25
        self._replay = []                # exact (ids row, labels row, task) samples of earlier steps
        self._ewc_anchored = False

    # ------------------------------------------------------------------ configuration
    def compile(self, optimizer=None, cfg: Optional[TrainConfig] = None, symm=None):
        """``optimizer``: None / a name ("adamw", "adafactor", ...) / a FlatOptimizer instance."""
        from .engine import TrainEngine
        self.cfg = cfg or self.cfg
        c = self.cfg
        self.model.activation_checkpointing = c.activation_checkpointing
        name = optimizer if isinstance(optimizer, str) else (c.optimizer if optimizer is None else None)
        fused = name == "adamw"
        self.engine = TrainEngine(self.model, lr=c.learning_rate, weight_decay=c.weight_decay, betas=(0.9, 0.999),
                                  max_grad_norm=c.max_grad_norm, zero_stage=c.zero_stage, cuda_graph=c.cuda_graph and fused,
                                  comm="fused" if symm is not None else "nccl", symm=symm,
                                  grad_accum_steps=c.grad_accum_steps)
        if fused:
            self.opt = self.engine.opt
        else:
            self.opt = optimizer if isinstance(optimizer, FlatOptimizer) else build_optimizer(
                name, self.model.flat, lr=c.learning_rate, weight_decay=c.weight_decay, max_grad_norm=c.max_grad_norm,
                shard=self.engine.shard if self.engine.zero_stage else None)
            self.engine.opt = self.opt if hasattr(self.opt, "stage_hyper") else self.engine.opt
        if c.ema_decay > 0:
            self.ema = ModelEMA(self.model.flat, c.ema_decay)
        self.loss_scale = c.loss_scale if c.dynamic_loss_scale else 1.0
        if c.qat_bits > 0:
            self.enable_qat(c.qat_bits, c.qat_symmetric)
        if c.mtp_loss_weight > 0:
            self.model.mtp_loss_weight = c.mtp_loss_weight
        return self

    def init_mixed_precision(self) -> float:
        """(Re)start mixed-precision training: the optimizer's fp32 master weights are re-read from the model's
        compute-dtype weights, and for an fp16 model dynamic loss scaling is switched on at the configured scale (bf16 and
        fp32 have fp32's exponent range and train unscaled).  Returns the loss scale in effect."""
        c = self.cfg
        if self.opt is not None and hasattr(self.opt, "master"):
            lo, hi = getattr(self.opt, "lo", 0), getattr(self.opt, "hi", self.model.flat.numel)
            self.opt.master.copy_(self.model.flat.params[lo:hi].float())
        if self.model.flat.params.dtype == torch.float16:
            c.dynamic_loss_scale = True
        self.loss_scale = c.loss_scale if c.dynamic_loss_scale else 1.0
        self._good_steps = 0
        return self.loss_scale

    def set_log_callback(self, cb): self.log_cb = cb
    def set_epoch_callback(self, cb): self.epoch_cb = cb
    def set_step_callback(self, cb): self.step_cb = cb
    def metrics(self) -> TrainMetrics: return self._metrics

    def lr_at(self, step):
        c = self.cfg
        return schedule_lr(c.lr_schedule, c.learning_rate, step, c.max_steps, c.warmup_steps)

    # ------------------------------------------------------------------ steps
    def micro_step(self, ids, labels, loss_scale: float = 1.0):
        """Forward + backward of one micro-batch (gradients accumulate in main_grad).  Returns the loss tensor."""
        return self.model.forward_backward(ids, labels, loss_scale=loss_scale / max(1, self.cfg.grad_accum_steps),
                                           label_smoothing=self.cfg.label_smoothing)

    def clip_gradients(self, max_norm: float) -> float:
        g = self.model.flat.grads
        n = float(g.norm())
        if max_norm > 0 and n > max_norm:
            g.mul_(max_norm / (n + 1e-6))
        return n

    def inject_gradient_noise(self, step, eta, gamma):
        std = math.sqrt(eta / (1 + step) ** gamma)
        self.model.flat.grads.add_(torch.randn_like(self.model.flat.grads) * std)

    def train_step(self, ids, labels) -> float:
        """One optimizer step (with gradient accumulation over ``grad_accum_steps`` equal slices)."""
        c = self.cfg
        lr = self.lr_at(self.global_step)
        fused = isinstance(self.opt, FlatAdamW)
        plain = self._qat is None and self.continual is None
        if fused and plain and c.grad_accum_steps == 1 and not c.dynamic_loss_scale and c.grad_noise_eta == 0:
            self.model.loss_label_smoothing = c.label_smoothing
            loss = self.engine.step(ids, labels, lr)
        else:
            if self.continual is not None:
                ids, labels = self._mix_replay(ids, labels)
            shadow = self._qat_quantize_weights() if self._qat is not None else None
            chunks = zip(ids.chunk(c.grad_accum_steps), labels.chunk(c.grad_accum_steps))
            loss = sum(self.micro_step(i, l, self.loss_scale) for i, l in chunks) / c.grad_accum_steps
            if shadow is not None:
                self._qat_restore_weights(shadow)          # straight-through: the update is applied to the unquantised weights
            if self.continual is not None:
                lr = self._continual_after_backward(lr)
            if c.grad_noise_eta > 0:
                self.inject_gradient_noise(self.global_step, c.grad_noise_eta, c.grad_noise_gamma)
            if self.loss_scale != 1.0:
                self.model.flat.grads.mul_(1.0 / self.loss_scale)
            overflow = c.dynamic_loss_scale and not bool(torch.isfinite(self.model.flat.grads).all())
            if overflow:
                self.loss_scale = max(1.0, self.loss_scale / 2)
                self._good_steps = 0
                self.model.flat.grads.zero_()
            else:
                self.opt.step(lr)
                if c.dynamic_loss_scale:
                    self._good_steps += 1
                    if self._good_steps >= c.loss_scale_interval:
                        self.loss_scale = min(65536.0, self.loss_scale * 2)
                        self._good_steps = 0
        if self.ema:
            self.ema.step()
        self.global_step += 1
        lv = float(loss)
        m = self._metrics
        m.loss, m.perplexity, m.learning_rate, m.step = lv, math.exp(min(lv, 30.0)), lr, self.global_step
        m.grad_norm = float(self.opt.grad_norm.reshape(-1)[0]) if hasattr(self.opt, "grad_norm") else 0.0
        return lv

    @torch.no_grad()
    def eval_loss(self, val_dl, max_batches=20) -> float:
        tot, n = 0.0, 0
        for _ in range(min(max_batches, max(1, len(val_dl)))):
            ids, labels = val_dl.next_batch()
            logits = self.model(ids).float()
            tot += float(torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1)))
            n += 1
        self._metrics.val_loss = tot / max(1, n)
        return self._metrics.val_loss

    def fit(self, dl, cfg: Optional[TrainConfig] = None, val_dl=None):
        if cfg is not None or self.engine is None:
            self.compile(None, cfg or self.cfg)
        c = self.cfg
        dev = self.model.tok_embeddings.device
        for epoch in range(c.epochs):
            dl.reset()
            t0, toks = time.perf_counter(), 0
            for _ in range(len(dl)):
                if self.global_step >= c.max_steps:
                    break
                ids, labels = dl.next_batch()
                self.train_step(ids.to(dev), labels.to(dev))
                toks += ids.numel()
                m = self._metrics
                m.epoch = epoch
                if self.global_step % c.log_interval == 0:
                    m.tokens_per_sec = toks / max(1e-9, time.perf_counter() - t0)
                    if self.log_cb:
                        self.log_cb(m)
                if self.step_cb:
                    self.step_cb(m)
                if val_dl is not None and c.val_interval and self.global_step % c.val_interval == 0:
                    self.eval_loss(val_dl)
                if c.save_interval and self.global_step % c.save_interval == 0:
                    self.save_checkpoint(c.checkpoint_path, dl)
            if self.epoch_cb:
                self.epoch_cb(self._metrics)
            if self.global_step >= c.max_steps:
                break
        self.save_checkpoint(c.checkpoint_path, dl)
        return self._metrics

    # ------------------------------------------------------------------ loss helpers (reference: trainer.h:265-267)
    @torch.no_grad()
    def rdrop_loss(self, ids, labels, alpha: float) -> float:
        """Cross entropy of one forward pass + alpha x mean KL(p1 || p2) between two forward passes of the same batch.
        The two passes differ only through stochastic layers (gating dropout of the MoE variants); for a deterministic
        model the second term is zero.  Reference: Trainer::rdrop_loss, src/trainer/trainer_core.cpp:960-992."""
        was = self.model.training
        self.model.train()
        l1 = self.model(ids).float()
        l2 = self.model(ids).float()
        self.model.train(was)
        V = l1.shape[-1]
        lp1, lp2 = torch.log_softmax(l1.reshape(-1, V), -1), torch.log_softmax(l2.reshape(-1, V), -1)
        kl = (lp1.exp() * (lp1 - lp2)).sum(-1).mean()
        ce = torch.nn.functional.cross_entropy(l1.reshape(-1, V), labels.reshape(-1), ignore_index=-100)
        return float(ce + alpha * kl)

    @staticmethod
    def label_smoothing_loss(logits, labels, smoothing: float):
        """Per-token loss [B, S] against (1 - smoothing) one-hot + smoothing / V uniform targets; tokens whose label is
        outside the vocabulary get 0.  Reference: src/trainer/trainer_core.cpp:994-1028."""
        V = logits.shape[-1]
        lp = torch.log_softmax(logits.float().reshape(-1, V), -1)
        lab = labels.reshape(-1).long()
        ok = (lab >= 0) & (lab < V)
        picked = lp.gather(1, lab.clamp(0, V - 1)[:, None])[:, 0]
        loss = -(1.0 - smoothing) * picked - (smoothing / V) * lp.sum(-1)
        return torch.where(ok, loss, torch.zeros_like(loss)).view(labels.shape)

    @staticmethod
    def mtp_loss(mtp_logits, labels, ignore_index: int = -100) -> float:
        """Mean over the extra heads of the cross entropy of head k against the labels moved k + 1 further left."""
        if not mtp_logits:
            return 0.0
        tot = 0.0
        for k, lg in enumerate(mtp_logits):
            sh = torch.full_like(labels, ignore_index)
            if labels.shape[1] > k + 1:
                sh[:, :-(k + 1)] = labels[:, k + 1:]
            tot += float(torch.nn.functional.cross_entropy(lg.float().reshape(-1, lg.shape[-1]), sh.reshape(-1),
                                                           ignore_index=ignore_index))
        return tot / len(mtp_logits)

    def dynamic_loss_scale(self, grad_norm: float, max_grad_norm: float):
        """The reference's scale rule as a call (src/trainer/trainer_core.cpp:1071-1084): a norm above the threshold
        halves the scale, ``loss_scale_interval`` quiet steps double it; a scale of 1 means scaling is off."""
        if self.loss_scale == 1.0:
            return self.loss_scale
        if not math.isfinite(grad_norm) or grad_norm > max_grad_norm:
            self.loss_scale, self._good_steps = max(1.0, self.loss_scale / 2), 0
        else:
            self._good_steps += 1
            if self._good_steps >= self.cfg.loss_scale_interval:
                self.loss_scale, self._good_steps = min(65536.0, self.loss_scale * 2), 0
        return self.loss_scale

    def unscale_gradients(self, scale: float):
        if scale != 1.0:
            self.model.flat.grads.mul_(1.0 / scale)

    def get_model_params(self): return list(self.model.parameters())

    # ------------------------------------------------------------------ quantisation-aware training (trainer.h:281-288)
    def enable_qat(self, bits: int = 8, symmetric: bool = True, use_lsq: bool = False, init_scale: float = 0.1):
        """From the next step on every matrix is replaced by its fake-quantised value for forward and backward and the
        optimizer updates the unquantised weights (straight-through estimator).  ``use_lsq``: one learned step size per
        matrix (started from the weights' statistics, or ``init_scale`` for an all-zero matrix) instead of the per-tensor
        absmax grid; the step sizes learn from the same backward pass."""
        self._qat = (int(bits), bool(symmetric), bool(use_lsq), float(init_scale))
        self._qat_steps = {}

    def disable_qat(self):
        self._qat, self._qat_steps = None, {}

    def qat_enabled(self) -> bool: return self._qat is not None

    def qat_fake_quantize(self, weight):
        """Per-tensor absmax fake quantisation at the configured width (what the forward pass sees)."""
        bits, sym = (self._qat[0], self._qat[1]) if self._qat else (8, True)
        qmax = (1 << (bits - 1)) - 1 if sym else (1 << bits) - 1
        qmin = -qmax if sym else 0
        w = weight.float()
        if sym:
            sc = w.abs().max().clamp(min=1e-8) / qmax
            return (torch.round(w / sc).clamp(qmin, qmax) * sc).to(weight.dtype)
        lo, hi = w.min(), w.max()
        sc = ((hi - lo) / qmax).clamp(min=1e-8)
        return ((torch.round((w - lo) / sc).clamp(0, qmax)) * sc + lo).to(weight.dtype)

    def qat_fake_quantize_lsq(self, weight, scale_param):
        from ..quant.qat import lsq_fake_quantize
        bits, sym = (self._qat[0], self._qat[1]) if self._qat else (8, True)
        return lsq_fake_quantize(weight, scale_param, bits, sym)

    @torch.no_grad()
    def _qat_quantize_weights(self):
        """Replace the matrices by their quantised values; returns what is needed to undo it."""
        from ..quant.qat import lsq_init_step
        bits, sym, lsq, init = self._qat
        flat = self.model.flat
        shadow = flat.params.clone()
        for i, p in enumerate(flat.params_list):
            if p.dim() < 2 or p.numel() < 64:
                continue
            if lsq:
                st = self._qat_steps.get(i)
                if st is None:
                    st = lsq_init_step(p.data.float(), bits, sym)
                    st = torch.as_tensor(st, dtype=torch.float32, device=p.device).reshape(())
                    if float(st) <= 0:
                        st = torch.tensor(init, device=p.device)
                    self._qat_steps[i] = st
                qmax = (1 << (bits - 1)) - 1
                p.data.copy_((torch.round(p.data.float() / st).clamp(-qmax if sym else 0, qmax) * st).to(p.dtype))
            else:
                p.data.copy_(self.qat_fake_quantize(p.data))
        return shadow

    @torch.no_grad()
    def _qat_restore_weights(self, shadow):
        bits, sym, lsq, _ = self._qat
        flat = self.model.flat
        if lsq:
            # step-size gradient of LSQ: sum over weights of g * (round(w/s) - w/s inside the range, the bound outside),
            # scaled by 1 / sqrt(n * qmax); a plain SGD step at the trainer's learning rate keeps the step positive
            qmax = (1 << (bits - 1)) - 1
            off = 0
            for i, (p, o) in enumerate(zip(flat.params_list, flat.offsets)):
                st = self._qat_steps.get(i)
                if st is None:
                    continue
                w = shadow[o:o + p.numel()].view(p.shape).float()
                g = p.main_grad.float()
                v = w / st
                inside = (v > (-qmax if sym else 0)) & (v < qmax)
                ds = torch.where(inside, torch.round(v) - v, v.clamp(-qmax if sym else 0, qmax))
                gs = (g * ds).sum() / math.sqrt(p.numel() * qmax)
                self._qat_steps[i] = (st - self.lr_at(self.global_step) * gs).clamp(min=1e-8)
        flat.params.copy_(shadow)

    # ------------------------------------------------------------------ continual learning (trainer.h:290-302)
    def enable_continual(self, cfg=None):
        """Elastic weight consolidation (Fisher-weighted pull towards the weights at the last task boundary) + replay of
        earlier tasks' samples + a forgetting-aware learning rate, driven by ``trainer.continual.ContinualEngine``."""
        from .continual import ContinualEngine, ContinualEngineConfig
        self.continual = ContinualEngine(cfg or ContinualEngineConfig())
        self.current_task = 0
        self._replay = []
        self._ewc_anchored = False
        return self.continual

    def disable_continual(self):
        self.continual, self._replay = None, []

    def continual_enabled(self) -> bool: return self.continual is not None
    def continual_engine(self): return self.continual

    def set_ewc_lambda(self, lam: float):
        if self.continual is not None:
            self.continual.cfg.ecc_lambda = float(lam)

    def set_replay_ratio(self, r: float):
        self.replay_ratio = min(1.0, max(0.0, float(r)))

    def on_task_boundary(self, new_task_id: int, eval_dl=None, max_batches: int = 4):
        """The task that ends becomes the anchor of the consolidation penalty; its loss on ``eval_dl`` (when given) is the
        baseline later forgetting is measured against."""
        if self.continual is None:
            self.current_task = new_task_id
            return None
        base = self.eval_loss(eval_dl, max_batches) if eval_dl is not None else None
        w = self.model.flat.params.detach().float()
        if not self.continual.ecc.initialized:
            self.continual.ecc.initialize(w.numel(), w.device)
        self.continual.on_task_boundary(new_task_id, w, base)
        self._ewc_anchored = True
        self.current_task = new_task_id
        return base

    def _mix_replay(self, ids, labels):
        """Remember this batch's rows for later tasks and replace ``replay_ratio`` of the rows by rows of earlier tasks."""
        cap = max(1, self.continual.cfg.replay_capacity)
        old = [r for r in self._replay if r[2] != self.current_task]
        n = min(len(old), int(round(self.replay_ratio * ids.shape[0])))
        new_ids, new_lab = ids, labels
        if n > 0:
            g = torch.Generator().manual_seed(self.cfg.seed * 7919 + self.global_step)
            pick = torch.randperm(len(old), generator=g)[:n].tolist()
            new_ids, new_lab = ids.clone(), labels.clone()
            for row, j in enumerate(pick):
                if old[j][0].numel() == ids.shape[1]:
                    new_ids[row], new_lab[row] = old[j][0].to(ids.device), old[j][1].to(labels.device)
        for b in range(ids.shape[0]):
            self._replay.append((ids[b].detach().cpu(), labels[b].detach().cpu(), self.current_task))
        while len(self._replay) > cap:                                   # evict from the task that holds the most rows,
            counts = {}                                                  # so that earlier tasks keep their share
            for r in self._replay:
                counts[r[2]] = counts.get(r[2], 0) + 1
            big = max(counts, key=counts.get)
            self._replay.pop(next(i for i, r in enumerate(self._replay) if r[2] == big))
        return new_ids, new_lab

    def _continual_after_backward(self, lr: float) -> float:
        flat = self.model.flat
        w = flat.params.detach().float()
        eng = self.continual
        lr = eng.on_step(flat.grads, w, lr, self.current_task)            # Fisher update, forgetting-aware rate
        if eng.cfg.ecc_lambda > 0 and self._ewc_anchored:               # no pull before the first task has ended
            flat.grads.copy_(eng.regularized_grads(flat.grads, w))
        return lr

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, path, dl=None):
        codec.save_model(self.model, path)
        self._save_opt(path + ".opt")
        state = {"step": self.global_step, "loader_offset": dl.offset if dl is not None else 0,
                 "loss_scale": self.loss_scale, "rng": torch.get_rng_state().tolist(), "config": asdict(self.cfg)}
        with open(path + ".state.json", "w") as f:
            json.dump(state, f)

    def load_checkpoint(self, path, dl=None, resume=True):
        from ..quant.codec import load_state
        _, tensors = load_state(path)
        with torch.no_grad():
            for name, dst in self.model.named_tensors():
                dst.copy_(tensors[name].view(dst.shape).to(dst.dtype))
        if self.opt is not None:
            if hasattr(self.opt, "master"):
                lo, hi = getattr(self.opt, "lo", 0), getattr(self.opt, "hi", self.model.flat.numel)
                self.opt.master.copy_(self.model.flat.params[lo:hi].float())
            if os.path.exists(path + ".opt"):
                self._load_opt(path + ".opt")
        sp = path + ".state.json"
        if resume and os.path.exists(sp):
            st = json.load(open(sp))
            self.global_step = st["step"]
            self.loss_scale = st.get("loss_scale", self.loss_scale)
            if dl is not None:
                dl.offset = st.get("loader_offset", 0)
            torch.set_rng_state(torch.tensor(st["rng"], dtype=torch.uint8))

    def _param_slices(self):
        flat = self.model.flat
        lo, hi = getattr(self.opt, "lo", 0), getattr(self.opt, "hi", flat.numel)
        for p, off in zip(flat.params_list, flat.offsets):
            a, b = max(off, lo), min(off + p.numel(), hi)
            if a < b:
                yield a - lo, b - lo

    def _save_opt(self, path):
        """{i32 step, f32 lr, i32 n, per parameter: i64 n_m, m floats, i64 n_v, v floats} (little endian)."""
        import struct
        m = getattr(self.opt, "m", None)
        v = getattr(self.opt, "v", None)
        if m is None:
            m = self.opt.state.get("m") if hasattr(self.opt, "state") else None
            v = self.opt.state.get("v") if hasattr(self.opt, "state") else None
        slices = list(self._param_slices())
        with open(path, "wb") as f:
            f.write(struct.pack("<ifi", int(getattr(self.opt, "step_count", self.global_step)), float(self.cfg.learning_rate),
                                len(slices) if m is not None else 0))
            if m is None:
                return
            mc, vc = m.detach().float().cpu(), (v if v is not None else torch.zeros_like(m)).detach().float().cpu()
            for a, b in slices:
                f.write(struct.pack("<q", b - a)); f.write(mc[a:b].numpy().tobytes())
                f.write(struct.pack("<q", b - a)); f.write(vc[a:b].numpy().tobytes())

    def _load_opt(self, path):
        import struct

        import numpy as np
        data = open(path, "rb").read()
        step, lr, n = struct.unpack_from("<ifi", data, 0)
        if hasattr(self.opt, "step_count"):
            self.opt.step_count = step
        m = getattr(self.opt, "m", None)
        v = getattr(self.opt, "v", None)
        slices = list(self._param_slices())
        if m is None or n != len(slices):
            return
        off = 12
        for a, b in slices:
            (cnt,) = struct.unpack_from("<q", data, off); off += 8
            if cnt != b - a:
                raise ValueError(f"{path}: parameter size mismatch")
            m[a:b].copy_(torch.from_numpy(np.frombuffer(data, np.float32, cnt, off).copy())); off += 4 * cnt
            off += 8
            v[a:b].copy_(torch.from_numpy(np.frombuffer(data, np.float32, cnt, off).copy())); off += 4 * cnt

    # ---- EMA (reference ema_init / ema_step / ema_apply / ema_swap)
    def ema_init(self, decay=0.999): self.ema = ModelEMA(self.model.flat, decay)
    def ema_step(self): self.ema and self.ema.step()
    def ema_swap(self): self.ema and self.ema.swap()
    def ema_apply(self): self.ema and self.ema.apply()
    def ema_enabled(self) -> bool: return self.ema is not None


KINDS = {"dense": "dense", "pretrain": "dense", "finetune": "finetune", "fine_tune": "finetune", "ft": "finetune",
         "moe": "moe", "native": "native"}


def unified_trainer_parse_kind(s: str) -> Optional[str]:
    return KINDS.get(s.lower())


@dataclass
class UnifiedTrainArgs:
    kind: str = "dense"
    data: str = ""
    optimizer: str = "adafactor"
    batch_size: int = 8
    seq_length: int = 512
    epochs: int = 3
    lr: float = 3e-4
    log_interval: int = 10
    save_interval: int = 1000
    output: str = "model.quant"
    max_steps: int = 10000
    seed: int = 42


class UnifiedTrainer:
    """Single entry for the CLIs (reference UnifiedTrainer: configure / run / train_step_once /
    save_checkpoint / load_checkpoint / metrics, src/trainer/trainer_core.cpp:1190-1327)."""

    def __init__(self, model, tokenizer=None):
        self.model, self.tok = model, tokenizer
        self.trainer: Optional[Trainer] = None
        self.args: Optional[UnifiedTrainArgs] = None

    def configure(self, args: UnifiedTrainArgs):
        if unified_trainer_parse_kind(args.kind) is None:
            raise ValueError(f"unknown trainer kind '{args.kind}'")
        if args.optimizer.lower() not in ("adafactor", "adamw") and args.optimizer.lower() not in __import__(
                "transformers_fusion_b200.trainer.optimizers", fromlist=["OPTIMIZERS"]).OPTIMIZERS:
            raise ValueError(f"unknown optimizer '{args.optimizer}'")
        self.args = args
        cfg = TrainConfig(batch_size=args.batch_size, seq_length=args.seq_length, epochs=args.epochs, learning_rate=args.lr,
                          log_interval=args.log_interval, save_interval=args.save_interval, optimizer=args.optimizer.lower(),
                          checkpoint_path=args.output, max_steps=args.max_steps, seed=args.seed, zero_stage=0)
        if unified_trainer_parse_kind(args.kind) == "moe":
            from .moe_trainer import MoETrainer
            self.trainer = MoETrainer(self.model, self.tok)
        else:
            self.trainer = Trainer(self.model, self.tok)
        self.trainer.compile(None, cfg)
        return self

    def run(self, log_cb=None):
        a = self.args
        dev = self.model.tok_embeddings.device
        dl = DataLoader(self.tok, a.data, a.batch_size, a.seq_length, device=dev)
        if log_cb:
            self.trainer.set_log_callback(log_cb)
        return self.trainer.fit(dl)

    def train_step_once(self, ids, labels) -> float:
        return self.trainer.train_step(ids, labels)

    def inner(self) -> Optional["Trainer"]:
        """The trainer built by ``configure`` (None before it)."""
        return self.trainer

    def set_log_callback(self, cb):
        if self.trainer is None:
            raise RuntimeError("configure() first")
        self.trainer.set_log_callback(cb)

    def save_checkpoint(self, path): self.trainer.save_checkpoint(path)
    def load_checkpoint(self, path): self.trainer.load_checkpoint(path)
    def metrics(self): return self.trainer.metrics()
