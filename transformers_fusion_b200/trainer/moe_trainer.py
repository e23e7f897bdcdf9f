"""MoE trainer: the Trainer loop with the mixture-of-experts bookkeeping of the reference's MoETrainer
(include/quant/moe_trainer.h:63-190, src/trainer/moe_trainer.cpp).

What it adds to ``Trainer``:

* auxiliary losses with true gradients: load balance and router z-loss flow through the router (in the reference they
  only rescale the cross-entropy gradient, src/trainer/moe_trainer.cpp:342-410); per-step metrics report them separately
  (``load_balance_loss``, ``z_loss``, ``aux_loss``, ``total_loss``), with the tokens no expert served and the number of
  experts that received tokens;
* its own accumulation window: ``train_step(ids, labels, loader=dl)`` draws a fresh micro-batch from the loader for every
  micro-step after the first (src/trainer/moe_trainer.cpp:289-340); without a loader the batch is cut into equal slices;
* a loss-scaled path (``mixed_precision``): gradients are produced under ``loss_scale``, unscaled before clipping, a step
  with non-finite gradients is skipped and halves the scale, a norm above twice the clip threshold halves it too, any
  other step grows it by 1 % (src/trainer/moe_trainer.cpp:231-287);
* fp32 master copies of the parameters (``init_mixed_precision`` / ``mp_quantize_forward`` / ``mp_restore_master``,
  src/trainer/moe_trainer.cpp:641-672) and the EMA calls (``ema_init / ema_step / ema_apply / ema_swap``);
* ``MoETrainingPipeline``: file-to-checkpoints loop with per-epoch ``moe_epoch_{e}.quant`` + JSON metadata, a log file,
  early stopping on the validation loss and a status report (src/trainer/moe_trainer.cpp:676-891).

The fast path is unchanged: with one micro-step, no loss scaling and the fused AdamW, ``train_step`` is the engine's
graph-replayable step."""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .fused_optim import FlatAdamW
from .trainer import DataLoader, TrainConfig, Trainer, TrainMetrics


@dataclass
class MoETrainConfig(TrainConfig):
    load_balance_weight: float = 0.01
    router_z_weight: float = 0.001
    aux_loss_weight: float = 0.01
    capacity_factor: float = 2.0
    expert_dropout: float = 0.0
    expert_parallel: int = 1
    expert_parallel_rank: int = 0
    mixed_precision: bool = False
    optimizer: str = "adamw"
    zero_stage: int = 0
    output_path: str = "moe_model.quant"


@dataclass
class MoEMetrics(TrainMetrics):
    aux_loss: float = 0.0               # weighted sum that was added to the loss (what the gradients saw)
    load_balance_loss: float = 0.0      # E * sum_e f_e P_e, mean over layers (unweighted)
    z_loss: float = 0.0                 # mean logsumexp(router logits)^2, mean over layers (unweighted)
    total_loss: float = 0.0
    expert_utilization: List[float] = field(default_factory=list)   # routed fraction per expert, mean over layers
    mean_expert_utilization: float = 0.0    # fraction of experts that received at least one token
    load_imbalance: float = 0.0         # max / mean routed fraction
    dropped_tokens: int = 0
    tokens_dropped_total: int = 0       # the reference's name for the same count
    num_experts_used: int = 0
    tokens_processed: int = 0
    active_params: int = 0
    total_params: int = 0


def load_balance_loss(router_logits: torch.Tensor, expert_indices: torch.Tensor, num_experts: Optional[int] = None) -> float:
    """Switch / GShard balance term E * sum_e f_e * P_e: f_e the fraction of (token, slot) picks that went to expert e,
    P_e the mean soft-max probability of e (reference: moe::compute_load_balance_loss, src/model/moe_variants.cpp:141-174)."""
    if router_logits.numel() == 0 or expert_indices.numel() == 0:
        return 0.0
    E = num_experts or router_logits.shape[-1]
    lg = router_logits.reshape(-1, router_logits.shape[-1]).float()
    idx = expert_indices.reshape(-1).long()
    idx = idx[(idx >= 0) & (idx < E)]
    f = torch.bincount(idx, minlength=E).float() / max(1, idx.numel())
    P = torch.softmax(lg, -1).mean(0)
    return float(E * (f * P[:E]).sum())


class MoETrainer(Trainer):
    def __init__(self, model, tokenizer=None, expert_parallel=None):
        super().__init__(model, tokenizer)
        self._metrics = MoEMetrics()
        self.expert_parallel = expert_parallel
        self.verbose = False
        self._mp_master: Optional[torch.Tensor] = None
        self._tokens = 0

    # ------------------------------------------------------------------ configuration
    def compile(self, optimizer=None, cfg=None, symm=None):
        cfg = cfg or MoETrainConfig()
        for blk in self.model.layers:
            blk.cfg.load_balance_weight = getattr(cfg, "load_balance_weight", blk.cfg.load_balance_weight)
            blk.cfg.router_z_weight = getattr(cfg, "router_z_weight", blk.cfg.router_z_weight)
            if getattr(cfg, "capacity_factor", 0):
                blk.cfg.capacity_factor = cfg.capacity_factor
        super().compile(optimizer, cfg, symm)
        if getattr(cfg, "mixed_precision", False):
            self.loss_scale = cfg.loss_scale
            self.init_mixed_precision()
        m = self._metrics
        m.total_params = sum(p.numel() for p in self.model.parameters())
        m.active_params = self._active_params()
        return self

    def _active_params(self) -> int:
        """Parameters one token touches: everything except the experts it is not routed to."""
        c = self.model.cfg
        experts = sum(l.gate_up.numel() + l.down.numel() for l in self.model.layers)
        total = sum(p.numel() for p in self.model.parameters())
        k = min(getattr(c, "top_k", 1), c.num_experts)
        return int(total - experts + experts * k // max(1, c.num_experts))

    def set_gradient_accumulation_steps(self, n: int): self.cfg.grad_accum_steps = max(1, int(n))
    def gradient_accumulation_steps(self) -> int: return self.cfg.grad_accum_steps
    def set_verbose(self, v: bool): self.verbose = bool(v)
    def get_model_params(self): return list(self.model.parameters())

    # ------------------------------------------------------------------ expert statistics
    def compute_expert_utilization(self):
        u = self.model.expert_utilization()
        return torch.stack(u).mean(0) if u else torch.zeros(self.model.cfg.num_experts)

    def compute_aux_loss(self, router_logits=None, expert_indices=None) -> float:
        """Without arguments: the weighted auxiliary loss of the last forward.  With the router logits and the chosen
        expert ids of one layer: the canonical balance term of that layer."""
        if router_logits is not None:
            return load_balance_loss(router_logits, expert_indices)
        a = self.model.last_aux
        return float(a.detach()) if torch.is_tensor(a) else float(a or 0.0)

    def _collect_expert_stats(self, ce: float):
        m, layers = self._metrics, [l for l in self.model.layers if hasattr(l, "last_idx")]
        u = self.compute_expert_utilization()
        m.aux_loss = self.compute_aux_loss()
        m.expert_utilization = u.tolist()
        m.load_imbalance = float(u.max() / u.mean().clamp(min=1e-9))
        m.num_experts_used = int((u > 0).sum())
        m.mean_expert_utilization = m.num_experts_used / max(1, u.numel())
        lb = z = 0.0
        dropped = 0
        for l in layers:
            lg = getattr(l, "last_logits", None)
            if lg is not None:
                finite = lg.float().clamp(min=-1e4)              # masked logits carry a large negative fill
                lb += load_balance_loss(finite, l.last_idx)
                z += float(torch.logsumexp(finite, -1).pow(2).mean())
            cov = getattr(l, "last_covered", None)
            if cov is not None:
                dropped += int((cov == 0).sum())
        n = max(1, len(layers))
        m.load_balance_loss, m.z_loss = lb / n, z / n
        m.dropped_tokens = m.tokens_dropped_total = dropped
        m.total_loss = ce + m.aux_loss

    # ------------------------------------------------------------------ steps
    def micro_step(self, ids, labels, loss_scale: float = 1.0):
        """Forward + backward of one micro-batch under ``loss_scale`` (the caller divides by the window length).
        Returns cross entropy + the weighted auxiliary losses as a float."""
        ce = float(self.model.forward_backward(ids, labels, loss_scale=loss_scale, label_smoothing=self.cfg.label_smoothing))
        self._collect_expert_stats(ce)
        return self._metrics.total_loss

    def unscale_gradients(self, scale: float):
        if scale != 1.0:
            self.model.flat.grads.mul_(1.0 / scale)

    def train_step(self, ids, labels, loader=None) -> float:
        c = self.cfg
        accum = max(1, c.grad_accum_steps)
        mp = bool(getattr(c, "mixed_precision", False))
        fast = isinstance(self.opt, FlatAdamW) and accum == 1 and not mp and not c.dynamic_loss_scale \
            and c.grad_noise_eta == 0 and loader is None
        if fast:
            loss = super().train_step(ids, labels)
            self._collect_expert_stats(loss)
            self._tokens += ids.numel()
            self._metrics.tokens_processed = self._tokens
            return loss
        lr = self.lr_at(self.global_step)
        scale = self.loss_scale if (mp or c.dynamic_loss_scale) else 1.0
        if self._mp_master is not None:
            self.mp_quantize_forward()
        if loader is not None:
            batches = [(ids, labels)] + [loader.next_batch() for _ in range(accum - 1)]
            dev = ids.device
            batches = [(i.to(dev), l.to(dev)) for i, l in batches]
        else:
            batches = list(zip(ids.chunk(accum), labels.chunk(accum)))
        total = sum(self.micro_step(i, l, scale / len(batches)) for i, l in batches) / len(batches)
        self._tokens += sum(i.numel() for i, _ in batches)
        if c.grad_noise_eta > 0:
            self.inject_gradient_noise(self.global_step, c.grad_noise_eta, c.grad_noise_gamma)
        self.unscale_gradients(scale)
        g = self.model.flat.grads
        m = self._metrics
        if scale != 1.0 and not bool(torch.isfinite(g).all()):
            self.loss_scale = max(1.0, self.loss_scale / 2)     # overflow: drop the step
            g.zero_()
            m.grad_norm = float("inf")
        else:
            m.grad_norm = float(g.norm())                       # the optimizer clips; the norm also drives the scale rule
            if scale != 1.0:
                grew = c.max_grad_norm > 0 and m.grad_norm > 2 * c.max_grad_norm
                self.loss_scale = max(1.0, self.loss_scale / 2) if grew else min(65536.0, self.loss_scale * 1.01)
            self.opt.step(lr)
            if self._mp_master is not None:
                self.mp_restore_master()
            if self.ema:
                self.ema.step()
        self.global_step += 1
        m.loss = m.total_loss - m.aux_loss
        m.perplexity, m.learning_rate, m.step = math.exp(min(m.loss, 20.0)), lr, self.global_step
        m.tokens_processed = self._tokens
        return total

    # ------------------------------------------------------------------ EMA / master copies
    def ema_apply(self):
        """Overwrite the parameters with their moving average (the average itself is kept)."""
        if self.ema is not None:
            self.model.flat.params.copy_(self.ema.shadow.to(self.model.flat.params.dtype))

    def init_mixed_precision(self):
        """Keep an fp32 master copy of the flat parameter buffer."""
        if self._mp_master is None:
            self._mp_master = self.model.flat.params.detach().float().clone()

    def mixed_precision_active(self) -> bool: return self._mp_master is not None

    def mp_quantize_forward(self):
        """Write the master values, rounded to the compute dtype, into the parameters the forward pass reads."""
        if self._mp_master is not None:
            self.model.flat.params.copy_(self._mp_master.to(self.model.flat.params.dtype))

    def mp_restore_master(self):
        """Fold the optimizer's update back into the master copy: the master moves by exactly the step the (lower
        precision) parameters took, so small updates accumulate instead of being rounded away step after step.  (The
        reference blends 0.1 % of the parameters into the master instead, src/trainer/moe_trainer.cpp:661-672, which
        makes the master lag the trained weights; not reproduced.)"""
        if self._mp_master is not None:
            p = self.model.flat.params
            before = self._mp_master.to(p.dtype).float()
            self._mp_master.add_(p.float() - before)


class MoETrainingPipeline:
    """Epoch loop around a MoETrainer.

    ``MoETrainingPipeline(trainer, out_dir)`` + ``run(dl, epochs, steps_per_epoch)`` drives a given loader;
    ``MoETrainingPipeline(trainer, out_dir, train_path=..., val_path=...)`` + ``configure(cfg)`` + ``run(epochs)`` builds
    the loaders from text files with the trainer's tokenizer.  Every epoch writes ``moe_epoch{e}.quant`` and
    ``moe_epoch{e}.json``; with a validation loader the loop stops after ``patience`` epochs that did not improve the best validation loss by more
    than ``min_delta``."""

    def __init__(self, trainer: MoETrainer, out_dir: str = "checkpoints", train_path: str = "", val_path: str = ""):
        self.trainer, self.out_dir = trainer, out_dir
        self.train_path, self.val_path = train_path, val_path
        self.cfg = trainer.cfg
        self.log_path = ""
        self.patience, self.min_delta, self._best_val, self._no_improve = 3, 0.0, 1e10, 0
        self.world_size, self.rank = 1, 0
        self._train_dl = self._val_dl = None
        os.makedirs(out_dir, exist_ok=True)

    # ---- configuration
    def configure(self, cfg: MoETrainConfig):
        self.cfg = cfg
        self.trainer.compile(None, cfg)
        self._train_dl = self._loader(self.train_path)
        self._val_dl = self._loader(self.val_path)
        return self

    def set_log_file(self, path: str): self.log_path = path

    def set_checkpoint_dir(self, d: str):
        os.makedirs(d, exist_ok=True)
        self.out_dir = d

    def set_distributed(self, world_size: int, rank: int):
        self.world_size, self.rank = world_size, rank
        self.cfg.expert_parallel, self.cfg.expert_parallel_rank = world_size, rank

    def model(self): return self.trainer.model
    def last_metrics(self) -> MoEMetrics: return self.trainer.metrics()

    def _loader(self, path):
        if not path or self.trainer.tok is None:
            return None
        dev = self.trainer.model.tok_embeddings.device
        return DataLoader(self.trainer.tok, path, self.cfg.batch_size, self.cfg.seq_length, device=dev)

    def _log(self, line: str):
        if self.trainer.verbose:
            print(line)
        if self.log_path:
            with open(self.log_path, "a") as f:
                f.write(line + "\n")

    # ---- the loop
    def should_stop_early(self, val_loss: float) -> bool:
        if val_loss < self._best_val - self.min_delta:
            self._best_val, self._no_improve = val_loss, 0
            return False
        self._no_improve += 1
        return self._no_improve >= self.patience

    def run_epoch(self, epoch: int, dl=None, steps: Optional[int] = None, val_dl=None) -> dict:
        dl = dl if dl is not None else self._train_dl
        val_dl = val_dl if val_dl is not None else self._val_dl
        tr = self.trainer
        steps = min(len(dl), self.cfg.max_steps) if steps is None else steps
        t0, tok0 = time.perf_counter(), tr.metrics().tokens_processed
        losses = []
        for _ in range(steps):
            ids, labels = dl.next_batch()
            losses.append(tr.train_step(ids, labels, loader=dl if self.cfg.grad_accum_steps > 1 else None))
            m = tr.metrics()
            if self.cfg.log_interval and m.step % self.cfg.log_interval == 0:
                self._log(f"Step {m.step} | loss: {m.loss:.4f} | ppl: {m.perplexity:.2f} | aux_loss: {m.aux_loss:.6f} | "
                          f"grad_norm: {m.grad_norm:.4f} | lr: {m.learning_rate:.6f} | "
                          f"util: {100 * m.mean_expert_utilization:.2f}% | lb: {m.load_balance_loss:.6f} | z: {m.z_loss:.6f}")
        m = tr.metrics()
        m.epoch = epoch
        m.tokens_per_sec = (m.tokens_processed - tok0) / max(1e-9, time.perf_counter() - t0)
        val = None
        if val_dl is not None:
            val_dl.reset()                                       # the same validation batches every epoch
            val = tr.eval_loss(val_dl)
        meta = self.save_checkpoint(epoch, sum(losses) / max(1, len(losses)), val)
        self._log(f"Epoch {epoch} complete | avg_loss: {meta['mean_loss']:.4f} | ppl: {m.perplexity:.2f}"
                  + (f" | val_loss: {val:.4f}" if val is not None else ""))
        return meta

    def save_checkpoint(self, epoch: int, mean_loss: float, val_loss: Optional[float] = None) -> dict:
        tr, c = self.trainer, self.trainer.model.cfg
        path = os.path.join(self.out_dir, f"moe_epoch{epoch}.quant")
        tr.save_checkpoint(path)
        m = tr.metrics()
        meta = {"epoch": epoch, "mean_loss": mean_loss, "loss": m.loss, "val_loss": val_loss, "step": m.step,
                "perplexity": m.perplexity, "aux_loss": m.aux_loss, "load_balance_loss": m.load_balance_loss,
                "z_loss": m.z_loss, "expert_utilization": m.expert_utilization, "load_imbalance": m.load_imbalance,
                "tokens_dropped": m.tokens_dropped_total, "hidden_size": c.hidden_size, "num_layers": c.num_layers,
                "num_experts": c.num_experts, "top_k": c.top_k, "total_params": m.total_params,
                "active_params": m.active_params}
        with open(path[:-6] + ".json", "w") as f:
            json.dump(meta, f)
        return meta

    def run(self, dl=None, epochs: int = -1, steps_per_epoch: Optional[int] = None, val_dl=None):
        """``run(dl, epochs, steps_per_epoch)`` or, after ``configure``, ``run(epochs)``.  Returns one record per epoch."""
        if isinstance(dl, int):
            dl, epochs = None, dl
        epochs = self.cfg.epochs if epochs < 0 else epochs
        history = []
        for e in range(epochs):
            meta = self.run_epoch(e, dl, steps_per_epoch, val_dl)
            history.append(meta)
            if meta["val_loss"] is not None and self.should_stop_early(meta["val_loss"]):
                self._log(f"Early stop after epoch {e}: no improvement in {self.patience} epochs")
                break
        return history

    def status_report(self) -> str:
        m, c = self.trainer.metrics(), self.trainer.model.cfg
        return "\n".join([
            "MoE Training Report", "===================",
            f"Model: {m.total_params} total params, {m.active_params} active per token",
            f"Layers: {c.num_layers}", f"Experts: {c.num_experts} (top-{c.top_k})", f"Hidden: {c.hidden_size}",
            f"Steps: {m.step}", f"Loss: {m.loss:.4f}", f"Perplexity: {m.perplexity:.2f}", f"Grad Norm: {m.grad_norm:.4f}",
            f"LR: {m.learning_rate:.6g}", f"Expert Utilization: {100 * m.mean_expert_utilization:.1f}%",
            f"Tokens dropped (last step): {m.tokens_dropped_total}"])
