"""MoE trainer: the Trainer loop plus expert-utilisation metrics, true auxiliary-loss gradients
(load balance + router z-loss flow through the router, unlike the reference where they only rescale
the CE gradient: src/trainer/moe_trainer.cpp:342-410) and per-epoch pipeline checkpoints with JSON
metadata (``moe_epoch{e}.quant``, src/trainer/moe_trainer.cpp:676-891).

API parity: MoETrainer(compile, fit, train_step, micro_step, eval_loss, clip_gradients,
save/load_checkpoint, metrics -> MoEMetrics, compute_expert_utilization, compute_aux_loss)
(include/quant/moe_trainer.h:63-190); MoETrainConfig{lb .01, z .001, aux .01, capacity 2}."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List

import torch

from .trainer import TrainConfig, Trainer, TrainMetrics


@dataclass
class MoETrainConfig(TrainConfig):
    load_balance_weight: float = 0.01
    router_z_weight: float = 0.001
    aux_loss_weight: float = 0.01
    capacity_factor: float = 2.0
    expert_parallel: int = 1
    optimizer: str = "adamw"
    zero_stage: int = 0


@dataclass
class MoEMetrics(TrainMetrics):
    aux_loss: float = 0.0
    expert_utilization: List[float] = field(default_factory=list)
    load_imbalance: float = 0.0     # max / mean routed fraction
    dropped_tokens: int = 0


class MoETrainer(Trainer):
    def __init__(self, model, tokenizer=None):
        super().__init__(model, tokenizer)
        self._metrics = MoEMetrics()

    def compile(self, optimizer=None, cfg=None, symm=None):
        cfg = cfg or MoETrainConfig()
        for blk in self.model.layers:
            blk.cfg.load_balance_weight = getattr(cfg, "load_balance_weight", blk.cfg.load_balance_weight)
            blk.cfg.router_z_weight = getattr(cfg, "router_z_weight", blk.cfg.router_z_weight)
        return super().compile(optimizer, cfg, symm)

    def compute_expert_utilization(self):
        u = self.model.expert_utilization()
        return torch.stack(u).mean(0) if u else torch.zeros(self.model.cfg.num_experts)

    def compute_aux_loss(self) -> float:
        a = self.model.last_aux
        return float(a.detach()) if a is not None else 0.0

    def train_step(self, ids, labels) -> float:
        loss = super().train_step(ids, labels)
        m = self._metrics
        u = self.compute_expert_utilization()
        m.aux_loss = self.compute_aux_loss()
        m.expert_utilization = u.tolist()
        m.load_imbalance = float(u.max() / u.mean().clamp(min=1e-9))
        return loss


class MoETrainingPipeline:
    """Epoch loop that writes ``moe_epoch{e}.quant`` + ``moe_epoch{e}.json`` into ``out_dir``."""

    def __init__(self, trainer: MoETrainer, out_dir: str):
        self.trainer, self.out_dir = trainer, out_dir
        os.makedirs(out_dir, exist_ok=True)

    def run(self, dl, epochs: int, steps_per_epoch: int):
        history = []
        for e in range(epochs):
            losses = [self.trainer.train_step(*dl.next_batch()) for _ in range(steps_per_epoch)]
            path = os.path.join(self.out_dir, f"moe_epoch{e}.quant")
            self.trainer.save_checkpoint(path, dl)
            m = self.trainer.metrics()
            meta = {"epoch": e, "mean_loss": sum(losses) / len(losses), "aux_loss": m.aux_loss,
                    "expert_utilization": m.expert_utilization, "load_imbalance": m.load_imbalance,
                    "num_experts": self.trainer.model.cfg.num_experts, "top_k": self.trainer.model.cfg.top_k}
            with open(path[:-6] + ".json", "w") as f:
                json.dump(meta, f)
            history.append(meta)
        return history
