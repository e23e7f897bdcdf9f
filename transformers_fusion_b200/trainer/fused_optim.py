"""Flat-buffer optimizers driven by the fused kernels.

``FlatAdamW`` owns fp32 master weights and moments for a contiguous element range of the model's
flat parameter buffer (the whole buffer on one GPU, this rank's shard under ZeRO).  One step is:
sum-of-squares of the gradient range -> (all-reduce of the scalar when sharded) -> clip factor on
the device -> one fused kernel that applies the update, refreshes the bf16 compute copy and zeroes
the gradients.  Nothing in the step synchronises with the host.

Update rule and ordering follow the reference AdamW::step (src/trainer/optimizer.cpp:91-121):
clip, schedule, bias-corrected moments, decoupled weight decay.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..ops import functional as F


class FlatAdamW:
    def __init__(self, flat, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, max_grad_norm=1.0,
                 shard: Optional[tuple] = None, norm_reduce: Optional[Callable] = None):
        """``flat``: models.dense.FlatBuffers.  ``shard``: (start, end) element range owned by this
        rank (default: everything).  ``norm_reduce``: callable that sums the 1-element squared-norm
        tensor across the ranks that hold the other shards."""
        self.flat = flat
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.lo, self.hi = shard if shard is not None else (0, flat.numel)
        self.norm_reduce = norm_reduce
        dev = flat.params.device
        n = self.hi - self.lo
        self.master = flat.params[self.lo:self.hi].float().clone()
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.step_count = 0
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self._clip = torch.ones(1, dtype=torch.float32, device=dev)
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
        # {lr, 1 - beta1^t, 1 - beta2^t} staged through pinned memory so a captured graph sees fresh values
        self.hyper = torch.zeros(4, dtype=torch.float32, device=dev)
        # ring of slots: the host may run many steps ahead of the asynchronous uploads
        self._hyper_host = torch.zeros(256, 4, dtype=torch.float32)
        self._hyper_events = None
        if dev.type == "cuda":
            self._hyper_host = self._hyper_host.pin_memory()
            self._hyper_events = [None] * 256          # per slot: recorded after the slot's upload was enqueued

    def stage_hyper(self, lr: Optional[float] = None):
        """Advance the step counter and upload this step's scalars (call outside a graph replay)."""
        self.step_count += 1
        slot = self.step_count % 256
        h = self._hyper_host[slot]
        if self._hyper_events is not None and self._hyper_events[slot] is not None:
            self._hyper_events[slot].synchronize()     # the upload that last used this slot (256 steps ago) must be done
        h[0] = self.lr if lr is None else lr
        h[1] = 1.0 - self.betas[0] ** self.step_count
        h[2] = 1.0 - self.betas[1] ** self.step_count
        self.hyper.copy_(h, non_blocking=True)
        if self._hyper_events is not None:
            if self._hyper_events[slot] is None:
                self._hyper_events[slot] = torch.cuda.Event()
            self._hyper_events[slot].record()

    def step(self, lr: Optional[float] = None, inv_loss_scale: float = 1.0, staged: bool = False):
        if not staged:
            self.stage_hyper(lr)
        g = self.flat.grads[self.lo:self.hi]
        self._sumsq.zero_()
        F.sumsq(g, self._sumsq)
        if self.norm_reduce is not None:
            self.norm_reduce(self._sumsq)
        F.clip_factor(self._sumsq, inv_loss_scale, self.max_grad_norm, self.grad_norm, self._clip, self.found_inf)
        F.adamw_(self.master, g, self.m, self.v, self.flat.params[self.lo:self.hi], self.lr if lr is None else lr,
                 self.betas[0], self.betas[1], self.eps, self.weight_decay, self.step_count, self._clip, True, self.hyper)

    def zero_grad(self):
        self.flat.grads.zero_()

    # ---- checkpoint (reference `.opt` layout is produced by trainer.checkpoint from these) ----
    def state_dict(self):
        return {"step": self.step_count, "lr": self.lr, "m": self.m, "v": self.v, "master": self.master,
                "range": (self.lo, self.hi)}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        self.lr = float(sd.get("lr", self.lr))
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if "master" in sd and sd["master"] is not None:
            self.master.copy_(sd["master"])
            self.flat.params[self.lo:self.hi].copy_(self.master.to(self.flat.params.dtype))
