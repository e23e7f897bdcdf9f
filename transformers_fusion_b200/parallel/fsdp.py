"""Fully sharded data parallelism (ZeRO stage 3) and its relatives.

``FullyShardedDataParallel`` keeps 1/W of every weight matrix (contiguous 128-row blocks) plus the matching fp32 master /
Adam state on each rank.  A forward or backward GEMM that needs the whole matrix gathers it *inside the GEMM launch*:
a few CTAs of the kernel pull the ranks' row shards over NVLink into one of two per-block gather buffers and raise a flag
per 128-row block while the remaining CTAs already multiply the tiles of the local shard (``tfb_gemm_bf16_tp`` bit 4).
Gradients are reduce-scattered block by block while backward continues and the local shards are updated by one fused
AdamW; no parameter all-gather follows the update, because the next step's GEMMs pull what they need.  On CPU / gloo
(tests) the same schedule runs with all-gather / reduce-scatter collectives.  The engine itself is
``parallel.sharded.ShardedEngine``, which also composes this with tensor parallelism.

Also here: ``ZeroOptimizer`` (stage 1/2 facade with the reference's method names), ``CPUOffloadEngine`` (pinned host
pool + side stream for optimizer state), ``ActivationCheckpointing`` and ``profile_memory``.

Reference counterparts: include/quant/fsdp.h:18-155 + src/trainer/fsdp.cpp (forward :188-213, reduce_scatter_grads
:508-543, FSDPBlock :549-695), include/quant/zero_optimizer.h + zero_optimizer_core.cpp :41-335, CPUOffloadEngine
:366-603, zero_offload.cpp."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .collectives import DistributedContext


@dataclass
class FSDPConfig:
    stage: int = 3
    mixed_precision: bool = True
    max_grad_norm: float = 1.0
    activation_checkpointing: bool = False
    flatten_parameters: bool = True
    memory_limit_bytes: int = 0
    lr: float = 3e-4
    weight_decay: float = 0.01
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    copy_ctas: int = 8


@dataclass
class MemoryProfile:
    parameters: int = 0
    gradients: int = 0
    optimizer_state: int = 0
    activations: int = 0
    total: int = 0


class FullyShardedDataParallel:
    """ZeRO stage 3 over the ranks of ``ctx`` with the reference's method names; the work is done by
    ``parallel.sharded.ShardedEngine`` (tensor-parallel degree 1 here; ``parallel.launch`` builds the dp x tp form).

    ``symm``: symmetric heap over the same ranks.  With it (CUDA) the weight gather runs inside the consuming GEMM, the
    gradient reduce-scatter is one peer-memory kernel per block overlapped with backward, and the shard update is one fused
    AdamW; without it the same schedule uses the library collectives."""

    def __init__(self, model, cfg: Optional[FSDPConfig] = None, ctx: Optional[DistributedContext] = None, symm=None):
        from .sharded import Mesh, ShardedEngine
        self.model, self.cfg = model, cfg or FSDPConfig()
        self.ctx = ctx or DistributedContext.init()
        self.rank, self.world = self.ctx.rank, self.ctx.world_size
        self.symm = symm
        c = self.cfg
        mesh = Mesh(self.rank, self.world, 0, 1, self.ctx.group, None, self.ctx.group)
        fused = symm is not None and model.tok_embeddings.is_cuda and self.world > 1
        self.engine = ShardedEngine.from_dense(model, mesh, comm="fused" if fused else "nccl", dp_heap=symm if fused else None,
                                               lr=c.lr, betas=c.betas, eps=c.eps, weight_decay=c.weight_decay,
                                               max_grad_norm=c.max_grad_norm, copy_ctas=c.copy_ctas)
        self.engine.activation_checkpointing = c.activation_checkpointing
        self.weights = list(self.engine.params.values())
        self.step_count = 0

    @property
    def gathers(self):
        return self.engine.gathers

    @property
    def last_grad_norm(self):
        return float(self.engine.last_grad_norm)

    # ---- step --------------------------------------------------------------------------------------------------
    def forward_backward(self, ids, labels):
        """Forward + backward of the local batch; the gradient reduce-scatter of each block is issued as soon as that
        block's backward is complete (reduce_scatter_grads of the reference, fsdp.cpp:508-543)."""
        return self.engine.forward_backward(ids, labels)

    def forward(self, ids):
        """Logits [B, S, V] of the current weights (gathers the whole model into ``self.model``: evaluation helper)."""
        self.consolidate()
        with torch.no_grad():
            return self.model.forward(ids)

    def optimizer_step(self, lr: Optional[float] = None):
        self.step_count += 1
        self.engine.optimizer_step(lr)

    def train_step(self, ids, labels, lr=None):
        loss = self.forward_backward(ids, labels)
        self.optimizer_step(lr)
        return loss

    def clip_gradients(self, max_norm: float) -> float:
        """Sets the clip threshold used by the next optimizer_step (the norm is global over all shards)."""
        self.engine.max_grad_norm = max_norm
        return self.last_grad_norm

    def zero_grad(self):
        self.engine.full_grad.zero_()
        self.engine.gshard.zero_()
        self.engine.small_grad.zero_()

    def scrub(self):
        """Forget every gathered weight (the engine does this itself after each optimizer step)."""
        self.engine.invalidate_gathers()

    def consolidate(self):
        """Gather every weight into ``self.model`` (for checkpointing or evaluation)."""
        self.engine.export_to(self.model)

    def profile_memory(self) -> MemoryProfile:
        mp_ = self.engine.memory_profile()
        mp = MemoryProfile()
        mp.parameters = mp_["parameters"] + mp_["gather_buffers"]
        mp.gradients = mp_["gradients"]
        mp.optimizer_state = mp_["optimizer_state"]
        mp.total = mp_["total"]
        return mp

    def memory_savings_ratio(self) -> float:
        """Fraction of the parameter + optimizer-state bytes this rank does not hold."""
        e = self.engine
        full = sum(p.rows * p.cols for p in e.params.values()) + e.small_lp.numel()
        mine = e.shard_numel + e.small_lp.numel()
        return 1.0 - mine / max(1, full)

    @staticmethod
    def auto_wrap(model, min_params: int = 1 << 16):
        """Names of the modules a per-block wrapper would shard (every transformer block above the threshold)."""
        return [f"layers.{i}" for i, l in enumerate(model.layers) if sum(p.numel() for p in l.parameters()) >= min_params]


class FSDPBlock:
    """Per-block view: which sharded weights belong to a layer, and their gather / gradient state."""

    def __init__(self, fsdp: FullyShardedDataParallel, layer_index: int):
        self.fsdp = fsdp
        self.unit = 1 + layer_index
        self.weights = list(fsdp.engine.units[self.unit])

    def gather_and_install(self):
        """Full matrices of the block's weights (library gather; the training path gathers inside its GEMMs)."""
        e = self.fsdp.engine
        return {p.name: e.gather_full(p.name) for p in self.weights}

    def release(self):
        for p in self.weights:
            p.gathered = False

    def shard_gradients(self):
        """This rank's reduced fp32 gradient shards of the block (valid after the block's backward)."""
        e = self.fsdp.engine
        return [e.gshard[p.shard_off:p.shard_off + p.per * p.cols].view(p.per, p.cols) for p in self.weights]


class ActivationCheckpointing:
    """Switch recomputation of block activations in the backward pass on or off for a model."""

    def __init__(self, model):
        self.model = model

    def enable(self, on: bool = True):
        self.model.activation_checkpointing = bool(on)
        return self

    def memory_saved_bytes(self, batch, seq):
        cfg = self.model.cfg
        per_block = batch * seq * (6 * cfg.hidden_size + 3 * cfg.ffn_hidden_size + (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim) * 2
        return per_block * cfg.num_layers - batch * seq * cfg.hidden_size * 2 * cfg.num_layers


class ZeroOptimizer:
    """Stage 1/2 facade over the training engine with the reference's method names (contiguous shard ownership)."""

    def __init__(self, model, rank=0, world_size=1, lr=3e-4, stage=2, symm=None, comm="nccl", **kw):
        from ..trainer.engine import TrainEngine
        self.engine = TrainEngine(model, lr=lr, zero_stage=stage, comm=comm if world_size > 1 else "none", symm=symm, **kw)
        self.model, self.rank, self.world = model, rank, world_size
        self.lr = lr
        self.grad_hooks, self.forward_hooks = [], []

    def register_model_params(self):
        return len(self.model.flat.params_list)

    def num_owned(self):
        lo, hi = self.engine.shard
        return hi - lo

    def get_shard(self, i=0):
        lo, hi = self.engine.shard
        return self.model.flat.params[lo:hi]

    def get_owned_state(self, i=0):
        o = self.engine.opt
        return {"master": o.master, "m": o.m, "v": o.v}

    def memory_savings_ratio(self):
        return 1.0 - 1.0 / max(1, self.world)

    def set_lr(self, lr):
        self.lr = lr

    def get_lr(self):
        return self.lr

    def set_grad_clip_norm(self, n):
        self.engine.opt.max_grad_norm = n

    def register_grad_hook(self, fn):
        self.grad_hooks.append(fn)

    def register_forward_hook(self, fn):
        self.forward_hooks.append(fn)

    def step(self, ids, labels):
        for h in self.forward_hooks:
            h(ids)
        loss = self.engine.step(ids, labels, self.lr)
        for h in self.grad_hooks:
            h(self.model.flat.grads)
        return loss

    def zero_grad(self):
        self.model.flat.zero_grad()


class CPUOffloadEngine:
    """Pinned host pool for optimizer state with asynchronous transfers on a side stream (double-buffered: while one
    tensor's update runs on the device, the next one's state is already on its way)."""

    def __init__(self, pool_bytes: int = 8 << 30, device=None):
        self.device = torch.device(device) if device is not None else (torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu"))
        self.pool_bytes, self.used = pool_bytes, 0
        self.host: Dict[str, torch.Tensor] = {}
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def offload(self, name: str, t: torch.Tensor):
        nbytes = t.numel() * t.element_size()
        if name not in self.host:
            if self.used + nbytes > self.pool_bytes:
                raise MemoryError("host pool exhausted")
            self.host[name] = torch.empty(t.shape, dtype=t.dtype, pin_memory=self.device.type == "cuda")
            self.used += nbytes
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                self.host[name].copy_(t, non_blocking=True)
        else:
            self.host[name].copy_(t)

    def fetch(self, name: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        h = self.host[name]
        out = out if out is not None else torch.empty(h.shape, dtype=h.dtype, device=self.device)
        if self.stream is not None:
            with torch.cuda.stream(self.stream):
                out.copy_(h, non_blocking=True)
        else:
            out.copy_(h)
        return out

    def prefetch(self, name, out=None):
        return self.fetch(name, out)

    def synchronize(self):
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def release(self, name):
        t = self.host.pop(name, None)
        if t is not None:
            self.used -= t.numel() * t.element_size()


class ZeROOffloadManager:
    """Keeps Adam's m and v of a flat optimizer on the host between steps."""

    def __init__(self, opt, engine: Optional[CPUOffloadEngine] = None):
        self.opt, self.engine = opt, engine or CPUOffloadEngine()
        self.on_host = False

    def to_host(self):
        self.engine.offload("m", self.opt.m)
        self.engine.offload("v", self.opt.v)
        self.engine.synchronize()
        self.on_host = True

    def to_device(self):
        self.engine.fetch("m", self.opt.m)
        self.engine.fetch("v", self.opt.v)
        self.engine.synchronize()
        self.on_host = False

    def step(self, fn):
        """Run ``fn`` (the optimizer update) with the state brought back, then park it again."""
        if self.on_host:
            self.to_device()
        r = fn()
        self.to_host()
        return r


ZeROOptimizer = ZeroOptimizer


class GradientCheckpointManager:
    """Chooses which layers recompute their activations in backward so that the saved activations fit a byte budget:
    layers are taken in order of bytes saved per recomputed FLOP (greedy), which for equal layers is simply "as few as
    needed".  Reference counterparts: GradientCheckpointManager (src/trainer/zero_offload.cpp) and the greedy placement of
    ActivationCheckpoint regions (src/trainer/zero_optimizer_mem.cpp:638)."""

    def __init__(self, activation_bytes, recompute_flops=None):
        self.bytes = [int(b) for b in activation_bytes]
        self.flops = [float(f) for f in (recompute_flops or [1.0] * len(self.bytes))]
        self.checkpointed = [False] * len(self.bytes)

    def plan(self, budget_bytes: int):
        """Marks layers until the saved activations (those of the layers not recomputed) fit; returns the marks."""
        self.checkpointed = [False] * len(self.bytes)
        order = sorted(range(len(self.bytes)), key=lambda i: -self.bytes[i] / max(self.flops[i], 1e-9))
        saved = sum(self.bytes)
        for i in order:
            if saved <= budget_bytes:
                break
            self.checkpointed[i] = True
            saved -= self.bytes[i]
        return list(self.checkpointed)

    def saved_bytes(self) -> int:
        return sum(b for b, c in zip(self.bytes, self.checkpointed) if not c)

    def recompute_overhead(self) -> float:
        """Extra forward FLOPs as a fraction of one forward pass."""
        tot = sum(self.flops)
        return sum(f for f, c in zip(self.flops, self.checkpointed) if c) / tot if tot else 0.0

    def apply(self, model):
        """Sets the per-model switch when every layer is marked (the dense model recomputes all layers or none) and
        returns the per-layer marks for engines that checkpoint selectively."""
        if hasattr(model, "activation_checkpointing"):
            model.activation_checkpointing = all(self.checkpointed) and bool(self.checkpointed)
        return list(self.checkpointed)
