"""Fully sharded data parallelism (ZeRO stage 3) and its relatives.

``FullyShardedDataParallel`` keeps 1/W of every weight matrix (contiguous 128-row blocks) plus the matching fp32 master /
Adam state on each rank.  A forward or backward GEMM that needs the whole matrix gathers it *inside the GEMM launch*:
the weight lives in a symmetric buffer, a few CTAs of the kernel pull the peers' row blocks over NVLink and raise a
flag per block while the remaining CTAs already multiply the tiles of the local shard (``tfb_gemm_bf16_tp`` mode 3).
Gradients are reduce-scattered and the local shards updated by the fused ZeRO kernels; no parameter all-gather follows
the update, because the next step's GEMMs pull what they need.  On CPU / gloo (tests) the same schedule runs with
``all_gather_into_tensor`` / reduce-scatter collectives.

Also here: ``ZeroOptimizer`` (stage 1/2 facade with the reference's method names), ``CPUOffloadEngine`` (pinned host
pool + side stream for optimizer state), ``ActivationCheckpointing`` and ``profile_memory``.

Reference counterparts: include/quant/fsdp.h:18-155 + src/trainer/fsdp.cpp (forward :188-213, reduce_scatter_grads
:508-543, FSDPBlock :549-695), include/quant/zero_optimizer.h + zero_optimizer_core.cpp :41-335, CPUOffloadEngine
:366-603, zero_offload.cpp."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib, functional as F
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


class ShardedWeight:
    """One weight matrix [rows, cols] sharded by rows.  ``full`` is a [rows_padded, cols] gather buffer (symmetric on
    GPUs); this rank's rows are always valid in place, the others only after a gather."""

    def __init__(self, name, param, rank, world, symm=None):
        self.name, self.param, self.rank, self.world = name, param, rank, world
        rows, cols = param.shape
        gran = 128 * world
        self.rows, self.cols = rows, cols
        self.rows_p = (rows + gran - 1) // gran * gran
        self.per = self.rows_p // world
        dev, dt = param.device, param.dtype
        self.symm_buf = None
        if symm is not None:
            self.symm_buf = symm.alloc(self.rows_p * cols, dt)
            self.full = self.symm_buf.view(dt, self.rows_p * cols).view(self.rows_p, cols)
            self.full.zero_()
        else:
            self.full = torch.zeros((self.rows_p, cols), dtype=dt, device=dev)
        self.full[:rows].copy_(param.data)
        lo = rank * self.per
        self.shard = self.full[lo:lo + self.per]                   # bf16 / compute-dtype shard, in place
        self.master = self.shard.float().clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.ready = torch.zeros(self.rows_p // 128, dtype=torch.int32, device=dev) if symm is not None else None
        self.epoch = 0
        param.data = self.full[:rows]                               # the model's kernels read the gather buffer

    def scrub_remote(self):
        """Forget the peers' rows (what ZeRO-3 frees between uses); used by tests to prove that gathers happen."""
        lo = self.rank * self.per
        self.full[:lo].zero_()
        self.full[lo + self.per:].zero_()


class FullyShardedDataParallel:
    def __init__(self, model, cfg: Optional[FSDPConfig] = None, ctx: Optional[DistributedContext] = None, symm=None):
        self.model, self.cfg = model, cfg or FSDPConfig()
        self.ctx = ctx or DistributedContext.init()
        self.rank, self.world = self.ctx.rank, self.ctx.world_size
        self.symm = symm
        self.step_count = 0
        model.flatten()
        self.weights: List[ShardedWeight] = []
        self.small: List[torch.nn.Parameter] = []     # norms, biases, embeddings: replicated, gradients all-reduced
        for n, p in model.named_parameters():
            if p.dim() == 2 and p.shape[0] >= 128 * self.world and n not in ("tok_embeddings", "lm_head", "pos_embeddings"):
                self.weights.append(ShardedWeight(n, p, self.rank, self.world, symm))
            else:
                self.small.append(p)
        self._by_param = {id(w.param): w for w in self.weights}
        self.small_state = [(p.data.float().clone(), torch.zeros(p.shape, device=p.device), torch.zeros(p.shape, device=p.device))
                            for p in self.small]
        self._install_hooks()
        self.gathers = 0

    # ---- gather ------------------------------------------------------------------------------------------------
    def gather(self, w: ShardedWeight):
        """Make every row of ``w.full`` valid on this rank (library path; the fused path does this inside the GEMM)."""
        if self.world == 1:
            return
        dist.all_gather_into_tensor(w.full.view(-1), w.shard.contiguous().view(-1), group=self.ctx.group)
        self.gathers += 1

    def _install_hooks(self):
        """Route the model's linear layers through gemm_gathered for sharded weights."""
        fsdp = self
        orig = F.gemm

        def gemm(a, b, *args, **kw):
            base = b._base if b._base is not None else b
            w = fsdp._by_storage.get(base.data_ptr()) if hasattr(fsdp, "_by_storage") else None
            if w is None or fsdp.world == 1 or kw.get("a_mn"):
                return orig(a, b, *args, **kw)
            return fsdp.gemm_gathered(a, w, b, orig, *args, **kw)
        self._by_storage = {w.full.data_ptr(): w for w in self.weights}
        self._gemm = gemm

    def gemm_gathered(self, a, w: ShardedWeight, b_view, orig, *args, **kw):
        fused = self.symm is not None and a.is_cuda and not kw.get("bias") is not None and kw.get("residual") is None \
            and kw.get("act") is None and kw.get("out_dtype") in (None, torch.bfloat16) and not kw.get("accumulate") \
            and b_view.shape[0] == w.rows_p
        if not fused:
            self.gather(w)
            return orig(a, b_view, *args, **kw)
        b_mn = bool(kw.get("b_mn"))
        M, K = a.shape
        N = w.cols if b_mn else w.rows_p
        out = kw.get("out")
        y = out if out is not None else torch.empty((M, N), dtype=a.dtype, device=a.device)
        from .tp import _Tp, _fn
        self.symm.barrier()                       # every rank's shard holds this step's values
        w.epoch += 1
        tp = _Tp(3, self.rank, self.world, self.cfg.copy_ctas, w.epoch, w.ready.data_ptr(), w.symm_buf.ptrs.data_ptr(), None)
        _lib.check(_fn()(a.data_ptr(), a.stride(0), w.full.data_ptr(), w.full.stride(0), int(b_mn), y.data_ptr(), y.stride(0),
                         M, N, K, C.byref(tp), _lib.status_word(a.device).data_ptr(), _lib.stream()), "gemm_weight_gather")
        self.gathers += 1
        return y

    # ---- step --------------------------------------------------------------------------------------------------
    def forward_backward(self, ids, labels):
        import transformers_fusion_b200.models.dense as dense_mod
        saved = dense_mod.F.gemm
        dense_mod.F.gemm = self._gemm
        try:
            if self.cfg.activation_checkpointing:
                self.model.activation_checkpointing = True
            return self.model.forward_backward(ids, labels)
        finally:
            dense_mod.F.gemm = saved

    def forward(self, ids):
        import transformers_fusion_b200.models.dense as dense_mod
        saved = dense_mod.F.gemm
        dense_mod.F.gemm = self._gemm
        try:
            with torch.no_grad():
                return self.model.forward(ids)
        finally:
            dense_mod.F.gemm = saved

    def reduce_scatter_grads(self):
        """Average gradients over ranks; each rank keeps the fp32 gradient of its own row shard."""
        W = self.world
        out = []
        for w in self.weights:
            g = w.param.main_grad                                   # [rows, cols] fp32
            gp = torch.zeros((w.rows_p, w.cols), dtype=torch.float32, device=g.device)
            gp[: w.rows].copy_(g)
            if W > 1:
                out.append(self.ctx.reduce_scatter(gp, "avg"))
            else:
                out.append(gp)
        for p in self.small:
            if W > 1:
                self.ctx.all_reduce(p.main_grad, "avg")
        return out

    def clip_gradients(self, shard_grads, max_norm: float) -> float:
        ss = sum(float((g * g).sum()) for g in shard_grads)
        t = torch.tensor([ss], device=self.model.tok_embeddings.device)
        if self.world > 1:
            self.ctx.all_reduce(t, "sum")
        ss = float(t) + sum(float((p.main_grad * p.main_grad).sum()) for p in self.small)
        norm = ss ** 0.5
        self.last_grad_norm = norm
        return min(1.0, max_norm / (norm + 1e-6)) if max_norm > 0 else 1.0

    def optimizer_step(self, lr: Optional[float] = None):
        c = self.cfg
        lr = c.lr if lr is None else lr
        self.step_count += 1
        t = self.step_count
        grads = self.reduce_scatter_grads()
        clip = self.clip_gradients(grads, c.max_grad_norm)
        b1, b2 = c.betas
        bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t

        def adam(master, m, v, g, wd):
            g = g * clip
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            master.mul_(1 - lr * wd).addcdiv_(m / bc1, (v / bc2).sqrt().add_(c.eps), value=-lr)
        for w, g in zip(self.weights, grads):
            adam(w.master, w.m, w.v, g, c.weight_decay)
            w.shard.copy_(w.master.to(w.shard.dtype))
        for p, (master, m, v) in zip(self.small, self.small_state):
            adam(master, m, v, p.main_grad, 0.0 if p.dim() < 2 else c.weight_decay)
            p.data.copy_(master.to(p.dtype))
        self.zero_grad()

    def train_step(self, ids, labels, lr=None):
        loss = self.forward_backward(ids, labels)
        self.optimizer_step(lr)
        return loss

    def zero_grad(self):
        self.model.flat.zero_grad()

    def scrub(self):
        for w in self.weights:
            w.scrub_remote()

    def consolidate(self):
        """Gather every weight (for checkpointing or evaluation)."""
        for w in self.weights:
            self.gather(w)

    def profile_memory(self) -> MemoryProfile:
        esz = self.model.tok_embeddings.element_size()
        sharded = sum(w.per * w.cols for w in self.weights)
        small = sum(p.numel() for p in self.small)
        mp = MemoryProfile()
        mp.parameters = (sharded + small) * esz
        mp.gradients = self.model.flat.numel * 4
        mp.optimizer_state = (sharded + small) * 12
        mp.total = mp.parameters + mp.gradients + mp.optimizer_state
        return mp

    def memory_savings_ratio(self) -> float:
        full = sum(w.rows * w.cols for w in self.weights) + sum(p.numel() for p in self.small)
        mine = sum(w.per * w.cols for w in self.weights) + sum(p.numel() for p in self.small)
        return 1.0 - mine / max(1, full)

    @staticmethod
    def auto_wrap(model, min_params: int = 1 << 16):
        """Names of the modules a per-block wrapper would shard (every transformer block above the threshold)."""
        return [f"layers.{i}" for i, l in enumerate(model.layers) if sum(p.numel() for p in l.parameters()) >= min_params]


class FSDPBlock:
    """Per-block view: gather one block's weights ahead of use (``gather_and_install``), and drop them afterwards."""

    def __init__(self, fsdp: FullyShardedDataParallel, layer_index: int):
        self.fsdp = fsdp
        pre = f"layers.{layer_index}."
        self.weights = [w for w in fsdp.weights if w.name.startswith(pre)]

    def gather_and_install(self):
        for w in self.weights:
            self.fsdp.gather(w)

    def release(self):
        for w in self.weights:
            w.scrub_remote()

    def shard_gradients(self):
        return [self.fsdp.ctx.reduce_scatter(torch.nn.functional.pad(w.param.main_grad, (0, 0, 0, w.rows_p - w.rows)), "avg")
                for w in self.weights]


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
