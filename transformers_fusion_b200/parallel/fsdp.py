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

    def forward(self, ids, labels=None):
        """Logits [B, S, V] of the current weights (gathers the whole model into ``self.model``: evaluation helper).  The
        batch is remembered, so that the reference's two-call form ``forward(ids); backward()`` works (fsdp.h:46-52)."""
        self._pending = (ids, labels)
        self.consolidate()
        with torch.no_grad():
            return self.model.forward(ids)

    def backward(self, loss_value=None, labels=None):
        """Gradients of the batch last given to ``forward`` (labels: those given there or here, else the ids shifted left
        by one).  The engine's step is one fused forward + backward with the per-unit reduce-scatter issued as backward
        proceeds, so this runs that step; ``loss_value`` is accepted for signature parity and not needed.  Returns the loss."""
        ids, lab = getattr(self, "_pending", (None, None))
        if ids is None:
            raise RuntimeError("backward() needs a batch: call forward(ids) first")
        lab = labels if labels is not None else lab
        if lab is None:
            lab = torch.cat([ids[:, 1:], torch.full_like(ids[:, :1], -100)], 1)
        self._pending = (None, None)
        return self.forward_backward(ids, lab)

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

    def print_memory_profile(self, file=None):
        mp = self.profile_memory()
        un = self.engine.memory_profile()["unsharded_total"]
        rows = [("parameters (+ gather buffers)", mp.parameters), ("gradients", mp.gradients),
                ("optimizer state", mp.optimizer_state), ("total", mp.total), ("unsharded total", un)]
        lines = [f"FSDP memory, rank {self.rank} of {self.world} (stage {self.cfg.stage}):"]
        lines += [f"  {k:<32}{v / 2**20:12.1f} MiB" for k, v in rows]
        text = "\n".join(lines)
        print(text, file=file)
        return text

    # ---- mixed precision / flat views ----------------------------------------------------------------------------
    def stage(self) -> int: return self.cfg.stage
    def is_mixed_precision(self) -> bool: return self.cfg.mixed_precision
    def world_size(self) -> int: return self.world
    def world_rank(self) -> int: return self.rank

    def to_fp16(self, t: torch.Tensor) -> torch.Tensor:
        """The compute-precision copy of a tensor: the dtype of the engine's weight shards (bf16 on the GPU path; the
        reference's name is kept, fsdp.h:64)."""
        return t.to(self.engine.shard_lp.dtype) if self.cfg.mixed_precision else t

    def to_fp32(self, t: torch.Tensor) -> torch.Tensor:
        return t.float()

    def flatten_and_shard(self) -> torch.Tensor:
        """This rank's flat fp32 master shard of every sharded matrix (one contiguous buffer: the engine flattens and
        shards at construction; this hands out the view, fsdp.h:75)."""
        return self.engine.master

    def unflatten_params(self):
        """Write the full, unflattened weights back into the wrapped model (every rank ends with the whole model)."""
        return self.consolidate()

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

    @torch.no_grad()
    def forward(self, h: torch.Tensor, batch: int, seq_len: int) -> torch.Tensor:
        """The block alone: its weights are gathered (or read inside the GEMMs), ``h`` [tokens / tp, hidden] goes through
        attention and the feed-forward, and the activations the backward needs are kept on the block."""
        e = self.fsdp.engine
        out, self._ctx = e._block_fwd(self.unit - 1, h, batch, seq_len)
        self._bs = (batch, seq_len)
        return out

    @torch.no_grad()
    def backward(self, grad_output: torch.Tensor) -> torch.Tensor:
        """Gradient of the block's input; the weight gradients are reduce-scattered into this rank's shards on the way."""
        if getattr(self, "_ctx", None) is None:
            raise RuntimeError("FSDPBlock.backward needs a forward first")
        e = self.fsdp.engine
        dh = e._block_bwd(self.unit - 1, self._ctx, grad_output, *self._bs)
        self._ctx = None
        e._unit_done(self.unit)
        return dh

    def sync_gradients(self):
        """The block's gradients are reduce-scattered by the engine as soon as the block's backward is done; this returns
        the reduced shards (nothing is left to synchronise afterwards)."""
        return self.shard_gradients()

    def memory_usage(self) -> int:
        """Bytes this rank holds for the block: weight shards, fp32 master + two Adam moments, reduced gradient shards."""
        e = self.fsdp.engine
        n = sum(p.per * p.cols for p in self.weights)
        return n * (e.shard_lp.element_size() + 12 + 4)


class ActivationCheckpointing:
    """Switch recomputation of block activations in the backward pass on or off for a model."""

    def __init__(self, model=None):
        self.model = model
        self._saved: Dict[int, torch.Tensor] = {}

    def enable(self, on: bool = True):
        self.model.activation_checkpointing = bool(on)
        return self

    # ---- explicit form (reference: fsdp.h:204-231): keep only a layer's input, run the layer again when needed
    def save_input(self, layer_idx: int, x: torch.Tensor):
        if not hasattr(self, "_saved"):
            self._saved = {}
        self._saved[int(layer_idx)] = x.detach()

    def recompute(self, block, layer_idx: int, *args, **kw):
        """Run ``block`` again from the input saved for ``layer_idx`` (with autograd on, so that the caller can
        back-propagate through the recomputed activations); extra arguments are passed to the block."""
        x = self._saved[int(layer_idx)].requires_grad_(True)
        with torch.enable_grad():
            return block(x, *args, **kw)

    def clear(self):
        self._saved = {}

    def saved_memory(self) -> int:
        """Bytes held by the saved inputs."""
        return sum(t.numel() * t.element_size() for t in getattr(self, "_saved", {}).values())

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

    def total_params(self) -> int:
        """Parameter tensors registered with the optimizer."""
        return len(self.model.flat.params_list)

    def owned_params(self) -> int:
        """Parameter tensors of which this rank's contiguous shard holds at least one element."""
        lo, hi = self.engine.shard
        flat = self.model.flat
        return sum(1 for p, off in zip(flat.params_list, flat.offsets) if off < hi and off + p.numel() > lo)

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

    # ---- the stage-3 verbs of the reference (zero_optimizer.h:48-52) over the flat buffers --------------------------
    def rank_(self) -> int: return self.rank
    def world_size(self) -> int: return self.world
    def step_count(self) -> int: return int(getattr(self.engine, "steps", 0))

    def all_gather_params(self):
        """Every rank receives every owner's slice of the flat parameter buffer (after a sharded update the engine does
        this inside its fused step; the call is for callers that changed their shard themselves)."""
        if self.world > 1 and dist.is_initialized():
            flat = self.model.flat.params
            n = flat.numel()
            per = -(-n // self.world)
            pad = torch.zeros(per * self.world, dtype=flat.dtype, device=flat.device)
            pad[:n].copy_(flat)
            mine = pad[self.rank * per:(self.rank + 1) * per].clone()
            dist.all_gather_into_tensor(pad, mine) if pad.is_cuda else dist.all_gather(list(pad.view(self.world, per).unbind(0)), mine)
            flat.copy_(pad[:n])
        return self.model.flat.params

    def reduce_scatter_grads(self):
        """Average the flat gradient over the ranks and return this rank's slice of it."""
        g = self.model.flat.grads
        lo, hi = self.engine.shard
        if self.world > 1 and dist.is_initialized():
            dist.all_reduce(g)
            g.div_(self.world)
        return g[lo:hi]

    def clip_grad_norm(self) -> float:
        """Scale the gradients so that their global norm does not exceed the configured threshold; returns the norm."""
        g = self.model.flat.grads
        norm = float(g.norm())
        mx = float(getattr(self.engine.opt, "max_grad_norm", 0.0) or 0.0)
        if mx > 0 and norm > mx:
            g.mul_(mx / (norm + 1e-6))
        return norm

    def state_bytes_owned(self) -> int: return self.num_owned() * 12
    def state_bytes_full(self) -> int: return self.model.flat.params.numel() * 12


class ShardOptimizer:
    """Optimizer for one rank's parameter shards, called shard by shard (the reference's ``ZeROOptimizer``,
    fsdp.h:233-268: Adafactor with a persistent factored state per shard buffer).  ``step`` updates a shard in place;
    ``step_mixed`` updates an fp32 master and writes its rounded value into the lower-precision shard."""

    def __init__(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-2, world_size=1, world_rank=0):
        self.lr, self.beta1, self.beta2, self.eps, self.wd = lr, beta1, beta2, eps, weight_decay
        self.world_size, self.world_rank = world_size, world_rank
        self._state: Dict[int, dict] = {}
        self._count = 0

    def param_count(self) -> int: return self._count
    def set_param_count(self, n: int): self._count = int(n)

    def _update(self, key: int, w32: torch.Tensor, g: torch.Tensor, step_num: int) -> torch.Tensor:
        g = g.float()
        st = self._state.setdefault(key, {})
        rho = min(self.beta2, 1.0 - (max(1, step_num)) ** -0.8)       # Adafactor's increasing decay
        g2 = g * g + 1e-30
        if g.dim() == 2 and min(g.shape) > 1:                           # factored second moment: row and column means
            r = st.setdefault("r", torch.zeros(g.shape[0], device=g.device))
            c = st.setdefault("c", torch.zeros(g.shape[1], device=g.device))
            r.mul_(rho).add_(g2.mean(1), alpha=1 - rho)
            c.mul_(rho).add_(g2.mean(0), alpha=1 - rho)
            v = torch.outer(r, c) / r.mean().clamp(min=1e-30)
        else:
            v = st.setdefault("v", torch.zeros_like(g))
            v.mul_(rho).add_(g2, alpha=1 - rho)
        u = g / (v.sqrt() + self.eps)
        u = u / max(1.0, float(u.pow(2).mean().sqrt()))                 # update clipping at RMS 1
        if self.wd:
            w32.mul_(1.0 - self.lr * self.wd)
        return w32.add_(u, alpha=-self.lr)

    @torch.no_grad()
    def step(self, param_shard: torch.Tensor, grad_shard: torch.Tensor, step_num: int):
        w = self._update(param_shard.data_ptr(), param_shard.float(), grad_shard, step_num)
        param_shard.copy_(w.to(param_shard.dtype))
        return param_shard

    @torch.no_grad()
    def step_mixed(self, param_shard: torch.Tensor, fp32_master: torch.Tensor, grad_shard: torch.Tensor, step_num: int):
        self._update(fp32_master.data_ptr(), fp32_master, grad_shard, step_num)
        param_shard.copy_(fp32_master.to(param_shard.dtype))
        return param_shard


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

    # ---- the reference's verbs (include/quant/zero_optimizer.h: CPUOffloadEngine): parameters addressed by id, counters
    def offload_single(self, param_id: int, t: torch.Tensor):
        self.offload(f"param{int(param_id)}", t)
        self._count("off", t)
        self.__dict__.setdefault("_devs", {})[int(param_id)] = t

    def offload_params(self, params):
        """Copy every tensor of ``params`` (a list, ids = positions) to the host pool."""
        for i, t in enumerate(params):
            self.offload_single(i, t)

    def prefetch_params(self, param_ids):
        """Start bringing the listed parameters back into the tensors they were offloaded from."""
        devs = self.__dict__.setdefault("_devs", {})
        for i in param_ids:
            self.fetch(f"param{int(i)}", devs.get(int(i)))
            self._count("pre", self.host[f"param{int(i)}"])

    def prefetch_all(self):
        self.prefetch_params(sorted(self.__dict__.setdefault("_devs", {})))

    def async_transfer(self, dst: torch.Tensor, src: torch.Tensor, param_id: int = -1):
        """One copy on the transfer stream (either direction: host <-> device); ``synchronize`` makes it visible."""
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                dst.copy_(src, non_blocking=True)
            self._pending = getattr(self, "_pending", 0) + 1
        else:
            dst.copy_(src)
        self._count("off" if not dst.is_cuda else "pre", src)

    def double_buffer_transfer(self, compute_buf: torch.Tensor, transfer_buf: torch.Tensor, src: torch.Tensor):
        """Fill ``transfer_buf`` from ``src`` on the transfer stream while the caller computes on ``compute_buf``; returns
        the pair swapped, ready for the next round (call ``synchronize`` before using the new compute buffer)."""
        self.async_transfer(transfer_buf, src)
        return transfer_buf, compute_buf

    def pin_memory(self, t: torch.Tensor) -> torch.Tensor:
        return t.pin_memory() if self.device.type == "cuda" and not t.is_pinned() else t

    @staticmethod
    def unpin_memory(t: torch.Tensor) -> torch.Tensor:
        return t.clone() if t.is_pinned() else t               # an unpinned copy; the pinned block returns to the allocator

    def _count(self, which: str, t: torch.Tensor):
        k = "_bytes_off" if which == "off" else "_bytes_pre"
        setattr(self, k, getattr(self, k, 0) + t.numel() * t.element_size())

    def bytes_offloaded(self) -> int: return getattr(self, "_bytes_off", 0)
    def bytes_prefetched(self) -> int: return getattr(self, "_bytes_pre", 0)

    def pending_transfers(self) -> int:
        if self.stream is not None and self.stream.query():
            self._pending = 0
        return getattr(self, "_pending", 0)

    def is_busy(self) -> bool: return self.pending_transfers() > 0

    def clear(self):
        self.synchronize()
        self.host, self.used, self._devs = {}, 0, {}

    def reset_stats(self):
        self._bytes_off = self._bytes_pre = 0


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

    # ---- per-parameter form and gradient sharding (reference: ZeROOffloadManager, include/quant/zero_offload.h)
    def offload_optimizer_state(self, m: torch.Tensor, v: torch.Tensor, param_idx: int):
        self.engine.offload(f"m{param_idx}", m)
        self.engine.offload(f"v{param_idx}", v)
        self.engine.synchronize()
        self._off = getattr(self, "_off", 0) + (m.numel() + v.numel()) * m.element_size()
        self.__dict__.setdefault("_idx", set()).add(param_idx)

    def reload_optimizer_state(self, m: torch.Tensor, v: torch.Tensor, param_idx: int):
        self.engine.fetch(f"m{param_idx}", m)
        self.engine.fetch(f"v{param_idx}", v)
        self.engine.synchronize()
        self.__dict__.setdefault("_idx", set()).discard(param_idx)

    @staticmethod
    def shard_gradient(grad: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
        """This rank's contiguous slice of a flattened gradient (zero-padded so that it divides evenly)."""
        flat = grad.reshape(-1)
        per = -(-flat.numel() // world_size)
        lo = rank * per
        out = torch.zeros(per, dtype=flat.dtype, device=flat.device)
        n = max(0, min(per, flat.numel() - lo))
        out[:n] = flat[lo:lo + n]
        return out

    @staticmethod
    def unshard_gradient(local_grad: torch.Tensor, rank: int, world_size: int, numel: Optional[int] = None, group=None) -> torch.Tensor:
        """All ranks' slices put back together (an all-gather when a process group is up; alone, the slice in its place)."""
        if world_size > 1 and dist.is_initialized():
            parts = [torch.empty_like(local_grad) for _ in range(world_size)]
            dist.all_gather(parts, local_grad.contiguous(), group=group)
            full = torch.cat(parts)
        else:
            full = torch.zeros(local_grad.numel() * world_size, dtype=local_grad.dtype, device=local_grad.device)
            full[rank * local_grad.numel():(rank + 1) * local_grad.numel()] = local_grad
        return full[:numel] if numel else full

    def bytes_offloaded(self) -> int: return getattr(self, "_off", 0) if getattr(self, "_idx", None) else (self.engine.used if self.on_host else 0)

    def bytes_on_device(self) -> int:
        o = self.opt
        tot = sum(t.numel() * t.element_size() for t in (getattr(o, "m", None), getattr(o, "v", None)) if t is not None)
        return 0 if self.on_host else tot

    def offload_ratio(self) -> float:
        off, dev = self.bytes_offloaded(), self.bytes_on_device()
        return off / max(1, off + dev)

    def reset_stats(self):
        self._off, self._idx = 0, set()


ZeROOptimizer = ShardOptimizer


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

    # ---- run-time accounting (reference: GradientCheckpointManager statics, include/quant/zero_offload.h:11-22)
    _depth, _saved, _recomputed, _bytes = 0, 0, 0, 0

    @classmethod
    def begin_checkpoint(cls, activation_bytes: int = 0):
        """A checkpointed region starts: its activations (``activation_bytes``) are dropped and recomputed in backward."""
        cls._depth += 1
        cls._saved += 1
        cls._bytes += int(activation_bytes)

    @classmethod
    def end_checkpoint(cls, recomputed: bool = True):
        if cls._depth > 0:
            cls._depth -= 1
            cls._recomputed += 1 if recomputed else 0

    @classmethod
    def in_checkpoint(cls) -> bool: return cls._depth > 0

    @classmethod
    def activations_saved(cls) -> int: return cls._saved

    @classmethod
    def activations_recomputed(cls) -> int: return cls._recomputed

    @classmethod
    def memory_saved_bytes(cls) -> int: return cls._bytes

    @classmethod
    def compute_overhead(cls) -> float:
        """Extra forward passes per region entered."""
        return cls._recomputed / cls._saved if cls._saved else 0.0

    @classmethod
    def reset_stats(cls):
        cls._depth = cls._saved = cls._recomputed = cls._bytes = 0

    def apply(self, model):
        """Sets the per-model switch when every layer is marked (the dense model recomputes all layers or none) and
        returns the per-layer marks for engines that checkpoint selectively."""
        if hasattr(model, "activation_checkpointing"):
            model.activation_checkpointing = all(self.checkpointed) and bool(self.checkpointed)
        return list(self.checkpointed)


@dataclass
class MemoryBudget:
    total_bytes: int = 0              # 0 = unlimited
    activation_bytes: int = 0
    param_bytes: int = 0
    grad_bytes: int = 0
    opt_state_bytes: int = 0

    def usage_ratio(self) -> float:
        return (self.activation_bytes + self.param_bytes + self.grad_bytes + self.opt_state_bytes) / max(1, self.total_bytes)


@dataclass
class RegionInfo:
    name: str
    forward_activations_bytes: int = 0
    recompute_cost_flops: int = 0
    is_checkpointed: bool = False
    mode: str = "NONE"                # NONE | FULL | PARTIAL | BALANCED


class ActivationCheckpoint:
    """Named regions of the forward pass with the bytes each keeps for backward, and a placement rule that marks regions
    for recomputation until the activations fit what the budget leaves after parameters, gradients and optimizer state
    (largest regions first).  Reference counterpart: ActivationCheckpoint, include/quant/zero_optimizer.h:356-437 and
    src/trainer/zero_optimizer_mem.cpp:580-705.

    A region is either declared (``begin_region(name, mode, activation_bytes=, recompute_flops=)`` ... ``end_region()``)
    or measured: ``with ac.region(name): y = block(x)`` counts the bytes autograd saves inside the block."""

    MODES = ("NONE", "FULL", "PARTIAL", "BALANCED")

    def __init__(self, budget: Optional[MemoryBudget] = None):
        self.budget = budget or MemoryBudget()
        self.reset()

    def reset(self):
        self._regions: List[RegionInfo] = []
        self._stack: List[RegionInfo] = []
        self.total_saved = self.total_recomputed = 0

    def set_budget(self, b: MemoryBudget): self.budget = b
    def mutable_budget(self) -> MemoryBudget: return self.budget
    def regions(self) -> List[RegionInfo]: return list(self._regions)
    def total_activations_saved(self) -> int: return self.total_saved
    def total_activations_recomputed(self) -> int: return self.total_recomputed

    def begin_region(self, name: str, mode: str = "FULL", activation_bytes: int = 0, recompute_flops: int = 0):
        mode = mode.upper()
        assert mode in self.MODES, mode
        self._stack.append(RegionInfo(name, int(activation_bytes), int(recompute_flops), mode != "NONE", mode))

    def end_region(self):
        if not self._stack:
            return
        r = self._stack.pop()
        r.forward_activations_bytes = max(r.forward_activations_bytes, 1024)
        r.recompute_cost_flops = max(r.recompute_cost_flops, 1)
        self._regions.append(r)
        if r.is_checkpointed:
            self.total_saved += r.forward_activations_bytes
            self.total_recomputed += r.recompute_cost_flops

    def in_checkpoint_region(self) -> bool:
        return bool(self._stack) and self._stack[-1].is_checkpointed

    def region(self, name: str, mode: str = "NONE", recompute_flops: int = 0):
        """Context manager: the region's activation bytes are what autograd saves for backward inside it (each distinct
        storage counted once; parameters and views of parameters are not activations)."""
        ac = self

        class _Region:
            def __enter__(self_):
                ac.begin_region(name, mode, 0, recompute_flops)
                info, seen = ac._stack[-1], set()

                def pack(t):
                    key = t.untyped_storage().data_ptr() if t.numel() else None
                    is_param = isinstance(t, torch.nn.Parameter) or isinstance(getattr(t, "_base", None), torch.nn.Parameter)
                    if key is not None and key not in seen and not is_param:
                        seen.add(key)
                        info.forward_activations_bytes += t.numel() * t.element_size()
                    return t
                self_.hooks = torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t)
                self_.hooks.__enter__()
                return info

            def __exit__(self_, *exc):
                self_.hooks.__exit__(*exc)
                ac.end_region()
                return False
        return _Region()

    @staticmethod
    def estimate_layer_activations(batch: int, seq: int, hidden: int, ffn_hidden: int = 0, bytes_per_value: int = 2) -> int:
        """Bytes one transformer block keeps for backward when nothing is recomputed: normed inputs, q / k / v and the
        attention output, the two GLU halves and their product, the two residual streams."""
        ffn_hidden = ffn_hidden or 4 * hidden
        return batch * seq * (8 * hidden + 3 * ffn_hidden) * bytes_per_value

    def auto_place_checkpoints(self) -> List[str]:
        """Mark regions, largest first, until the unmarked ones fit the budget; returns the newly marked names."""
        b = self.budget
        if not self._regions or b.total_bytes <= 0:
            return []
        target = b.total_bytes - b.param_bytes - b.grad_bytes - b.opt_state_bytes
        if target <= 0:
            target = b.total_bytes // 4
        held = sum(r.forward_activations_bytes for r in self._regions if not r.is_checkpointed)
        marked = []
        for r in sorted(self._regions, key=lambda r: -r.forward_activations_bytes):
            if held <= target:
                break
            if r.is_checkpointed:
                continue
            r.is_checkpointed, r.mode = True, "BALANCED"
            held -= r.forward_activations_bytes
            self.total_saved += r.forward_activations_bytes
            self.total_recomputed += r.recompute_cost_flops
            marked.append(r.name)
        b.activation_bytes = held
        return marked

    def estimated_savings(self, region: RegionInfo) -> int:
        return region.forward_activations_bytes if region.is_checkpointed else 0

    def estimated_savings_all(self) -> int:
        return sum(self.estimated_savings(r) for r in self._regions)

    def compute_overhead(self) -> float:
        """Recomputed FLOPs per byte saved (the reference's figure of merit)."""
        return self.total_recomputed / self.total_saved if self.total_saved > 0 else 0.0
