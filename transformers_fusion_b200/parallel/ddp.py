"""Data-parallel wrappers over the flat gradient buffer.

``DistributedDataParallel`` reduces gradients in buckets of ``bucket_size`` elements (default 1 Mi = 4 MiB of fp32)
with optional compression, in SYNC mode (call ``sync_gradients`` after backward) or ASYNC mode (buckets are launched
as non-blocking collectives and joined by ``finish``).  Compression:
  TOP_K_SPARSE  each rank keeps its ``sparse_ratio`` largest-magnitude entries per bucket (the rest stays in a local
                residual that is added back next step), exchanges (index, value) pairs with an all-gather and
                scatter-adds them;
  INT8          per-bucket absmax int8 quantisation, all-gather of codes + scales, dequantise and sum (the reference
                calls this "FP8").
The production path on GPUs is the fused ZeRO step (parallel/zero_fused.py); this class is the general, any-backend
wrapper with the reference's API.  ``DDPWrapper`` is the minimal per-parameter all-reduce.

Reference counterparts: include/quant/ddp.h:24-93, src/trainer/ddp.cpp (allreduce_bucket :113-173, compression
:175-249, global_grad_norm / clip :280-312, broadcast_model :324), DDPWrapper src/trainer/distributed.cpp:129-164."""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

from .collectives import DistributedContext


class GradCompression:
    NONE, TOP_K_SPARSE, INT8 = "none", "top_k_sparse", "int8"


class DDPMode:
    SYNC, ASYNC = "sync", "async"


class DistributedDataParallel:
    def __init__(self, model, ctx: Optional[DistributedContext] = None, mode: str = DDPMode.SYNC):
        self.model = model
        self.ctx = ctx or DistributedContext.init()
        self.mode = mode
        self.flat = model.flatten()
        self.bucket_size = 1 << 20
        self.compression, self.sparse_ratio = GradCompression.NONE, 0.01
        self.residual = None
        self.accum_steps, self._micro = 1, 0
        self._pending: List = []
        self.bytes_sent = 0

    # ---- configuration (reference names)
    def set_bucket_size(self, numel: int):
        self.bucket_size = max(1, int(numel))

    def set_grad_compression(self, kind: str, sparse_ratio: float = 0.01):
        self.compression, self.sparse_ratio = kind, sparse_ratio
        self.residual = torch.zeros_like(self.flat.grads) if kind == GradCompression.TOP_K_SPARSE else None

    def set_grad_accumulation_steps(self, n: int):
        self.accum_steps = max(1, int(n))

    def grad_accumulation_steps(self) -> int: return self.accum_steps
    def grad_accum_count(self) -> int: return self._micro % self.accum_steps
    def reset_grad_accum_count(self): self._micro = 0
    def context(self) -> DistributedContext: return self.ctx
    def world_size(self) -> int: return self.ctx.world_size
    def rank(self) -> int: return self.ctx.rank

    # ---- forward / gradient path
    def forward(self, ids):
        return self.model.forward(ids)

    def forward_backward(self, ids, labels):
        """Fused step of the wrapped model; gradients are reduced when the accumulation window closes."""
        loss = self.model.forward_backward(ids, labels)
        self._micro += 1
        if self._micro % self.accum_steps == 0:
            if self.accum_steps > 1:
                self.flat.grads.div_(self.accum_steps)
            self.sync_gradients()
        return loss

    def _buckets(self):
        g = self.flat.grads
        for o in range(0, g.numel(), self.bucket_size):
            yield o, g[o:o + self.bucket_size]

    def allreduce_bucket(self, bucket: torch.Tensor, offset: int = 0):
        """Average one bucket over the ranks in place (with the configured compression)."""
        W = self.ctx.world_size
        if W == 1 or not self.ctx.is_distributed:
            return None
        if self.compression == GradCompression.NONE:
            self.bytes_sent += bucket.numel() * 4
            if self.mode == DDPMode.ASYNC:
                h = dist.all_reduce(bucket, group=self.ctx.group, async_op=True)
                self._pending.append((h, bucket))
                return h
            dist.all_reduce(bucket, group=self.ctx.group)
            bucket.div_(W)
            return None
        if self.compression == GradCompression.TOP_K_SPARSE:
            res = self.residual[offset:offset + bucket.numel()]
            full = bucket + res
            k = max(1, int(math.ceil(self.sparse_ratio * full.numel())))
            idx = full.abs().topk(k).indices
            val = full[idx]
            res.copy_(full)
            res[idx] = 0                       # what was not sent stays behind for the next step
            all_idx = self.ctx.all_gather(idx.to(torch.int64))
            all_val = self.ctx.all_gather(val)
            bucket.zero_()
            bucket.index_add_(0, all_idx, all_val)
            bucket.div_(W)
            self.bytes_sent += k * 12
            return None
        if self.compression == GradCompression.INT8:
            amax = bucket.abs().max().clamp(min=1e-30)
            scale = (amax / 127.0).reshape(1)
            q = torch.clamp(torch.round(bucket / scale), -127, 127).to(torch.int8)
            all_q = self.ctx.all_gather(q)
            all_s = self.ctx.all_gather(scale)
            deq = all_q.view(W, -1).float() * all_s.view(W, 1)
            bucket.copy_(deq.sum(0) / W)
            self.bytes_sent += bucket.numel() + 4
            return None
        raise ValueError(self.compression)

    def sync_gradients(self):
        for o, b in self._buckets():
            self.allreduce_bucket(b, o)
        if self.mode == DDPMode.SYNC:
            self.finish()

    def finish(self):
        """Join the outstanding non-blocking bucket reductions (ASYNC mode)."""
        W = self.ctx.world_size
        for h, b in self._pending:
            h.wait()
            b.div_(W)
        self._pending = []

    def sync_buffers(self, tensors):
        for t in tensors:
            self.ctx.broadcast(t, 0)

    def global_grad_norm(self) -> float:
        """Every rank holds the same (reduced) gradients after sync, so the local norm is the global one."""
        return float(self.flat.grads.norm())

    def clip_gradients(self, max_norm: float) -> float:
        n = self.global_grad_norm()
        if max_norm > 0 and n > max_norm:
            self.flat.grads.mul_(max_norm / (n + 1e-6))
        return n

    def broadcast_model(self, src: int = 0):
        self.ctx.broadcast(self.flat.params, src)

    def average_model(self, weight: float = 1.0):
        """Parameter averaging across ranks (local-SGD style): p = (1-w) p + w mean(p)."""
        mean = self.ctx.all_reduce(self.flat.params.float().clone(), "avg")
        self.flat.params.copy_(((1 - weight) * self.flat.params.float() + weight * mean).to(self.flat.params.dtype))

    def zero_grad(self):
        self.flat.zero_grad()

    def inject_gradient_noise(self, step: int, eta: float = 0.01, gamma: float = 0.55, seed: int = 0):
        std = math.sqrt(eta / (1 + step) ** gamma)
        g = torch.Generator(device=self.flat.grads.device).manual_seed(seed * 1000003 + step)   # same noise on every rank
        self.flat.grads.add_(torch.randn(self.flat.grads.shape, generator=g, device=self.flat.grads.device) * std)


class DDPWrapper:
    """Per-parameter gradient all-reduce (the reference's first DDP)."""

    def __init__(self, model, ctx: Optional[DistributedContext] = None):
        self.model, self.ctx = model, ctx or DistributedContext.init()
        model.flatten()

    def sync_gradients(self):
        for p in self.model.parameters():
            self.ctx.all_reduce(p.main_grad, "avg")

    def context(self) -> DistributedContext: return self.ctx


class TensorParallelWrapper:
    """The reference's first tensor-parallel wrapper (include/quant/distributed.h: TensorParallelWrapper): a model whose
    linear layers are split over the ranks of ``ctx``.  The work is done by ``parallel.tp_model.TPDenseModel``; this class
    keeps the small surface: ``forward(ids)``, ``context()``, ``split_linear(weight, dim)``."""

    def __init__(self, model, ctx: Optional[DistributedContext] = None):
        self.ctx = ctx or DistributedContext.init()
        self.ctx.mode = "TENSOR_PARALLEL"
        self.full = model
        self._tp = None

    def context(self) -> DistributedContext: return self.ctx

    def split_linear(self, weight: torch.Tensor, dim: int = 0) -> torch.Tensor:
        """This rank's slice of a weight: dim 0 = output rows (column-parallel layer), dim 1 = input columns (row-parallel)."""
        n = weight.shape[dim] // self.ctx.world_size
        return weight.narrow(dim, self.ctx.rank * n, n).contiguous()

    def forward(self, ids):
        if self.ctx.world_size == 1:
            return self.full.forward(ids)
        from .tp_model import TPDenseModel, TPGroup, _HeadFn, _RMSNormFn
        if self._tp is None:
            self._tp = TPDenseModel(self.full, TPGroup(self.ctx.rank, self.ctx.world_size, self.ctx.group))
        tp = self._tp
        B, S = ids.shape
        with torch.no_grad():
            h = torch.nn.functional.embedding(tp._shard_rows(ids.reshape(-1)), tp.tok_embeddings)
            rope = self.full.rope(ids.device)
            for blk in tp.layers:
                h = blk(h, B, S, rope)
            logits = _HeadFn.apply(_RMSNormFn.apply(h, tp.norm, tp.cfg.norm_eps), tp.lm_head)
            return tp.tp.all_gather_rows(logits.contiguous()).view(B, S, -1)


class PipelineParallelWrapper:
    """The reference's first pipeline wrapper (include/quant/distributed.h: PipelineParallelWrapper): rank r runs the
    r-th contiguous range of layers; ``forward(ids)`` returns the logits on the last rank (None elsewhere)."""

    def __init__(self, model, ctx: Optional[DistributedContext] = None):
        from .pp import PipelineParallel
        self.ctx = ctx or DistributedContext.init()
        self.ctx.mode = "PIPELINE_PARALLEL"
        self.pp = PipelineParallel(model, self.ctx.world_size, self.ctx.rank, self.ctx, num_microbatches=1)

    def context(self) -> DistributedContext: return self.ctx

    def forward(self, ids):
        return self.pp.forward(ids)
