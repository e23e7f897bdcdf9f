"""Tensor-parallel serving: every rank runs the same continuous-batching scheduler on the same requests and holds
1 / W of every layer (its query / kv heads, its slice of the FFN, its pages of the KV cache for those heads).  The two
row-parallel products of a block (attention output, FFN down) produce partial sums that are added across ranks over
NVLink peer memory: decode-sized messages by the flag-in-data all-reduce (every rank pushes its rows, tagged with a
sequence number, into the peers' receive areas and sums what arrives - no barrier - with the residual stream added in
the same kernel), prefill-sized ones by the two-shot kernel on a staging buffer; on CPU or without a symmetric heap the
sum goes through torch.distributed.  The all-reduce gives every rank bit-identical
activations, so sampling with the shared seed picks the same token everywhere and the schedulers stay in step without
exchanging anything else.

Reference counterparts: TensorParallelManager::parallelize_model / row_parallel_linear + allreduce_tensor
(src/trainer/tensor_parallelism.cpp:334-451) applied to the inference path; the reference has no multi-process
serving engine."""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.distributed as dist

from ..models.dense import DenseModel
from ..ops import functional as F
from .engine import EngineConfig, InferenceEngine


def shard_dense_for_tp(model: DenseModel, rank: int, world: int) -> DenseModel:
    """A DenseModel holding this rank's heads and FFN slice of ``model`` (embedding, norms and LM head replicated)."""
    cfg = model.cfg
    if cfg.num_heads % world or cfg.num_kv_heads % world or cfg.ffn_hidden_size % world:
        raise ValueError("heads, kv heads and FFN width must divide by the tensor-parallel degree")
    D = cfg.head_dim
    lc = dataclasses.replace(cfg, num_heads=cfg.num_heads // world, num_kv_heads=cfg.num_kv_heads // world, head_dim=D,
                             ffn_hidden_size=cfg.ffn_hidden_size // world)
    dev, dt = model.tok_embeddings.device, model.tok_embeddings.dtype
    local = DenseModel(lc, device=dev, dtype=dt, seed=None)
    nq, nkv = cfg.num_heads * D, cfg.num_kv_heads * D
    hq, hkv, Fh, Fl = lc.num_heads * D, lc.num_kv_heads * D, cfg.ffn_hidden_size, lc.ffn_hidden_size
    cut = lambda t, n: t[rank * n:(rank + 1) * n]
    with torch.no_grad():
        local.tok_embeddings.data.copy_(model.tok_embeddings.data)
        local.norm.data.copy_(model.norm.data)
        if local.lm_head is not local.tok_embeddings:
            local.lm_head.data.copy_(model.lm_head.data)
        if model.pos_embeddings is not None:
            local.pos_embeddings.data.copy_(model.pos_embeddings.data)
        for src, dst in zip(model.layers, local.layers):
            q, k, v = src.qkv.data[:nq], src.qkv.data[nq:nq + nkv], src.qkv.data[nq + nkv:]
            dst.qkv.data.copy_(torch.cat([cut(q, hq), cut(k, hkv), cut(v, hkv)], 0))
            dst.o.data.copy_(src.o.data[:, rank * hq:(rank + 1) * hq])
            if cfg.gated:
                dst.gate_up.data.copy_(torch.cat([cut(src.gate_up.data[:Fh], Fl), cut(src.gate_up.data[Fh:], Fl)], 0))
            else:
                dst.gate_up.data.copy_(cut(src.gate_up.data, Fl))
            dst.down.data.copy_(src.down.data[:, rank * Fl:(rank + 1) * Fl])
            dst.attention_norm.data.copy_(src.attention_norm.data)
            dst.ffn_norm.data.copy_(src.ffn_norm.data)
            for name in ("qkv_bias", "gate_up_bias"):
                if getattr(src, name, None) is not None:
                    raise ValueError("tensor-parallel serving covers bias-free projections")
    return local


class TPInferenceEngine(InferenceEngine):
    def __init__(self, model: DenseModel, tokenizer=None, cfg: Optional[EngineConfig] = None, rank: int = 0, world: int = 1,
                 symm=None, group=None):
        cfg = cfg or EngineConfig()
        # Decode graphs are safe across ranks: every rank captures and replays the same sequence of kernels, and the
        # all-reduce kernels keep their epoch and ticket in device memory.  The one piece of host-side state a graph bakes
        # in - which of the two staging buffers each collective uses - is kept consistent by the capture / replay hooks.
        self.tp_rank, self.tp_world, self.tp_group = rank, world, group
        local = shard_dense_for_tp(model, rank, world) if world > 1 else model
        super().__init__(local, tokenizer, cfg)
        self.coll = None
        if world > 1 and symm is not None and self.device.type == "cuda":
            from ..parallel.collectives import SymmCollectives
            self.coll = SymmCollectives(symm, capacity_bytes=max(8 << 20, 2 * cfg.max_prefill_tokens * model.cfg.hidden_size * 2))
        self.allreduce_calls = 0

    def _all_reduce(self, y: torch.Tensor) -> torch.Tensor:
        self.allreduce_calls += 1
        if self.coll is not None and y.numel() * y.element_size() <= self.coll.capacity:
            return self.coll.all_reduce(y.contiguous())
        dist.all_reduce(y, group=self.tp_group)
        return y

    def _graph_capture_begin(self):
        return self.coll.capture_begin() if self.coll is not None else None

    def _graph_capture_end(self, token):
        if self.coll is not None:
            self.coll.capture_end(token)

    def _graph_before_replay(self, token):
        if self.coll is not None:
            self.coll.before_replay(token)

    def _lin(self, x, li, name, w, bias=None, residual=None):
        if self.tp_world == 1 or name not in ("o", "down"):
            return super()._lin(x, li, name, w, bias, residual)
        M, N = x.shape[0], w.shape[0]
        if self.coll is not None and x.is_cuda and M * N * x.element_size() <= self.coll.one_shot_max_bytes \
                and (M * N * x.element_size()) % 16 == 0:
            # decode-sized: this rank's partial product stays in local memory; the flag-in-data all-reduce pushes it to
            # the peers, sums what arrives and adds the residual stream in the same kernel
            y = super()._lin(x, li, name, w, None, None)
            self.allreduce_calls += 1
            fuse = bias is None and residual is not None and residual.is_contiguous() and residual.data_ptr() % 16 == 0
            y = self.coll.all_reduce_ll(y.contiguous(), residual=residual if fuse else None, out=y if y.is_contiguous() else None)
            if fuse:
                return y
            if bias is not None:
                y = y + bias
            return y if residual is None else y + residual
        st = self.coll.stage_view(x.dtype, M * N) if (self.coll is not None and x.is_cuda) else None
        if st is not None:
            # the partial product lands in the staging buffer of the all-reduce, the residual stream is added inside the
            # reduction and the reduced rows are used where the kernel leaves them: no copy in, no copy out, no add
            pw = self.packed.get(f"layers.{li}.{name}")
            if pw is None:
                F.gemm(x, w.data, out=st.view(M, N))
            else:
                self._wq.gemm_wq(x, pw, None, out=st.view(M, N))
            self.allreduce_calls += 1
            fuse = bias is None and residual is not None
            y = self.coll.all_reduce_staged(M * N, x.dtype, residual=residual if fuse else None).view(M, N)
            if fuse:
                return y
        else:
            y = self._all_reduce(super()._lin(x, li, name, w, None, None))   # this rank's partial sum, then the sum
        if bias is not None:
            y = y + bias
        return y if residual is None else y + residual
