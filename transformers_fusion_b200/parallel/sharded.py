"""ZeRO-3 / FSDP composed with tensor + sequence parallelism: the training engine for models that do not fit one GPU.

Mesh: ``world = dp x tp`` with tp fastest.  Every weight matrix is first cut Megatron-style over the tp ranks (q / k / v /
gate / up by output rows, o / down by input columns, embedding and LM head by vocabulary rows), and the tp-local piece is
then sharded by rows (128-row blocks) over the dp ranks, which also own the matching fp32 master weights and Adam moments.

One step, per rank:

* forward / backward are written by hand over the sm_100a kernels (no autograd graph).  Between the tensor-parallel
  regions the token stream is a row shard [T / tp, H] (sequence parallelism); the two collectives of a tensor-parallel
  product ride inside its GEMM launch (all-gather -> GEMM, GEMM -> reduce-scatter; ``tfb_gemm_bf16_tp`` bits 1 / 2).
* the ZeRO-3 parameter gather fills one of two per-unit gather buffers (a unit's buffer is recycled two units later, so
  only two units' worth of full weights exist at any time).  Default (``gather="prefetch"``): one all-gather kernel per
  unit on a side stream, one unit ahead of the compute, whose small CTAs read every dp peer's row shards over NVLink
  beside the running GEMMs.  ``gather="fused"``: the first GEMM that consumes a weight pulls the peers' shards itself
  (bit 4 of the GEMM mode word) while the tiles of the local shard already multiply.
* the token embedding is read straight from the shards (each row from the dp rank that owns it), the LM head and the
  cross entropy are vocabulary-parallel (the ranks exchange [T, 4] row statistics, never logits).
* as soon as a unit's backward is complete its gradients are reduce-scattered over the dp group by one kernel on a side
  stream with a bounded grid (peer loads, 1/dp scale, squared-norm partial), overlapping the backward of the next unit.
* after the last unit: global gradient norm (one scalar all-reduce), clip, one fused AdamW over this rank's flat shard
  state, refreshed bf16 shards in place.  No parameter all-gather follows: the next step gathers what it needs.

``comm="nccl"`` (and every CPU / gloo run) replaces each fused piece by the library collective plus the plain kernel and is
the baseline the fused path is compared against.

Reference counterparts: FullyShardedDataParallel forward / backward / reduce_scatter_grads / optimizer_step
(src/trainer/fsdp.cpp:188-213, 275-308, 508-543), ColumnParallelLinear / RowParallelLinear / SequenceParallel
(src/trainer/tensor_parallelism.cpp:53-142, 334-451); the reference keeps each of them behind a private context and
never composes them (include/quant/fsdp.h:92, include/quant/tensor_parallelism.h:81)."""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib, functional as F

BLK = 128   # rows per shard block (one GEMM tile edge)


@dataclass
class Mesh:
    """Coordinates and process groups of this rank (``None`` groups mean a group of one)."""
    dp_rank: int = 0
    dp: int = 1
    tp_rank: int = 0
    tp: int = 1
    dp_group: object = None
    tp_group: object = None
    world_group: object = None     # dp x tp ranks that train one model replica set (default group when None)

    @property
    def world(self):
        return self.dp * self.tp


class ShardedParam:
    """One tp-local weight matrix [rows, cols], row-sharded over the dp ranks."""

    def __init__(self, name, unit, rows, cols, dp):
        self.name, self.unit, self.rows, self.cols = name, unit, rows, cols
        gran = BLK * dp
        self.rows_p = (rows + gran - 1) // gran * gran
        self.per = self.rows_p // dp
        self.shard_off = self.full_off = self.slot_off = 0
        self.src = None        # device int64[dp]: base address of every dp rank's shard (fused path)
        self.ready = None      # device int32[rows_p / 128]
        self.epoch = 0
        self.gathered = False


class _AgDesc(C.Structure):
    # seg: triples (device array of the W shard addresses, local destination, bytes per shard)
    _fields_ = [("rank", C.c_int), ("world", C.c_int), ("nseg", C.c_int), ("pad", C.c_int), ("seg", C.c_longlong * 24)]


class _RsDesc(C.Structure):
    _fields_ = [("flag_ptrs", C.c_void_p), ("epoch", C.c_void_p), ("rank", C.c_int), ("world", C.c_int), ("status", C.c_void_p),
                ("grad_ptrs", C.c_void_p), ("gshard", C.c_void_p), ("sumsq", C.c_void_p), ("ticket", C.c_void_p),
                ("scale", C.c_float), ("nseg", C.c_int), ("seg", C.c_longlong * 24)]


def _tp_slices(cfg, tp_rank, tp):
    """Row / column index ranges of this tp rank's piece of every block weight."""
    D = cfg.head_dim
    hq, hkv, Fl = cfg.num_heads // tp, cfg.num_kv_heads // tp, cfg.ffn_hidden_size // tp
    return hq, hkv, Fl, D


class ShardedEngine:
    """Training engine over a (dp x tp) mesh; see the module docstring.  Build with ``from_dense`` (a full model that every
    rank constructed identically; used by tests and small jobs) or ``from_config`` (weights drawn tensor by tensor on the
    device from per-tensor seeds, so that no rank ever holds the whole model)."""

    def __init__(self, cfg, mesh: Mesh, weight_of: Callable[[str], torch.Tensor], device, dtype=torch.bfloat16, comm="fused",
                 lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0, max_tokens=0, dp_heap=None,
                 tp_heap=None, rs_ctas=0, copy_ctas=12, loss_chunk_tokens=4096, gather="auto", ag_ctas=0):
        assert cfg.norm_type == "rmsnorm" and not cfg.use_parallel_residual and not cfg.attention_bias, \
            "the sharded engine covers the sequential RMSNorm block without biases"
        assert cfg.num_heads % mesh.tp == 0 and cfg.num_kv_heads % mesh.tp == 0 and cfg.ffn_hidden_size % mesh.tp == 0
        assert cfg.vocab_size % mesh.tp == 0 and cfg.position_type == "rope"
        self.cfg, self.mesh, self.device, self.dtype = cfg, mesh, torch.device(device), dtype
        self.fused = comm == "fused" and self.device.type == "cuda"
        self.comm = comm
        self.lr, self.betas, self.eps, self.weight_decay, self.max_grad_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.rs_ctas, self.copy_ctas, self.loss_chunk_tokens = rs_ctas, copy_ctas, loss_chunk_tokens
        # ZeRO-3 weight gather on the fused path: "prefetch" = one kernel per unit on a side stream, one unit ahead of the
        # compute (peer loads by small CTAs that sit beside the GEMM's); "fused" = the copy CTAs of the GEMM that first
        # uses a weight pull it (no separate launch, but a GEMM whose every tile needs the whole weight - the input
        # gradient - then runs at the speed of its copy CTAs)
        # "auto" is the prefetch kernel: measured on the 8-layer 8B shape with a group of two, 84.9 ms per step against 90.0 ms
        # with the gather inside the GEMM (whose wide products cannot use the grouped tile order, and whose input-gradient
        # products wait for the whole weight); for larger groups most of every weight is remote and the copy CTAs of the
        # GEMM fall further behind
        assert gather in ("auto", "prefetch", "fused")
        if gather == "auto":
            gather = "prefetch"
        self.gather_mode, self.ag_ctas = gather, ag_ctas
        self.step_count = 0
        self.dp_heap, self.tp_heap = dp_heap, tp_heap
        if self.fused and mesh.dp > 1:
            assert dp_heap is not None, "the fused path needs a symmetric heap over the data-parallel group"
        if self.fused and mesh.tp > 1:
            assert tp_heap is not None, "the fused path needs a symmetric heap over the tensor-parallel group"
        self._build(weight_of)
        self._tp_ctx = None
        self._tp_coll = None
        self._max_tokens = max_tokens
        self._rope = None
        self.gathers = 0
        self.activation_checkpointing = False      # keep only each block's input and rebuild the rest in backward
        self.last_grad_norm = torch.zeros(1, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------------------------------ construction
    @classmethod
    def from_dense(cls, model, mesh: Mesh, **kw):
        cfg = model.cfg
        named = dict(model.named_parameters())

        def weight_of(name):
            return named[name].data
        dev = kw.pop("device", model.tok_embeddings.device)
        return cls(cfg, mesh, weight_of, dev, dtype=model.tok_embeddings.dtype, **kw)

    @classmethod
    def from_config(cls, cfg, mesh: Mesh, device, seed=0, dtype=torch.bfloat16, **kw):
        """Random N(0, init_std) matrices drawn on the device, one tensor at a time from a seed derived from its name
        (every rank draws the same full tensor and keeps its own piece), ones for the norm weights."""
        import zlib
        dev = torch.device(device)
        H, V, D = cfg.hidden_size, cfg.vocab_size, cfg.head_dim
        shapes = {"tok_embeddings": (V, H), "lm_head": (V, H), "norm": (H,)}
        for i in range(cfg.num_layers):
            shapes[f"layers.{i}.qkv"] = ((cfg.num_heads + 2 * cfg.num_kv_heads) * D, H)
            shapes[f"layers.{i}.o"] = (H, cfg.num_heads * D)
            shapes[f"layers.{i}.gate_up"] = ((2 if cfg.gated else 1) * cfg.ffn_hidden_size, H)
            shapes[f"layers.{i}.down"] = (H, cfg.ffn_hidden_size)
            shapes[f"layers.{i}.attention_norm"] = (H,)
            shapes[f"layers.{i}.ffn_norm"] = (H,)

        def weight_of(name):
            shp = shapes[name]
            if len(shp) == 1:
                return torch.ones(shp, dtype=dtype, device=dev)
            g = torch.Generator(device=dev).manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
            return (torch.randn(shp, generator=g, device=dev, dtype=torch.float32) * cfg.init_std).to(dtype)
        return cls(cfg, mesh, weight_of, dev, dtype=dtype, **kw)

    def _tp_piece(self, name, w):
        """This tp rank's piece of the full tensor ``w`` (rows for column-parallel weights, columns for row-parallel)."""
        cfg, m = self.cfg, self.mesh
        r, W = m.tp_rank, m.tp
        hq, hkv, Fl, D = _tp_slices(cfg, r, W)
        base = name.split(".")[-1]
        if base in ("tok_embeddings", "lm_head"):
            n = cfg.vocab_size // W
            return w[r * n:(r + 1) * n]
        if base == "qkv":
            nq, nkv = cfg.num_heads * D, cfg.num_kv_heads * D
            q, k, v = w[:nq], w[nq:nq + nkv], w[nq + nkv:]
            return torch.cat([q[r * hq * D:(r + 1) * hq * D], k[r * hkv * D:(r + 1) * hkv * D], v[r * hkv * D:(r + 1) * hkv * D]], 0)
        if base == "o":
            return w[:, r * hq * D:(r + 1) * hq * D]
        if base == "gate_up":
            Fh = cfg.ffn_hidden_size
            if cfg.gated:
                return torch.cat([w[:Fh][r * Fl:(r + 1) * Fl], w[Fh:][r * Fl:(r + 1) * Fl]], 0)
            return w[r * Fl:(r + 1) * Fl]
        if base == "down":
            return w[:, r * Fl:(r + 1) * Fl]
        raise KeyError(name)

    def _build(self, weight_of):
        cfg, m, dev, dt = self.cfg, self.mesh, self.device, self.dtype
        L = cfg.num_layers
        self.tied = bool(cfg.tie_embeddings)
        names = [("tok_embeddings", 0)]
        for i in range(L):
            names += [(f"layers.{i}.{w}", 1 + i) for w in ("qkv", "o", "gate_up", "down")]
        if not self.tied:
            names.append(("lm_head", L + 1))
        self.num_units = L + 2
        # ---- geometry
        self.params: Dict[str, ShardedParam] = {}
        self.units: List[List[ShardedParam]] = [[] for _ in range(self.num_units)]
        shard_off = full_off = 0
        pieces = {}
        for name, unit in names:
            piece = self._tp_piece(name, weight_of(name))
            p = ShardedParam(name, unit, piece.shape[0], piece.shape[1], m.dp)
            p.shard_off, p.full_off = shard_off, full_off
            p.slot_off = sum(q.rows_p * q.cols for q in self.units[unit])
            shard_off += p.per * p.cols
            full_off += p.rows_p * p.cols
            self.params[name] = p
            self.units[unit].append(p)
            # keep only this rank's shard of the piece (padded rows are zero)
            lo = m.dp_rank * p.per
            sh = torch.zeros((p.per, p.cols), dtype=dt, device=dev)
            hi = min(piece.shape[0], lo + p.per)
            if hi > lo:
                sh[: hi - lo].copy_(piece[lo:hi])
            pieces[name] = sh
            del piece
        self.shard_numel, self.full_numel = shard_off, full_off
        slot_numel = max(sum(q.rows_p * q.cols for q in u) for u in self.units if u)
        # ---- storage
        heap = self.dp_heap if (self.fused and m.dp > 1) else None
        if heap is not None:
            self._sym_shard = heap.alloc(self.shard_numel, dt)
            self._sym_grad = heap.alloc(self.full_numel, torch.float32)
            self.shard_lp = self._sym_shard.view(dt, self.shard_numel)
            self.full_grad = self._sym_grad.view(torch.float32, self.full_numel)
        else:
            self.shard_lp = torch.zeros(self.shard_numel, dtype=dt, device=dev)
            self.full_grad = torch.zeros(self.full_numel, dtype=torch.float32, device=dev)
        for name, sh in pieces.items():
            p = self.params[name]
            self.shard_lp[p.shard_off:p.shard_off + p.per * p.cols].copy_(sh.reshape(-1))
        del pieces
        self.master = self.shard_lp.float().clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.gshard = torch.zeros_like(self.master)
        self.slots = [torch.zeros(slot_numel, dtype=dt, device=dev) for _ in range(2)] if m.dp > 1 else None
        self.slot_owner = [None, None]
        # ---- small replicated parameters (norm weights): one flat vector, plain data parallelism over the whole mesh
        small_names = [f"layers.{i}.{w}" for i in range(L) for w in ("attention_norm", "ffn_norm")] + ["norm"]
        H = cfg.hidden_size
        self.small_lp = torch.zeros(len(small_names) * H, dtype=dt, device=dev)
        self.small_index = {n: k for k, n in enumerate(small_names)}
        for n, k in self.small_index.items():
            self.small_lp[k * H:(k + 1) * H].copy_(weight_of(n).reshape(-1))
        self.small_master = self.small_lp.float().clone()
        self.small_m = torch.zeros_like(self.small_master)
        self.small_v = torch.zeros_like(self.small_master)
        self.small_grad = torch.zeros_like(self.small_master)
        # ---- device-side bookkeeping
        f32 = dict(dtype=torch.float32, device=dev)
        self.sumsq = torch.zeros(1, **f32)
        self._sumsq_small = torch.zeros(1, **f32)
        self._clip = torch.ones(1, **f32)
        self._found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
        self.hyper = torch.zeros(4, **f32)
        if heap is not None:
            self._ticket = torch.zeros(4, dtype=torch.int32, device=dev)
            heap.on_reset(self._ticket.zero_)
            for p in self.params.values():
                addrs = [b + p.shard_off * self.shard_lp.element_size() for b in self._sym_shard.peer_ptrs]
                p.src = torch.tensor(addrs, dtype=torch.int64, device=dev)
                p.ready = torch.zeros(p.rows_p // BLK, dtype=torch.int32, device=dev)
            self._rs_desc = [self._make_rs_desc(u) for u in range(self.num_units)]
            self._ag_desc = [self._make_ag_desc(u) for u in range(self.num_units)]
            self._side = torch.cuda.Stream(device=dev, priority=-1)
            self._ag_stream = torch.cuda.Stream(device=dev, priority=-1)
            self._ev_main = torch.cuda.Event()
            self._ev_side = torch.cuda.Event()
            self._ev_main_ag = torch.cuda.Event()
            self._ag_done = [torch.cuda.Event(), torch.cuda.Event()]
            self._ag_pending = [False, False]
            lib = _lib.lib()
            lib.tfb_fsdp_reduce_scatter.argtypes = [C.POINTER(_RsDesc), C.c_int, C.c_void_p]
            lib.tfb_fsdp_reduce_scatter.restype = C.c_int
            lib.tfb_fsdp_all_gather.argtypes = [C.POINTER(_AgDesc), C.c_int, C.c_void_p]
            lib.tfb_fsdp_all_gather.restype = C.c_int
        self._pending = []

    def _make_ag_desc(self, unit):
        ps = self.units[unit]
        if not ps or self.slots is None:
            return None
        d = _AgDesc()
        d.rank, d.world, d.nseg = self.mesh.dp_rank, self.mesh.dp, len(ps)
        slot, esz = self.slots[unit % 2], self.shard_lp.element_size()
        for k, p in enumerate(ps):
            d.seg[3 * k] = p.src.data_ptr()
            d.seg[3 * k + 1] = slot.data_ptr() + p.slot_off * esz
            d.seg[3 * k + 2] = p.per * p.cols * esz
        return d

    def _make_rs_desc(self, unit):
        ps = self.units[unit]
        if not ps:
            return None
        heap, m = self.dp_heap, self.mesh
        d = _RsDesc()
        d.flag_ptrs, d.epoch = heap.flags.ptrs.data_ptr(), heap.epoch.data_ptr()
        d.rank, d.world = m.dp_rank, m.dp
        d.status = _lib.status_word(self.device).data_ptr()
        d.grad_ptrs = self._sym_grad.ptrs.data_ptr()
        d.gshard, d.sumsq, d.ticket = self.gshard.data_ptr(), self.sumsq.data_ptr(), self._ticket.data_ptr()
        d.scale = 1.0 / m.dp
        d.nseg = len(ps)
        for k, p in enumerate(ps):
            d.seg[3 * k], d.seg[3 * k + 1], d.seg[3 * k + 2] = p.full_off, p.shard_off, p.per * p.cols
        return d

    # ------------------------------------------------------------------------------------------ views
    def small(self, name):
        H, k = self.cfg.hidden_size, self.small_index[name]
        return self.small_lp[k * H:(k + 1) * H]

    def small_g(self, name):
        H, k = self.cfg.hidden_size, self.small_index[name]
        return self.small_grad[k * H:(k + 1) * H]

    def grad_view(self, p: ShardedParam):
        """fp32 gradient of the whole tp-local matrix [rows, cols] (this rank's contribution until the reduce-scatter)."""
        return self.full_grad[p.full_off:p.full_off + p.rows_p * p.cols].view(p.rows_p, p.cols)[: p.rows]

    def shard_view(self, p: ShardedParam):
        return self.shard_lp[p.shard_off:p.shard_off + p.per * p.cols].view(p.per, p.cols)

    # ------------------------------------------------------------------------------------------ parameter gather
    def _slot_view(self, p: ShardedParam):
        if self.mesh.dp == 1:
            return self.shard_view(p)                   # the shard is the whole matrix
        s = p.unit % 2
        if self.slot_owner[s] != p.unit:
            if self.slot_owner[s] is not None:
                for q in self.units[self.slot_owner[s]]:
                    q.gathered = False
            self.slot_owner[s] = p.unit
        return self.slots[s][p.slot_off:p.slot_off + p.rows_p * p.cols].view(p.rows_p, p.cols)

    def _gather_unit(self, unit):
        """Launch the all-gather of every weight of ``unit`` into its slot, on the gather stream.  The slot's previous
        contents are dead once everything enqueued on the main stream so far has run, so this is called where that
        holds: when the unit is first needed, or - as a prefetch - at the start of the unit before it."""
        ps = self.units[unit]
        s = unit % 2
        prev = self.slot_owner[s]
        if prev == unit and all(q.gathered for q in ps):
            return
        if prev is not None and prev != unit:
            for q in self.units[prev]:
                q.gathered = False
        self.slot_owner[s] = unit
        self._ev_main_ag.record()
        self._ag_stream.wait_event(self._ev_main_ag)
        _lib.check(_lib.lib().tfb_fsdp_all_gather(C.byref(self._ag_desc[unit]), self.ag_ctas, self._ag_stream.cuda_stream),
                   "fsdp_all_gather")
        self._ag_done[s].record(self._ag_stream)
        self._ag_pending[s] = True
        for q in ps:
            q.gathered = True
        self.gathers += len(ps)

    def _prefetch(self, unit, current):
        """Start gathering ``unit`` while ``current`` (whose kernels are about to be enqueued) computes; skipped when both
        live in the same slot."""
        if self.fused and self.gather_mode == "prefetch" and self.mesh.dp > 1 and 0 <= unit < self.num_units \
                and self.units[unit] and unit % 2 != current % 2:
            self._gather_unit(unit)

    def weight(self, p: ShardedParam):
        """(full [rows_p, cols] matrix view, WeightGather or None).  A non-None second value means the matrix is not in
        the gather buffer yet and the GEMM that receives it must pull it (fused path, gather="fused"); otherwise the
        gather has been enqueued ahead of whatever the caller enqueues next."""
        if self.fused and self.gather_mode == "prefetch" and self.mesh.dp > 1:
            if not (self.slot_owner[p.unit % 2] == p.unit and p.gathered):
                self._gather_unit(p.unit)
            s = p.unit % 2
            if self._ag_pending[s]:
                torch.cuda.current_stream().wait_event(self._ag_done[s])
                self._ag_pending[s] = False
            return self.slots[s][p.slot_off:p.slot_off + p.rows_p * p.cols].view(p.rows_p, p.cols), None
        buf = self._slot_view(p)
        if self.mesh.dp == 1 or p.gathered:
            return buf, None
        p.gathered = True
        self.gathers += 1
        if self.fused:
            from .tp import WeightGather
            p.epoch += 1
            # this rank's own rows by a plain device copy (HBM speed); the GEMM's copy CTAs then pull only the peers' rows
            lo = self.mesh.dp_rank * p.per
            buf[lo:lo + p.per].copy_(self.shard_view(p))
            return buf, WeightGather(buf, p.src, p.ready, p.epoch, self.mesh.dp_rank, self.mesh.dp, skip_local=True)
        sh = self.shard_view(p).contiguous()
        if buf.is_cuda:
            dist.all_gather_into_tensor(buf.view(-1), sh.view(-1), group=self.mesh.dp_group)
        else:
            parts = [torch.empty_like(sh) for _ in range(self.mesh.dp)]
            dist.all_gather(parts, sh, group=self.mesh.dp_group)
            buf.copy_(torch.cat(parts, 0))
        return buf, None

    def invalidate_gathers(self):
        for p in self.params.values():
            p.gathered = False
        self.slot_owner = [None, None]

    # ------------------------------------------------------------------------------------------ tensor-parallel plumbing
    def _tp(self, T):
        """Fused tensor-parallel context (gather / staging buffers for [T, H] activations), created at first use."""
        if self._tp_ctx is None:
            from .collectives import SymmCollectives
            from .tp import TpContext
            H = self.cfg.hidden_size
            T = max(T, self._max_tokens)
            self._tp_ctx = TpContext(self.tp_heap, self.mesh.tp_rank, self.mesh.tp, T, H, H, copy_ctas=self.copy_ctas)
            self._tp_coll = SymmCollectives(self.tp_heap, capacity_bytes=T * H * 2)
        return self._tp_ctx

    def tp_all_gather_rows(self, x):
        m = self.mesh
        if m.tp == 1:
            return x
        if self.fused:
            self._tp(x.shape[0] * m.tp)
            return self._tp_coll.all_gather(x.contiguous()).view(x.shape[0] * m.tp, *x.shape[1:])
        parts = [torch.empty_like(x) for _ in range(m.tp)]
        dist.all_gather(parts, x.contiguous(), group=m.tp_group)
        return torch.cat(parts, 0)

    def tp_reduce_scatter_rows(self, y):
        """Sum over the tp ranks of y [T, N]; this rank keeps rows [tp_rank * T / tp, ...)."""
        m = self.mesh
        if m.tp == 1:
            return y
        n = y.shape[0] // m.tp
        if self.fused:
            self._tp(y.shape[0])
            return self._tp_coll.reduce_scatter(y.contiguous()).view(n, *y.shape[1:])
        if y.is_cuda:
            out = torch.empty((n,) + tuple(y.shape[1:]), dtype=y.dtype, device=y.device)
            dist.reduce_scatter_tensor(out, y.contiguous(), group=m.tp_group)
            return out
        y = y.float().contiguous()                                # gloo has no reduce-scatter
        dist.all_reduce(y, group=m.tp_group)
        return y[m.tp_rank * n:(m.tp_rank + 1) * n].to(self.dtype).clone()

    # ---- the four products of a tensor-parallel linear layer -------------------------------------------------------------
    def col_fwd(self, x_shard, p: ShardedParam):
        """Column-parallel forward: y [T, rows] = all_gather_rows(x_shard) @ W^T.  Returns (y, gathered x)."""
        m = self.mesh
        w, wg = self.weight(p)
        if m.tp > 1 and self.fused:
            y, xg = self._tp(x_shard.shape[0] * m.tp).all_gather_gemm(x_shard.contiguous(), w, wg=wg, n=p.rows)
            return y, xg.clone()                                  # the gather buffer is reused by the next fused call
        xg = self.tp_all_gather_rows(x_shard)
        if wg is not None:
            from .tp import fused_gemm
            return fused_gemm(xg, w, n=p.rows, wg=wg, copy_ctas=self.copy_ctas), xg
        return F.gemm(xg, w[: p.rows]), xg

    def row_fwd(self, x, p: ShardedParam, residual_shard):
        """Row-parallel forward: y_shard [T / tp, rows] = reduce_scatter_rows(x @ W^T) + residual_shard."""
        m = self.mesh
        w, wg = self.weight(p)
        if m.tp > 1 and self.fused:
            return self._tp(x.shape[0]).gemm_reduce_scatter(x, w, residual_shard, wg=wg, n=p.rows)
        if m.tp == 1:
            if wg is not None:
                from .tp import fused_gemm
                return fused_gemm(x, w, n=p.rows, wg=wg, residual=residual_shard, copy_ctas=self.copy_ctas)
            return F.gemm(x, w[: p.rows], residual=residual_shard)
        y = self.tp_reduce_scatter_rows(F.gemm(x, w[: p.rows], out_dtype=torch.float32))
        return (y.float() + residual_shard.float()).to(x.dtype)

    def col_bwd(self, dy, xg, p: ShardedParam):
        """Backward of col_fwd: weight gradient dy^T xg into the full gradient, returns dx_shard [T / tp, cols]."""
        m = self.mesh
        F.gemm(dy, xg, a_mn=True, b_mn=True, out=self.grad_view(p), accumulate=True)
        w, wg = self.weight(p)
        if m.tp > 1 and self.fused:
            return self._tp(dy.shape[0]).gemm_reduce_scatter(dy, w, None, b_mn=True, wg=wg, n=p.cols, k=p.rows)
        if m.tp == 1:
            if wg is not None:
                from .tp import fused_gemm
                return fused_gemm(dy, w, b_mn=True, n=p.cols, k=p.rows, wg=wg, copy_ctas=self.copy_ctas)
            return F.gemm(dy, w[: p.rows], b_mn=True)
        return self.tp_reduce_scatter_rows(F.gemm(dy, w[: p.rows], b_mn=True, out_dtype=torch.float32)).to(dy.dtype)

    def row_bwd(self, dy_shard, x, p: ShardedParam):
        """Backward of row_fwd: returns dx [T, cols]; weight gradient gathered(dy)^T x into the full gradient."""
        m = self.mesh
        w, wg = self.weight(p)
        if m.tp > 1 and self.fused:
            dx, dyg = self._tp(dy_shard.shape[0] * m.tp).all_gather_gemm(dy_shard.contiguous(), w, b_mn=True, wg=wg, n=p.cols,
                                                                         k=p.rows)
        else:
            dyg = self.tp_all_gather_rows(dy_shard)
            if wg is not None:
                from .tp import fused_gemm
                dx = fused_gemm(dyg, w, b_mn=True, n=p.cols, k=p.rows, wg=wg, copy_ctas=self.copy_ctas)
            else:
                dx = F.gemm(dyg, w[: p.rows], b_mn=True)
        F.gemm(dyg, x, a_mn=True, b_mn=True, out=self.grad_view(p), accumulate=True)
        return dx

    # ------------------------------------------------------------------------------------------ model
    def rope(self):
        if self._rope is None:
            c = self.cfg
            self._rope = F.rope_tables(c.head_dim, c.max_seq_len, c.rope_theta, c.rope_scaling_mode, c.rope_scaling_factor,
                                       c.rope_original_max_seq_len, c.yarn_attn_factor, c.yarn_beta_fast, c.yarn_beta_slow,
                                       device=self.device)
        return self._rope

    def _embed(self, ids_f):
        """Partial embedding [T, H] of this tp rank's vocabulary slice (zero rows for ids of other slices)."""
        cfg, m = self.cfg, self.mesh
        p = self.params["tok_embeddings"]
        Vl = cfg.vocab_size // m.tp
        lo = m.tp_rank * Vl
        T, H = ids_f.numel(), cfg.hidden_size
        if self.fused and m.dp > 1:
            out = torch.empty((T, H), dtype=self.dtype, device=self.device)
            lib = _lib.lib()
            lib.tfb_embedding_fwd_sharded.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_int,
                                                      C.c_longlong, C.c_longlong, C.c_void_p]
            lib.tfb_embedding_fwd_sharded.restype = C.c_int
            _lib.check(lib.tfb_embedding_fwd_sharded(ids_f.data_ptr(), p.src.data_ptr(), out.data_ptr(), T, H, p.per, m.dp, lo, Vl,
                                                     _lib.stream()), "embedding_fwd_sharded")
            return out
        w, _ = self.weight(p)
        loc = ids_f - lo
        bad = (loc < 0) | (loc >= Vl)
        out = F.embedding_fwd(loc.masked_fill(bad, 0), w[: p.rows], None, 1)
        if m.tp > 1:
            out = out.masked_fill(bad[:, None], 0)
        return out

    def _embed_bwd(self, ids_f, dh_full):
        cfg, m = self.cfg, self.mesh
        p = self.params["tok_embeddings"]
        Vl = cfg.vocab_size // m.tp
        loc = ids_f - m.tp_rank * Vl
        if m.tp > 1:
            bad = (loc < 0) | (loc >= Vl)
            loc = loc.masked_fill(bad, 0)
            dh_full = dh_full.masked_fill(bad[:, None], 0)
        F.embedding_bwd(loc, dh_full.contiguous(), self.grad_view(p), None, 1)

    def _block_fwd(self, i, h, B, S):
        cfg, m = self.cfg, self.mesh
        hq, hkv, Fl, D = _tp_slices(cfg, m.tp_rank, m.tp)
        P = self.params
        pre = f"layers.{i}."
        rope = self.rope()
        a, _, st1 = F.rmsnorm_fwd(h, self.small(pre + "attention_norm"), cfg.norm_eps)
        qkv, ag = self.col_fwd(a, P[pre + "qkv"])
        F.rope_(qkv, rope[0], rope[1], hq + hkv, D, S)
        o, lse = F.attn_fwd(qkv, qkv, qkv, B, S, hq, hkv, D, k_col0=hq * D, v_col0=(hq + hkv) * D)
        h_mid = self.row_fwd(o, P[pre + "o"], h)
        f, _, st2 = F.rmsnorm_fwd(h_mid, self.small(pre + "ffn_norm"), cfg.norm_eps)
        gu, fg = self.col_fwd(f, P[pre + "gate_up"])
        act = F.glu_fwd(gu, cfg.act_kernel) if cfg.gated else F.act_fwd(gu, cfg.act_kernel)
        h_out = self.row_fwd(act, P[pre + "down"], h_mid)
        return h_out, (h, st1, ag, qkv, o, lse, h_mid, st2, fg, gu, act)

    def _block_bwd(self, i, ctx, dh_out, B, S):
        cfg, m = self.cfg, self.mesh
        hq, hkv, Fl, D = _tp_slices(cfg, m.tp_rank, m.tp)
        P = self.params
        pre = f"layers.{i}."
        rope = self.rope()
        h, st1, ag, qkv, o, lse, h_mid, st2, fg, gu, act = ctx
        d_act = self.row_bwd(dh_out, act, P[pre + "down"])
        d_gu = F.glu_bwd(gu, d_act, cfg.act_kernel) if cfg.gated else F.act_bwd(gu, d_act, cfg.act_kernel)
        d_f = self.col_bwd(d_gu, fg, P[pre + "gate_up"])
        dh_mid = F.rmsnorm_bwd(d_f, h_mid, self.small(pre + "ffn_norm"), st2, self.small_g(pre + "ffn_norm"), dh_out)
        d_o = self.row_bwd(dh_mid, o, P[pre + "o"])
        d_qkv = torch.empty_like(qkv)
        F.attn_bwd(qkv, qkv, qkv, o, d_o, lse, d_qkv, B, S, hq, hkv, D, k_col0=hq * D, v_col0=(hq + hkv) * D)
        F.rope_(d_qkv, rope[0], rope[1], hq + hkv, D, S, backward=True)
        d_a = self.col_bwd(d_qkv, ag, P[pre + "qkv"])
        return F.rmsnorm_bwd(d_a, h, self.small(pre + "attention_norm"), st1, self.small_g(pre + "attention_norm"), dh_mid)

    def _vp_cross_entropy(self, logits, labels, scale, ignore_index):
        """In-place gradient over the local vocabulary slice; returns the per-token loss [t] (same on every tp rank)."""
        m, cfg = self.mesh, self.cfg
        Vl = cfg.vocab_size // m.tp
        lo = m.tp_rank * Vl
        t = logits.shape[0]
        if m.tp == 1:
            return F.cross_entropy_fwd_bwd(logits, labels, scale, ignore_index, 0.0)
        if logits.is_cuda:
            lib = _lib.lib()
            lib.tfb_ce_vp_stats.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_longlong,
                                            C.c_longlong, C.c_longlong, C.c_void_p]
            lib.tfb_ce_vp_grad.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_longlong,
                                           C.c_longlong, C.c_longlong, C.c_void_p]
            lib.tfb_ce_vp_stats.restype = lib.tfb_ce_vp_grad.restype = C.c_int
            stats = torch.empty((t, 4), dtype=torch.float32, device=logits.device)
            _lib.check(lib.tfb_ce_vp_stats(logits.data_ptr(), labels.data_ptr(), stats.data_ptr(), t, Vl, logits.stride(0), lo,
                                           cfg.vocab_size, ignore_index, _lib.stream()), "ce_vp_stats")
        else:
            z = logits.float()
            mx = z.max(-1).values
            loc = labels - lo
            own = (labels != ignore_index) & (loc >= 0) & (loc < Vl)
            zy = torch.where(own, z.gather(1, loc.clamp(0, Vl - 1)[:, None])[:, 0], torch.zeros_like(mx))
            stats = torch.stack([mx, torch.exp(z - mx[:, None]).sum(-1), zy, torch.zeros_like(mx)], 1)
        if self.fused:
            allst = self._tp_coll.all_gather(stats.view(-1)).view(m.tp, t, 4)
        else:
            parts = [torch.empty_like(stats) for _ in range(m.tp)]
            dist.all_gather(parts, stats, group=m.tp_group)
            allst = torch.stack(parts, 0)
        gmx = allst[:, :, 0].max(0).values
        gsum = (allst[:, :, 1] * torch.exp(allst[:, :, 0] - gmx[None])).sum(0)
        lse = gmx + torch.log(gsum)
        valid = labels != ignore_index
        loss = torch.where(valid, lse - allst[:, :, 2].sum(0), torch.zeros_like(lse))
        if logits.is_cuda:
            _lib.check(_lib.lib().tfb_ce_vp_grad(logits.data_ptr(), labels.data_ptr(), lse.contiguous().data_ptr(), scale.data_ptr(),
                                                 t, Vl, logits.stride(0), lo, ignore_index, _lib.stream()), "ce_vp_grad")
        else:
            g = torch.exp(logits.float() - lse[:, None])
            loc = labels - lo
            own = valid & (loc >= 0) & (loc < Vl)
            g[own, loc[own]] -= 1.0
            logits.copy_((g * (scale.float() * valid.float())[:, None]).to(logits.dtype))
        return loss

    def _head_loss_bwd(self, h_shard, lab_f, ignore_index):
        cfg, m = self.cfg, self.mesh
        f_s, _, st = F.rmsnorm_fwd(h_shard, self.small("norm"), cfg.norm_eps)
        fg = self.tp_all_gather_rows(f_s)
        T = fg.shape[0]
        p = self.params["tok_embeddings" if self.tied else "lm_head"]
        n_valid = (lab_f != ignore_index).sum().clamp(min=1).float()
        scale = (1.0 / n_valid).reshape(1)
        d_fg = torch.empty_like(fg)
        losses = torch.empty(T, dtype=torch.float32, device=fg.device)
        ck = max(BLK, min(self.loss_chunk_tokens, T))
        gw = self.grad_view(p)
        for t0 in range(0, T, ck):
            t1 = min(T, t0 + ck)
            w, wg = self.weight(p)
            if wg is not None:
                from .tp import fused_gemm
                logits = fused_gemm(fg[t0:t1], w, n=p.rows, wg=wg, copy_ctas=self.copy_ctas)
            else:
                logits = F.gemm(fg[t0:t1], w[: p.rows])
            losses[t0:t1] = self._vp_cross_entropy(logits, lab_f[t0:t1], scale, ignore_index)
            F.gemm(logits, w[: p.rows], b_mn=True, out=d_fg[t0:t1])
            F.gemm(logits, fg[t0:t1], a_mn=True, b_mn=True, out=gw, accumulate=True)
        loss = losses.sum() / n_valid
        d_f = self.tp_reduce_scatter_rows(d_fg)
        dh = F.rmsnorm_bwd(d_f, h_shard, self.small("norm"), st, self.small_g("norm"), None)
        return loss, dh

    # ------------------------------------------------------------------------------------------ gradient reduction
    def _unit_done(self, unit):
        """The backward of ``unit`` is complete on this rank: reduce-scatter its gradients over the dp group."""
        m = self.mesh
        ps = self.units[unit]
        if not ps:
            return
        if m.dp == 1:
            for p in ps:    # the full gradient is the shard gradient
                self.gshard[p.shard_off:p.shard_off + p.per * p.cols].copy_(self.full_grad[p.full_off:p.full_off + p.rows_p * p.cols])
            return
        if self.fused:
            self._ev_main.record()
            self._side.wait_event(self._ev_main)
            with torch.cuda.stream(self._side):
                _lib.check(_lib.lib().tfb_fsdp_reduce_scatter(C.byref(self._rs_desc[unit]), self.rs_ctas, self._side.cuda_stream),
                           "fsdp_reduce_scatter")
            return
        for p in ps:
            full = self.full_grad[p.full_off:p.full_off + p.rows_p * p.cols]
            dst = self.gshard[p.shard_off:p.shard_off + p.per * p.cols]
            if full.is_cuda:
                self._pending.append(dist.reduce_scatter_tensor(dst, full, op=dist.ReduceOp.AVG, group=m.dp_group, async_op=True))
            else:
                tmp = full.clone()
                dist.all_reduce(tmp, group=m.dp_group)
                n = p.per * p.cols
                dst.copy_(tmp[m.dp_rank * n:(m.dp_rank + 1) * n] / m.dp)

    # ------------------------------------------------------------------------------------------ step
    @torch.no_grad()
    def forward_backward(self, ids, labels, ignore_index: int = -100):
        """ids / labels [B, S] of this data-parallel group (identical on its tp ranks).  Leaves reduced gradients in the
        shard buffers and returns the mean loss of the group's batch (device scalar)."""
        cfg, m = self.cfg, self.mesh
        B, S = ids.shape
        T = B * S
        assert T % (m.tp * (BLK if (self.fused and m.tp > 1) else 1)) == 0, "tokens per step must divide into 128-row tiles per tp rank"
        ids_f, lab_f = ids.reshape(-1).contiguous(), labels.reshape(-1).contiguous()
        L = cfg.num_layers
        head_unit = 0 if self.tied else L + 1
        self._prefetch(1, 0)
        h = self.tp_reduce_scatter_rows(self._embed(ids_f))
        ctxs = []
        ckpt = self.activation_checkpointing
        for i in range(L):
            self._prefetch(2 + i if i + 1 < L else head_unit, 1 + i)
            h_in = h
            h, c = self._block_fwd(i, h, B, S)
            ctxs.append(h_in if ckpt else c)
        self._prefetch(L, head_unit)
        loss, dh = self._head_loss_bwd(h, lab_f, ignore_index)
        if not self.tied:
            self._unit_done(cfg.num_layers + 1)
        for i in range(cfg.num_layers - 1, -1, -1):
            if i > 0:
                self._prefetch(i, 1 + i)
            c = self._block_fwd(i, ctxs[i], B, S)[1] if ckpt else ctxs[i]
            dh = self._block_bwd(i, c, dh, B, S)
            ctxs[i] = None
            self._unit_done(1 + i)
        self._embed_bwd(ids_f, self.tp_all_gather_rows(dh))
        self._unit_done(0)
        return loss

    def _all_reduce_world(self, t):
        if self.mesh.world > 1:
            dist.all_reduce(t, group=self.mesh.world_group)
        return t

    @torch.no_grad()
    def optimizer_step(self, lr: Optional[float] = None):
        m = self.mesh
        self.step_count += 1
        t = self.step_count
        lr = self.lr if lr is None else lr
        if self.fused and m.dp > 1:
            self._ev_side.record(self._side)
            torch.cuda.current_stream().wait_event(self._ev_side)
        for w in self._pending:
            w.wait()
        self._pending = []
        # norm weights: every rank holds a partial gradient (its tokens); sum over tp, average over dp
        self._all_reduce_world(self.small_grad)
        if m.dp > 1:
            self.small_grad.div_(m.dp)
        if not (self.fused and m.dp > 1):
            self.sumsq.zero_()
            F.sumsq(self.gshard, self.sumsq)
        self._sumsq_small.zero_()
        F.sumsq(self.small_grad, self._sumsq_small)
        self.sumsq.add_(self._sumsq_small / m.world)        # replicated on every rank of the mesh: counted once
        self._all_reduce_world(self.sumsq)
        F.clip_factor(self.sumsq, 1.0, self.max_grad_norm, self.last_grad_norm, self._clip, self._found_inf)
        b1, b2 = self.betas
        self.hyper[:3] = torch.tensor([lr, 1.0 - b1 ** t, 1.0 - b2 ** t], dtype=torch.float32)
        F.adamw_(self.master, self.gshard, self.m, self.v, self.shard_lp, lr, b1, b2, self.eps, self.weight_decay, t, self._clip,
                 True, self.hyper)
        F.adamw_(self.small_master, self.small_grad, self.small_m, self.small_v, self.small_lp, lr, b1, b2, self.eps, 0.0, t,
                 self._clip, True, self.hyper)
        if self.fused and m.dp > 1:
            self.dp_heap.barrier()      # every rank finished reading gradients and refreshed its shards
        self.full_grad.zero_()
        self.sumsq.zero_()
        self.invalidate_gathers()

    def train_step(self, ids, labels, lr: Optional[float] = None):
        loss = self.forward_backward(ids, labels)
        self.optimizer_step(lr)
        return loss

    # ------------------------------------------------------------------------------------------ reporting / export
    def memory_profile(self):
        """Bytes this rank holds, and the figure without any sharding for comparison."""
        esz = self.shard_lp.element_size()
        params = self.shard_numel * esz + self.small_lp.numel() * esz
        gather = sum(s.numel() for s in self.slots) * esz if self.slots else 0
        opt = (self.master.numel() + self.small_master.numel()) * 12
        grads = self.full_numel * 4 + self.gshard.numel() * 4
        full_model = sum(p.rows * p.cols for p in self.params.values()) * self.mesh.tp + self.small_lp.numel()
        return {"parameters": params, "gather_buffers": gather, "optimizer_state": opt, "gradients": grads,
                "total": params + gather + opt + grads, "unsharded_total": full_model * (esz + 12 + 4)}

    @torch.no_grad()
    def gather_full(self, name):
        """The whole (all dp shards, all tp pieces) matrix of a sharded parameter, for checkpoints and tests."""
        m, cfg = self.mesh, self.cfg
        p = self.params[name]
        sh = self.shard_view(p).contiguous()
        if m.dp > 1:
            parts = [torch.empty_like(sh) for _ in range(m.dp)]
            dist.all_gather(parts, sh, group=m.dp_group)
            piece = torch.cat(parts, 0)[: p.rows]
        else:
            piece = sh[: p.rows]
        if m.tp == 1:
            return piece
        parts = [torch.empty_like(piece) for _ in range(m.tp)]
        dist.all_gather(parts, piece.contiguous(), group=m.tp_group)
        base = name.split(".")[-1]
        D = cfg.head_dim
        hq, hkv, Fl, _ = _tp_slices(cfg, 0, m.tp)
        if base in ("tok_embeddings", "lm_head"):
            return torch.cat(parts, 0)
        if base == "qkv":
            return torch.cat([torch.cat([x[:hq * D] for x in parts]), torch.cat([x[hq * D:(hq + hkv) * D] for x in parts]),
                              torch.cat([x[(hq + hkv) * D:] for x in parts])], 0)
        if base == "gate_up":
            if cfg.gated:
                return torch.cat([torch.cat([x[:Fl] for x in parts]), torch.cat([x[Fl:] for x in parts])], 0)
            return torch.cat(parts, 0)
        return torch.cat(parts, 1)        # o, down: column pieces

    @torch.no_grad()
    def export_to(self, model):
        """Write the trained weights back into a DenseModel (every rank ends with the full model)."""
        named = dict(model.named_parameters())
        for name in self.params:
            named[name].data.copy_(self.gather_full(name))
        for name in self.small_index:
            named[name].data.copy_(self.small(name))
        return model
