"""Tensor parallelism with sequence parallelism (Megatron layout) on the fused kernels.

``ColumnParallelLinear``  y[M, N/W]   = all_gather_rows(x_shard[M/W, K]) @ W_local[N/W, K]^T   (all-gather -> GEMM)
``RowParallelLinear``     y_shard[M/W, N] = reduce_scatter_rows(x[M, K/W] @ W_local[N, K/W]^T)  (GEMM -> reduce-scatter)

With ``comm="fused"`` both run as ONE tcgen05 GEMM launch whose CTAs also move the data over NVLink
(see csrc/comm/tp_fused.cu); ``comm="nccl"`` is the library baseline (all_gather_into_tensor /
reduce_scatter_tensor around the same GEMM).  Helper functions mirror the reference's
TensorParallelManager: ``column_parallel_split``, ``row_parallel_split``, ``partition_heads``,
``reconstruct_weight``, ``communication_volume`` (include/quant/tensor_parallelism.h:16-173,
src/trainer/tensor_parallelism.cpp:26-508)."""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib, functional as F
from ..ops._lib import c_i, c_ll, c_p, check, stream


class _Tp(C.Structure):
    """Mirror of TfbGemmTp (csrc/kernels/gemm_bf16.cu): ``mode`` bits 1 all-gather -> GEMM, 2 GEMM -> reduce-scatter,
    4 weight gather -> GEMM."""
    _fields_ = [("mode", C.c_int), ("rank", C.c_int), ("world", C.c_int), ("copy_ctas", C.c_int), ("epoch", C.c_int),
                ("ready", C.c_void_p), ("peer_a", C.c_void_p), ("peer_c", C.c_void_p), ("peer_c_host", C.c_void_p),
                ("wg_rank", C.c_int), ("wg_world", C.c_int), ("wg_epoch", C.c_int), ("wg_rows", C.c_int),
                ("wg_ready", C.c_void_p), ("wg_src", C.c_void_p), ("wg_skip_local", C.c_int)]


def _fn():
    fn = _lib.lib().tfb_gemm_bf16_tp
    fn.argtypes = [c_p, c_ll, c_p, c_ll, c_i, c_p, c_ll, c_i, c_i, c_i, c_p, c_ll, C.POINTER(_Tp), c_p, c_p]
    fn.restype = c_i
    _lib.lib().tfb_tp_reduce.argtypes = [c_p, c_p, c_p, c_ll, c_i, c_i, c_p]
    _lib.lib().tfb_tp_reduce.restype = c_i
    return fn


class WeightGather:
    """What the GEMM needs to pull a row-sharded weight (ZeRO-3 / FSDP) into its local gather buffer while it runs:
    ``buf`` [rows_p, cols] local bf16 gather buffer, ``src`` device int64[world] with the base address of every rank's
    shard ([rows_p / world, cols], symmetric memory), ``ready`` local int32[rows_p / 128] flags and the value ``epoch``
    they take once a block has landed (one more than at the previous gather into the same flags)."""
    __slots__ = ("buf", "src", "ready", "epoch", "rank", "world", "rows_p", "skip_local")

    def __init__(self, buf, src, ready, epoch, rank, world, skip_local=False):
        """``skip_local``: this rank's own rows are already in ``buf`` (copied by the caller): only remote rows travel."""
        self.buf, self.src, self.ready, self.epoch, self.rank, self.world = buf, src, ready, epoch, rank, world
        self.rows_p = buf.shape[0]
        self.skip_local = skip_local


def fused_gemm(x, w, *, b_mn=False, n=None, k=None, out=None, residual=None, tp=None, wg: WeightGather = None, copy_ctas=8):
    """One launch of the tcgen05 GEMM with a collective folded in: ``tp`` = (mode bit 1 or 2, rank, world, epoch, ready,
    peer_a ptrs, peer_c ptrs) for the tensor-parallel all-gather / reduce-scatter, ``wg`` for the weight gather.
    x [M, K]; ``w`` [N, K] (or [K, N] with ``b_mn``; for a gathered weight pass the gather buffer's view); returns y
    [M, N] (None for the reduce-scatter form, whose partial products go to the peers' staging buffers)."""
    M = x.shape[0]
    K = k if k is not None else x.shape[1]
    N = n if n is not None else (w.shape[1] if b_mn else w.shape[0])
    d = _Tp()
    mode = 0
    if tp is not None:
        mode |= tp[0]
        d.rank, d.world, d.epoch = tp[1], tp[2], tp[3]
        d.ready, d.peer_a, d.peer_c = tp[4], tp[5], tp[6]
        if len(tp) > 7 and tp[7] is not None:
            d.peer_c_host = C.cast(tp[7], C.c_void_p)
    if wg is not None:
        mode |= 4
        d.wg_rank, d.wg_world, d.wg_epoch, d.wg_rows = wg.rank, wg.world, wg.epoch, wg.rows_p
        d.wg_ready, d.wg_src = wg.ready.data_ptr(), wg.src.data_ptr()
        d.wg_skip_local = int(wg.skip_local)
    d.mode, d.copy_ctas = mode, copy_ctas
    y = None
    if not (mode & 2):
        y = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ldc = y.stride(0) if y is not None else N
    check(_fn()(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), int(b_mn), ptr_or_none(y), ldc, M, N, K,
                ptr_or_none(residual), residual.stride(0) if residual is not None else 0, C.byref(d),
                _lib.status_word(x.device).data_ptr(), stream()), "fused_gemm")
    return y


def ptr_or_none(t):
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------------------------------- splits
def column_parallel_split(w, world, rank):
    """Rows (output features) in ceil chunks, like the reference (tensor_parallelism.cpp:26-35)."""
    per = (w.shape[0] + world - 1) // world
    return w[rank * per: min(w.shape[0], (rank + 1) * per)].contiguous()


def row_parallel_split(w, world, rank):
    per = (w.shape[1] + world - 1) // world
    return w[:, rank * per: min(w.shape[1], (rank + 1) * per)].contiguous()


def partition_heads(num_heads, world, rank):
    per = (num_heads + world - 1) // world
    return list(range(rank * per, min(num_heads, (rank + 1) * per)))


def reconstruct_weight(shards, column=True):
    return torch.cat(shards, 0 if column else 1)


def communication_volume(M, K, N, world, dtype_bytes=2):
    """Bytes each rank moves per column-parallel + row-parallel pair with sequence parallelism."""
    ag = (world - 1) * (M // world) * K * dtype_bytes
    rs = (world - 1) * (M // world) * N * dtype_bytes
    return {"all_gather": ag, "reduce_scatter": rs, "total": ag + rs}


# ---------------------------------------------------------------------------------------------- fused ops
class TpContext:
    """Symmetric buffers shared by the fused TP ops of one model shard (double-buffered gather / staging)."""

    def __init__(self, symm, rank, world, max_rows, max_k, max_n, copy_ctas=16):
        self.symm, self.rank, self.world, self.copy_ctas = symm, rank, world, copy_ctas
        dev = symm.device
        self.gather = [symm.alloc(max_rows * max_k, torch.bfloat16) for _ in range(2)]
        self.stage = [symm.alloc(world * (max_rows // world) * max_n, torch.bfloat16) for _ in range(2)]
        self.ready = torch.zeros(max_rows // 128 + 1, dtype=torch.int32, device=dev)
        self.epoch = 0
        self.parity = 0
        self._stage_host = {}     # staging buffer -> ctypes array of the W peer addresses (for the TMA-store epilogue)

    def all_gather_gemm(self, x_shard, w, out=None, b_mn=False, wg: WeightGather = None, n=None, k=None):
        """x_shard [M/W, K] -> y [M, N_local]; ``w`` [N_local, K], or [K, N_local] with ``b_mn``.  With ``wg`` the
        weight's row shards are gathered over the data-parallel group inside the same launch."""
        Ms, K = x_shard.shape
        M = Ms * self.world
        buf = self.gather[self.parity]
        xg = buf.view(torch.bfloat16, M * K).view(M, K)
        xg[self.rank * Ms:(self.rank + 1) * Ms].copy_(x_shard)      # producer kernels may write here directly
        self.symm.barrier()                                           # every rank's shard is in place
        self.epoch += 1
        tp = (1, self.rank, self.world, self.epoch, self.ready.data_ptr(), buf.ptrs.data_ptr(), None)
        y = fused_gemm(xg, w, b_mn=b_mn, n=n, k=k, out=out, tp=tp, wg=wg, copy_ctas=self.copy_ctas)
        self.parity ^= 1
        return y, xg

    def gemm_reduce_scatter(self, x, w, residual=None, b_mn=False, wg: WeightGather = None, n=None, k=None):
        """x [M, K_local], ``w`` [N, K_local] (or [K_local, N] with ``b_mn``) -> y_shard [M/W, N] = sum over ranks of the
        partial products (+ ``residual`` [M/W, N])."""
        M = x.shape[0]
        N = n if n is not None else (w.shape[1] if b_mn else w.shape[0])
        Ms = M // self.world
        buf = self.stage[self.parity]
        host = self._stage_host.get(id(buf))
        if host is None:
            host = self._stage_host[id(buf)] = (C.c_void_p * self.world)(*buf.peer_ptrs)
        tp = (2, self.rank, self.world, 0, None, None, buf.ptrs.data_ptr(), host)
        fused_gemm(x, w, b_mn=b_mn, n=N, k=k, tp=tp, wg=wg, copy_ctas=self.copy_ctas)
        self.symm.barrier()                                           # all partial tiles have arrived
        out = torch.empty((Ms, N), dtype=torch.bfloat16, device=x.device)
        stage = buf.view(torch.bfloat16, self.world * Ms * N)
        check(_lib.lib().tfb_tp_reduce(stage.data_ptr(), residual.data_ptr() if residual is not None else None,
                                       out.data_ptr(), Ms, N, self.world, stream()), "tp_reduce")
        self.parity ^= 1
        return out


class ColumnParallelLinear(torch.nn.Module):
    def __init__(self, weight_full, rank, world, ctx: TpContext = None, group=None):
        super().__init__()
        self.weight = torch.nn.Parameter(column_parallel_split(weight_full, world, rank))
        self.rank, self.world, self.ctx, self.group = rank, world, ctx, group

    def local_weight(self): return self.weight
    def local_bias(self): return None                      # the dense blocks carry their biases outside the TP products
    def local_out_features(self) -> int: return self.weight.shape[0]

    def forward(self, x_shard):
        if self.world == 1:
            return F.gemm(x_shard, self.weight.data)
        if self.ctx is not None and x_shard.is_cuda:
            return self.ctx.all_gather_gemm(x_shard, self.weight.data)[0]
        xs = [torch.empty_like(x_shard) for _ in range(self.world)]
        dist.all_gather(xs, x_shard.contiguous(), group=self.group)
        return F.gemm(torch.cat(xs, 0), self.weight.data)


class RowParallelLinear(torch.nn.Module):
    def __init__(self, weight_full, rank, world, ctx: TpContext = None, group=None):
        super().__init__()
        self.weight = torch.nn.Parameter(row_parallel_split(weight_full, world, rank))
        self.rank, self.world, self.ctx, self.group = rank, world, ctx, group

    def local_weight(self): return self.weight
    def local_bias(self): return None
    def local_in_features(self) -> int: return self.weight.shape[1]

    def forward(self, x, residual_shard=None):
        if self.world == 1:
            return F.gemm(x, self.weight.data, residual=residual_shard)
        if self.ctx is not None and x.is_cuda:
            return self.ctx.gemm_reduce_scatter(x, self.weight.data, residual_shard)
        y = F.gemm(x, self.weight.data, out_dtype=torch.float32)
        dist.all_reduce(y, group=self.group)
        Ms = y.shape[0] // self.world
        out = y[self.rank * Ms:(self.rank + 1) * Ms]
        if residual_shard is not None:
            out = out + residual_shard.float()
        return out.to(x.dtype)


# ---------------------------------------------------------------------------------------------- manager API
class HeadPartitioner:
    """Attention heads per rank (query heads and, for grouped-query attention, the kv heads they share)."""

    def __init__(self, num_heads, num_kv_heads, world, rank: int = 0, head_dim: int = 0, group=None):
        assert num_heads % world == 0, "query heads must divide over the ranks"
        self.h, self.kv, self.world = num_heads, num_kv_heads, world
        self.rank, self.head_dim, self.group = rank, head_dim, group

    # ---- this rank's range and the tensor forms (reference: HeadPartitioner, include/quant/tensor_parallelism.h:141-171)
    def heads_per_rank(self) -> int: return self.h // self.world
    def head_start(self) -> int: return self.rank * self.heads_per_rank()
    def head_end(self) -> int: return self.head_start() + self.heads_per_rank()

    def partition_heads(self, x: torch.Tensor, seq_len: int = 0) -> torch.Tensor:
        """This rank's heads of a [..., num_heads * head_dim] tensor."""
        d = self.head_dim or x.shape[-1] // self.h
        return x[..., self.head_start() * d:self.head_end() * d].contiguous()

    def merge_heads(self, local: torch.Tensor, seq_len: int = 0) -> torch.Tensor:
        """Inverse of ``partition_heads``: every rank's heads side by side (an all-gather over the ranks)."""
        if self.world == 1 or not dist.is_initialized():
            return local
        parts = [torch.empty_like(local) for _ in range(self.world)]
        dist.all_gather(parts, local.contiguous(), group=self.group)
        return torch.cat(parts, -1)

    def sync_output(self, output: torch.Tensor) -> torch.Tensor:
        """Sum the ranks' partial outputs of the projection that follows the heads (in place)."""
        if self.world > 1 and dist.is_initialized():
            dist.all_reduce(output, group=self.group)
        return output

    def q_heads(self, rank):
        return partition_heads(self.h, self.world, rank)

    def kv_heads(self, rank):
        """kv heads used by this rank's query heads (replicated when there are fewer kv heads than ranks)."""
        g = self.h // self.kv
        return sorted({q // g for q in self.q_heads(rank)})


class SequenceParallel:
    """Scatter / gather along the sequence dimension around tensor-parallel regions."""

    def __init__(self, rank, world, group=None):
        self.rank, self.world, self.group = rank, world, group

    def scatter(self, x, seq_dim=1):
        n = x.shape[seq_dim] // self.world
        return x.narrow(seq_dim, self.rank * n, n).contiguous()

    def gather(self, x_shard, seq_dim=1):
        if self.world == 1 or not dist.is_initialized():
            return x_shard
        parts = [torch.empty_like(x_shard) for _ in range(self.world)]
        dist.all_gather(parts, x_shard.contiguous(), group=self.group)
        return torch.cat(parts, seq_dim)

    def reduce_scatter(self, x, seq_dim=1):
        if self.world > 1 and dist.is_initialized():
            x = x.clone()
            dist.all_reduce(x, group=self.group)
        return self.scatter(x, seq_dim)

    def allreduce(self, x):
        if self.world > 1 and dist.is_initialized():
            dist.all_reduce(x, group=self.group)
        return x

    def world_size(self) -> int: return self.world
    def world_rank(self) -> int: return self.rank


class TensorParallelManager:
    """The reference's manager API on top of the fused kernels: weight splitting, column / row parallel products,
    head partitioning, sequence-parallel scatter / gather, strategy selection and whole-model parallelisation."""

    def __init__(self, model=None, world_size=1, rank=0, ctx: TpContext = None, group=None):
        self.model, self.world, self.rank, self.ctx, self.group = model, world_size, rank, ctx, group
        self.sp = SequenceParallel(rank, world_size, group)

    column_parallel_split = staticmethod(column_parallel_split)
    row_parallel_split = staticmethod(row_parallel_split)
    reconstruct_weight = staticmethod(reconstruct_weight)
    communication_volume = staticmethod(communication_volume)

    def world_size(self) -> int: return self.world
    def world_rank(self) -> int: return self.rank

    def partition_heads(self, num_heads):
        return partition_heads(num_heads, self.world, self.rank)

    def column_parallel_linear(self, x_shard, local_w):
        return ColumnParallelLinear.forward(_Lin(local_w, self), x_shard)

    def row_parallel_linear(self, x, local_w, residual_shard=None):
        return RowParallelLinear.forward(_Lin(local_w, self, row=True), x, residual_shard)

    def sequence_parallel_scatter(self, x, seq_dim=1):
        return self.sp.scatter(x, seq_dim)

    def sequence_parallel_gather(self, x, seq_dim=1):
        return self.sp.gather(x, seq_dim)

    def allreduce_tensor(self, t):
        if self.world > 1 and dist.is_initialized():
            dist.all_reduce(t, group=self.group)
        return t

    def allgather_tensor(self, t, dim=0):
        return SequenceParallel(self.rank, self.world, self.group).gather(t, dim)

    def reduce_scatter_tensor(self, t, dim=0):
        return SequenceParallel(self.rank, self.world, self.group).reduce_scatter(t, dim)

    @staticmethod
    def select_strategy(cfg, world_size, batch_tokens=8192):
        """'none' | 'tp' | 'tp+sp': tensor parallelism pays once a layer's weights dominate its activations; sequence
        parallelism is added when the activations between the TP regions are large enough to be worth sharding."""
        if world_size == 1 or cfg.num_heads % world_size:
            return "none"
        w_bytes = 2 * cfg.hidden_size * ((cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim + cfg.hidden_size + 3 * cfg.ffn_hidden_size)
        a_bytes = 2 * batch_tokens * cfg.hidden_size
        if w_bytes < a_bytes // 4:
            return "none"
        return "tp+sp" if batch_tokens % world_size == 0 and a_bytes > (1 << 20) else "tp"

    def parallelize_block(self, blk, cfg):
        """This rank's shards of one block: q / k / v / gate / up by output rows (column parallel, by whole heads),
        o / down by input columns (row parallel)."""
        W, r, D = self.world, self.rank, cfg.head_dim
        hp = HeadPartitioner(cfg.num_heads, cfg.num_kv_heads, W)
        nq, nkv = cfg.num_heads * D, cfg.num_kv_heads * D
        qkv = blk.qkv.data
        q_rows = torch.cat([torch.arange(h * D, (h + 1) * D) for h in hp.q_heads(r)])
        kv_sel = torch.cat([torch.arange(h * D, (h + 1) * D) for h in hp.kv_heads(r)])
        out = {"q": qkv[:nq][q_rows], "k": qkv[nq:nq + nkv][kv_sel], "v": qkv[nq + nkv:][kv_sel],
               "o": blk.o.data[:, q_rows], "down": row_parallel_split(blk.down.data, W, r)}
        F_ = cfg.ffn_hidden_size
        if cfg.gated:
            out["gate"] = column_parallel_split(blk.gate_up.data[:F_], W, r)
            out["up"] = column_parallel_split(blk.gate_up.data[F_:], W, r)
        else:
            out["up"] = column_parallel_split(blk.gate_up.data, W, r)
        return out

    def parallelize_model(self, model=None):
        """{layer index: shards} plus vocabulary-parallel embedding / LM-head rows."""
        m = model or self.model
        out = {i: self.parallelize_block(l, m.cfg) for i, l in enumerate(m.layers)}
        out["tok_embeddings"] = column_parallel_split(m.tok_embeddings.data, self.world, self.rank)
        out["lm_head"] = column_parallel_split(m.lm_head.data, self.world, self.rank)
        return out


class _Lin:
    """Adapter that lets the manager reuse the module forward paths with an externally owned weight."""

    def __init__(self, w, mgr: TensorParallelManager, row=False):
        self.weight = torch.nn.Parameter(w, requires_grad=False)
        self.rank, self.world, self.ctx, self.group = mgr.rank, mgr.world, mgr.ctx, mgr.group


