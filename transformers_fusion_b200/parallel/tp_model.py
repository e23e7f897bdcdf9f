"""Tensor-parallel + sequence-parallel training of the dense model.

Layout (Megatron-style with sequence parallelism): between the tensor-parallel regions every rank holds a row shard
[T / W, H] of the token stream; inside them it holds all T rows of its own heads / FFN columns.

  h_shard -> norm -> [all-gather rows -> qkv GEMM]  (column parallel: this rank's q / k / v heads)
          -> RoPE + flash attention on the local heads
          -> [o GEMM -> reduce-scatter rows] + h_shard                      (row parallel)
          -> norm -> [all-gather rows -> gate|up GEMM] -> GLU -> [down GEMM -> reduce-scatter rows] + residual

On CUDA with a ``TpContext`` the bracketed pairs are single fused kernels over NVLink peer memory (all_gather_gemm,
gemm_reduce_scatter); otherwise they are a torch.distributed collective plus a GEMM, which is also the CPU / gloo path.
The backward of a column-parallel product is a row-parallel one and vice versa, so the same two fused kernels serve it.
Embedding, norms and LM head are replicated; each rank computes the loss of its own rows and the replicated gradients
are summed over the TP group after backward.

Reference counterparts: TensorParallelManager::parallelize_model / column_parallel_linear / row_parallel_linear and the
sequence-parallel scatter / gather (src/trainer/tensor_parallelism.cpp:53-142, 334-451)."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..models.dense import DenseModel, _ensure_main_grad
from ..models.moe import _RMSNormFn
from ..ops import functional as F


class TPGroup:
    def __init__(self, rank: int, world: int, group=None, ctx=None):
        self.rank, self.world, self.group, self.ctx = rank, world, group, ctx

    def fused(self, t: torch.Tensor) -> bool:
        return self.ctx is not None and t.is_cuda and self.world > 1

    def all_gather_rows(self, x):
        if self.world == 1:
            return x
        out = torch.empty((x.shape[0] * self.world,) + x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, y):
        """Sum over ranks of y [T, N] (fp32), keep this rank's row block."""
        if self.world == 1:
            return y
        y = y.contiguous()
        if y.is_cuda:
            out = torch.empty((y.shape[0] // self.world,) + y.shape[1:], dtype=y.dtype, device=y.device)
            dist.reduce_scatter_tensor(out, y, group=self.group)
            return out
        dist.all_reduce(y, group=self.group)                 # gloo has no reduce-scatter
        n = y.shape[0] // self.world
        return y[self.rank * n:(self.rank + 1) * n].clone()

    def all_reduce(self, t):
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t


class _ColumnParallelFn(torch.autograd.Function):
    """y [T, N_local] = all_gather_rows(x_shard) @ W_local^T."""

    @staticmethod
    def forward(ctx, x_shard, w, tp: TPGroup):
        if tp.fused(x_shard):
            y, xg = tp.ctx.all_gather_gemm(x_shard.contiguous(), w.data)
            xg = xg.clone()                                  # the gather buffer is reused by the next fused call
        else:
            xg = tp.all_gather_rows(x_shard)
            y = F.gemm(xg, w.data)
        ctx.save_for_backward(xg)
        ctx.w, ctx.tp = w, tp
        return y

    @staticmethod
    def backward(ctx, dy):
        (xg,) = ctx.saved_tensors
        w, tp = ctx.w, ctx.tp
        dy = dy.contiguous()
        _ensure_main_grad(w)
        F.gemm(dy, xg, a_mn=True, b_mn=True, out=w.main_grad, accumulate=True)
        if tp.fused(dy):
            dx = tp.ctx.gemm_reduce_scatter(dy, w.data, b_mn=True)
        else:
            dx = tp.reduce_scatter_rows(F.gemm(dy, w.data, b_mn=True, out_dtype=torch.float32)).to(dy.dtype)
        return dx, None, None


class _RowParallelFn(torch.autograd.Function):
    """y_shard [T / W, N] = reduce_scatter_rows(x @ W_local^T) + residual_shard."""

    @staticmethod
    def forward(ctx, x, w, residual_shard, tp: TPGroup):
        if tp.fused(x):
            y = tp.ctx.gemm_reduce_scatter(x.contiguous(), w.data, residual_shard)
        else:
            y = tp.reduce_scatter_rows(F.gemm(x, w.data, out_dtype=torch.float32))
            if residual_shard is not None:
                y = y + residual_shard.float()
            y = y.to(x.dtype)
        ctx.save_for_backward(x)
        ctx.w, ctx.tp, ctx.has_res = w, tp, residual_shard is not None
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        (x,) = ctx.saved_tensors
        w, tp = ctx.w, ctx.tp
        dy_shard = dy_shard.contiguous()
        _ensure_main_grad(w)
        if tp.fused(dy_shard):
            dx, dyg = tp.ctx.all_gather_gemm(dy_shard, w.data, b_mn=True)
        else:
            dyg = tp.all_gather_rows(dy_shard)
            dx = F.gemm(dyg, w.data, b_mn=True)
        F.gemm(dyg, x, a_mn=True, b_mn=True, out=w.main_grad, accumulate=True)
        return dx, None, (dy_shard if ctx.has_res else None), None


class _AttentionCoreFn(torch.autograd.Function):
    """RoPE + causal flash attention over the local heads of a packed [T, (Hq + 2 Hkv) D] projection."""

    @staticmethod
    def forward(ctx, qkv, B, S, Hq, Hkv, D, rope):
        qkv = qkv.clone() if rope is not None else qkv
        if rope is not None:
            F.rope_(qkv, rope[0], rope[1], Hq + Hkv, D, S)
        o, lse = F.attn_fwd(qkv, qkv, qkv, B, S, Hq, Hkv, D, k_col0=Hq * D, v_col0=(Hq + Hkv) * D)
        ctx.save_for_backward(qkv, o, lse)
        ctx.dims, ctx.rope = (B, S, Hq, Hkv, D), rope
        return o

    @staticmethod
    def backward(ctx, d_o):
        qkv, o, lse = ctx.saved_tensors
        B, S, Hq, Hkv, D = ctx.dims
        d_qkv = torch.empty_like(qkv)
        F.attn_bwd(qkv, qkv, qkv, o, d_o.contiguous(), lse, d_qkv, B, S, Hq, Hkv, D, k_col0=Hq * D, v_col0=(Hq + Hkv) * D)
        if ctx.rope is not None:
            F.rope_(d_qkv, ctx.rope[0], ctx.rope[1], Hq + Hkv, D, S, backward=True)
        return d_qkv, None, None, None, None, None, None


class _GluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, act, gated):
        ctx.save_for_backward(gu)
        ctx.act, ctx.gated = act, gated
        return F.glu_fwd(gu, act) if gated else F.act_fwd(gu, act)

    @staticmethod
    def backward(ctx, d):
        (gu,) = ctx.saved_tensors
        d = d.contiguous()
        return (F.glu_bwd(gu, d, ctx.act) if ctx.gated else F.act_bwd(gu, d, ctx.act)), None, None


class _HeadFn(torch.autograd.Function):
    """logits = h @ W^T with the weight gradient accumulated into W.main_grad."""

    @staticmethod
    def forward(ctx, h, w):
        ctx.save_for_backward(h)
        ctx.w = w
        return F.gemm(h, w.data)

    @staticmethod
    def backward(ctx, dy):
        (h,) = ctx.saved_tensors
        w = ctx.w
        dy = dy.contiguous().to(h.dtype)
        _ensure_main_grad(w)
        F.gemm(dy, h, a_mn=True, b_mn=True, out=w.main_grad, accumulate=True)
        return F.gemm(dy, w.data, b_mn=True), None


class TPBlock(nn.Module):
    def __init__(self, cfg, blk, tp: TPGroup):
        super().__init__()
        W, r, D = tp.world, tp.rank, cfg.head_dim
        assert cfg.num_heads % W == 0 and cfg.num_kv_heads % W == 0, "query and kv heads must divide over the TP ranks"
        assert cfg.ffn_hidden_size % W == 0
        assert not cfg.use_parallel_residual and cfg.norm_type == "rmsnorm", "the TP path covers the sequential RMSNorm block"
        self.cfg, self.tp = cfg, tp
        self.hq, self.hkv = cfg.num_heads // W, cfg.num_kv_heads // W
        nq, nkv = cfg.num_heads * D, cfg.num_kv_heads * D
        q, k, v = blk.qkv.data[:nq], blk.qkv.data[nq:nq + nkv], blk.qkv.data[nq + nkv:]
        cut = lambda t, n: t[r * n:(r + 1) * n]
        self.qkv = nn.Parameter(torch.cat([cut(q, self.hq * D), cut(k, self.hkv * D), cut(v, self.hkv * D)], 0).clone())
        self.o = nn.Parameter(blk.o.data[:, r * self.hq * D:(r + 1) * self.hq * D].clone())
        Fh = cfg.ffn_hidden_size
        Fl = Fh // W
        if cfg.gated:
            gu = torch.cat([cut(blk.gate_up.data[:Fh], Fl), cut(blk.gate_up.data[Fh:], Fl)], 0)
        else:
            gu = cut(blk.gate_up.data, Fl)
        self.gate_up = nn.Parameter(gu.clone())
        self.down = nn.Parameter(blk.down.data[:, r * Fl:(r + 1) * Fl].clone())
        self.attention_norm = nn.Parameter(blk.attention_norm.data.clone())
        self.ffn_norm = nn.Parameter(blk.ffn_norm.data.clone())

    def forward(self, h_shard, B, S, rope):
        cfg, tp = self.cfg, self.tp
        a = _RMSNormFn.apply(h_shard, self.attention_norm, cfg.norm_eps)
        qkv = _ColumnParallelFn.apply(a, self.qkv, tp)
        o = _AttentionCoreFn.apply(qkv, B, S, self.hq, self.hkv, cfg.head_dim, rope)
        h_mid = _RowParallelFn.apply(o, self.o, h_shard, tp)
        f = _RMSNormFn.apply(h_mid, self.ffn_norm, cfg.norm_eps)
        gu = _ColumnParallelFn.apply(f, self.gate_up, tp)
        act = _GluFn.apply(gu, cfg.act_kernel, cfg.gated)
        return _RowParallelFn.apply(act, self.down, h_mid, tp)


class TPDenseModel(nn.Module):
    """This rank's shard of a DenseModel.  Build every rank's DenseModel with the same seed (or load the same checkpoint),
    then wrap it; ``gather_into(dense)`` writes the trained shards back for saving."""

    def __init__(self, dense: DenseModel, tp: TPGroup):
        super().__init__()
        cfg = dense.cfg
        assert cfg.position_type == "rope" or dense.pos_embeddings is None
        self.cfg, self.tp, self.dense = cfg, tp, [dense]          # list: keep the source model out of .parameters()
        self.tok_embeddings = nn.Parameter(dense.tok_embeddings.data.clone())
        self.norm = nn.Parameter(dense.norm.data.clone())
        self.tied = dense.lm_head is dense.tok_embeddings or cfg.tie_embeddings
        self.lm_head = self.tok_embeddings if self.tied else nn.Parameter(dense.lm_head.data.clone())
        self.layers = nn.ModuleList(TPBlock(cfg, b, tp) for b in dense.layers)

    def replicated_parameters(self) -> List[nn.Parameter]:
        out = [self.tok_embeddings, self.norm] + ([] if self.tied else [self.lm_head])
        for l in self.layers:
            out += [l.attention_norm, l.ffn_norm]
        return out

    def sharded_parameters(self) -> List[nn.Parameter]:
        return [p for l in self.layers for p in (l.qkv, l.o, l.gate_up, l.down)]

    def _shard_rows(self, t):
        n = t.shape[0] // self.tp.world
        return t[self.tp.rank * n:(self.tp.rank + 1) * n]

    def loss(self, ids, labels, ignore_index: int = -100):
        """Mean next-token loss over ALL rows of the batch (every rank returns the same value after the final sum)."""
        B, S = ids.shape
        T, W = B * S, self.tp.world
        assert T % (W * (128 if ids.is_cuda and W > 1 else 1)) == 0, "tokens per step must divide into 128-row tiles per rank"
        rope = self.dense[0].rope(ids.device)
        ids_f, lab_f = ids.reshape(-1), labels.reshape(-1)
        my_ids, my_lab = self._shard_rows(ids_f), self._shard_rows(lab_f)
        h = torch.nn.functional.embedding(my_ids, self.tok_embeddings)
        for blk in self.layers:
            h = blk(h, B, S, rope)
        h = _RMSNormFn.apply(h, self.norm, self.cfg.norm_eps)
        logits = _HeadFn.apply(h, self.lm_head).float()
        n_valid = (lab_f != ignore_index).sum().clamp(min=1)
        return torch.nn.functional.cross_entropy(logits, my_lab, ignore_index=ignore_index, reduction="sum") / n_valid

    def forward_backward(self, ids, labels):
        """One loss + backward; replicated gradients summed over the TP group.  Returns the global mean loss."""
        for p in self.parameters():
            _ensure_main_grad(p)
        loss = self.loss(ids, labels)
        loss.backward()
        if self.tok_embeddings.grad is not None:                  # the embedding lookup goes through torch autograd
            self.tok_embeddings.main_grad += self.tok_embeddings.grad.float()
            self.tok_embeddings.grad = None
        for p in self.replicated_parameters():
            self.tp.all_reduce(p.main_grad)
        return self.tp.all_reduce(loss.detach().clone())

    @torch.no_grad()
    def gather_into(self, dense: Optional[DenseModel] = None) -> DenseModel:
        """All-gather the shards back into the full DenseModel layout (for checkpoints and evaluation)."""
        dense = dense or self.dense[0]
        cfg, tp, D = self.cfg, self.tp, self.cfg.head_dim
        ag = lambda t: [x for x in self._gather_list(t)]
        dense.tok_embeddings.data.copy_(self.tok_embeddings.data)
        dense.norm.data.copy_(self.norm.data)
        if not self.tied:
            dense.lm_head.data.copy_(self.lm_head.data)
        for src, dst in zip(self.layers, dense.layers):
            nq_l, nkv_l = src.hq * D, src.hkv * D
            parts = ag(src.qkv.data)
            dst.qkv.data.copy_(torch.cat([torch.cat([p[:nq_l] for p in parts]), torch.cat([p[nq_l:nq_l + nkv_l] for p in parts]),
                                          torch.cat([p[nq_l + nkv_l:] for p in parts])], 0))
            dst.o.data.copy_(torch.cat(ag(src.o.data), 1))
            parts = ag(src.gate_up.data)
            if cfg.gated:
                Fl = parts[0].shape[0] // 2
                dst.gate_up.data.copy_(torch.cat([torch.cat([p[:Fl] for p in parts]), torch.cat([p[Fl:] for p in parts])], 0))
            else:
                dst.gate_up.data.copy_(torch.cat(parts, 0))
            dst.down.data.copy_(torch.cat(ag(src.down.data), 1))
            dst.attention_norm.data.copy_(src.attention_norm.data)
            dst.ffn_norm.data.copy_(src.ffn_norm.data)
        return dense

    def _gather_list(self, t):
        if self.tp.world == 1:
            return [t]
        out = [torch.empty_like(t) for _ in range(self.tp.world)]
        dist.all_gather(out, t.contiguous(), group=self.tp.group)
        return out


class TPTrainer:
    """AdamW over this rank's shards and the replicated tensors (fp32 masters), with global-norm clipping over the TP group."""

    def __init__(self, model: TPDenseModel, lr=3e-4, weight_decay=0.01, max_grad_norm=1.0, dp_group=None):
        from ..engines.dense import OptimSuite
        self.model, self.max_grad_norm, self.dp_group = model, max_grad_norm, dp_group
        self.opt = OptimSuite("adamw", lr, weight_decay)
        self.opt.add_group(model.sharded_parameters(), 1.0, 1.0)
        self.opt.add_group(model.replicated_parameters(), 1.0, 0.0)
        self.grad_norm = 0.0

    def train_step(self, ids, labels, lr: Optional[float] = None) -> float:
        m = self.model
        loss = m.forward_backward(ids, labels)
        if self.dp_group is not None and dist.get_world_size(self.dp_group) > 1:
            n = dist.get_world_size(self.dp_group)
            for p in m.parameters():
                dist.all_reduce(p.main_grad, group=self.dp_group)
                p.main_grad.div_(n)
        sq = sum(p.main_grad.pow(2).sum() for p in m.sharded_parameters())
        sq = m.tp.all_reduce(sq.reshape(1).clone())[0] + sum(p.main_grad.pow(2).sum() for p in m.replicated_parameters())
        self.grad_norm = float(sq.sqrt())
        if self.max_grad_norm > 0 and self.grad_norm > self.max_grad_norm:
            for p in m.parameters():
                p.main_grad.mul_(self.max_grad_norm / (self.grad_norm + 1e-6))
        if lr is not None:
            self.opt.set_lr(lr)
        self.opt.step()
        self.opt.zero_grad()
        return float(loss)
