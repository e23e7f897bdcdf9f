"""Dense decoder-only transformer (Llama-style: RMSNorm, rotate-half RoPE, GQA, gated or plain
FFN, optional parallel residual; plus the GPT-2-shaped variant with LayerNorm, learned positions
and biases).

The training path is written as explicit forward and backward passes over the sm_100a kernels
(one autograd node per transformer block rather than one per op): the activations that the
backward needs are saved by hand, weight gradients are accumulated by the GEMM epilogue straight
into each parameter's fp32 ``main_grad`` slice of the flat gradient buffer, and the residual adds
ride in GEMM epilogues.  The same code runs on CPU tensors through the PyTorch statement of each op.

Parity: DenseModel / TransformerBlock / Attention / FFN of the reference
(src/model/model.cpp:33-132, src/model/transformer.cpp:273-627); tensor names follow
src/model/model.cpp:138-166 so ``.quant`` checkpoints interchange.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as F
from .config import TransformerConfig


# =================================================================================================
# flat parameter storage
# =================================================================================================
class RotaryEmbedding:
    """Rotary position embedding as an object: the cos / sin tables of a head size (with the linear, NTK and YaRN context
    scalings) and their application to [T, heads * head_dim] rows, in place, through the RoPE kernel.  The models keep
    their tables themselves (``DenseModel.rope``); this class is the stand-alone form (reference: RotaryEmbedding,
    src/model/transformer.cpp:124-270)."""

    def __init__(self, head_dim: int, max_seq_len: int, theta: float = 10000.0, scaling_mode: str = "none",
                 scaling_factor: float = 1.0, original_max_seq_len: int = 0, device="cpu", **yarn):
        self.head_dim, self.max_seq_len = head_dim, max_seq_len
        self.cos, self.sin = F.rope_tables(head_dim, max_seq_len, theta, scaling_mode, scaling_factor, original_max_seq_len,
                                           device=device, **yarn)

    @classmethod
    def from_config(cls, cfg: TransformerConfig, device="cpu"):
        return cls(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta, cfg.rope_scaling_mode, cfg.rope_scaling_factor,
                   cfg.rope_original_max_seq_len, device=device, yarn_attn_factor=cfg.yarn_attn_factor,
                   yarn_beta_fast=cfg.yarn_beta_fast, yarn_beta_slow=cfg.yarn_beta_slow)

    def apply_(self, x, n_heads: int, seq_len: int, pos_offset: int = 0, positions=None, inverse: bool = False):
        """Rotate the first ``n_heads`` heads of every row of x [T, ld] in place (``inverse`` undoes it: the backward)."""
        return F.rope_(x, self.cos, self.sin, n_heads, self.head_dim, seq_len, pos_offset, positions, backward=inverse)

    def __call__(self, x, n_heads: int, seq_len: int, pos_offset: int = 0):
        return self.apply_(x.clone(), n_heads, seq_len, pos_offset)

    def apply(self, x: torch.Tensor, seq_start: int, seq_len: int) -> torch.Tensor:
        """The reference's form (include/quant/transformer.h:93): x [batch, heads, seq_len, head_dim] (or [heads, seq_len,
        head_dim]) is rotated in place for positions seq_start .. seq_start + seq_len - 1 and returned."""
        D = self.head_dim
        lead = x.shape[:-2]
        assert x.shape[-1] == D and x.shape[-2] == seq_len
        flat = x.reshape(-1, seq_len, D)                                   # [B * heads, S, D]: one "head" per row block
        rows = flat.reshape(-1, D).contiguous()                            # [(B * heads) * S, D], positions cycle every S rows
        F.rope_(rows, self.cos, self.sin, 1, D, seq_len, seq_start)
        x.copy_(rows.view(*lead, seq_len, D))
        return x

    def attn_scale_mult(self) -> float:
        """The factor YaRN scaling puts on the attention logits' inputs (it is already folded into the cos / sin tables
        here, so q and k each carry it once); 1 for the other modes."""
        return float(self.cos[0, 0])                                       # cos(0) * mscale


class FlatBuffers:
    """Contiguous parameter / gradient storage.

    ``params``  bf16 (compute dtype) flat buffer that every nn.Parameter of the model is a view of;
    ``grads``   fp32 flat gradient buffer; every parameter gets ``p.main_grad`` = its fp32 slice.
    Each tensor starts on a 128-element boundary so slices stay 256-byte aligned (TMA needs 16).
    Shard-friendly: ZeRO / FSDP split these buffers by contiguous element ranges.
    """

    ALIGN = 128

    def __init__(self, module: nn.Module, dtype=torch.bfloat16, pad_to: int = 1, allocator=None):
        """``allocator(numel, dtype)`` returns an object with ``.view(dtype, numel)`` (the symmetric
        heap's ``alloc``) when the buffers must be visible to peer GPUs; default: plain torch tensors."""
        seen, params = set(), []
        for p in module.parameters():
            if id(p) not in seen:
                seen.add(id(p))
                params.append(p)
        self.params_list = params
        offs, n = [], 0
        for p in params:
            offs.append(n)
            n += (p.numel() + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        n = (n + pad_to - 1) // pad_to * pad_to
        dev = params[0].device if params else torch.device("cpu")
        self.numel = n
        self.offsets = offs
        self.symm_params = self.symm_grads = None
        if allocator is not None:
            self.symm_params = allocator(n, dtype)
            self.symm_grads = allocator(n, torch.float32)
            self.params = self.symm_params.view(dtype, n)
            self.grads = self.symm_grads.view(torch.float32, n)
            self.params.zero_()
            self.grads.zero_()
        else:
            self.params = torch.zeros(n, dtype=dtype, device=dev)
            self.grads = torch.zeros(n, dtype=torch.float32, device=dev)
        for p, o in zip(params, offs):
            view = self.params[o: o + p.numel()].view(p.shape)
            view.copy_(p.data.to(dtype))
            p.data = view
            p.main_grad = self.grads[o: o + p.numel()].view(p.shape)

    def zero_grad(self):
        self.grads.zero_()


# =================================================================================================
# per-block forward / backward
# =================================================================================================
def _norm_fwd(cfg, x, w, b):
    if cfg.norm_type == "layernorm":
        y, _, rstd, mean = F.layernorm_fwd(x, w, b, cfg.norm_eps)
        return y, (rstd, mean)
    y, _, rstd = F.rmsnorm_fwd(x, w, cfg.norm_eps)
    return y, (rstd, None)


def _norm_bwd(cfg, dy, h, w, b, stats, dres):
    rstd, mean = stats
    if cfg.norm_type == "layernorm":
        return F.layernorm_bwd(dy, h, w, rstd, mean, w.main_grad, b.main_grad if b is not None else None, dres)
    return F.rmsnorm_bwd(dy, h, w, rstd, w.main_grad, dres)


def _bias_grad(bias, dy):
    if bias is not None:
        bias.main_grad.add_(dy.float().sum(0))


class BlockCtx:
    """Activations one block keeps for its backward pass."""
    __slots__ = ("h_in", "st1", "a", "qkv", "o", "lse", "h_mid", "st2", "f", "gu", "act", "B", "S")


def block_forward(cfg: TransformerConfig, w, h_in, B, S, rope, save: bool):
    """One transformer block on the flattened token stream h_in [T, H].  Returns (h_out, ctx)."""
    Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    ctx = BlockCtx() if save else None
    a, st1 = _norm_fwd(cfg, h_in, w.attention_norm, w.attention_norm_bias)
    qkv = F.gemm(a, w.qkv, bias=w.qkv_bias)
    if rope is not None:
        F.rope_(qkv, rope[0], rope[1], Hq + Hkv, D, S)
    o, lse = F.attn_fwd(qkv, qkv, qkv, B, S, Hq, Hkv, D, k_col0=Hq * D, v_col0=(Hq + Hkv) * D)
    if cfg.use_parallel_residual:
        # h_out = h_in + attn(norm1(h_in)) + ffn(norm2(h_in))
        h_mid = h_in
        attn_out = F.gemm(o, w.o, bias=w.o_bias)
        f, st2 = _norm_fwd(cfg, h_in, w.ffn_norm, w.ffn_norm_bias)
    else:
        h_mid = F.gemm(o, w.o, bias=w.o_bias, residual=h_in)
        f, st2 = _norm_fwd(cfg, h_mid, w.ffn_norm, w.ffn_norm_bias)
    gu = F.gemm(f, w.gate_up, bias=w.gate_up_bias)
    act = F.glu_fwd(gu, cfg.act_kernel) if cfg.gated else F.act_fwd(gu, cfg.act_kernel)
    h_out = F.gemm(act, w.down, bias=w.down_bias, residual=h_mid)
    if cfg.use_parallel_residual:
        h_out = h_out + attn_out if not h_out.is_cuda else _add(h_out, attn_out)
    if save:
        ctx.h_in, ctx.st1, ctx.a, ctx.qkv, ctx.o, ctx.lse = h_in, st1, a, qkv, o, lse
        ctx.h_mid, ctx.st2, ctx.f, ctx.gu, ctx.act, ctx.B, ctx.S = h_mid, st2, f, gu, act, B, S
    return h_out, ctx


def _add(a, b):
    from ..ops import _lib
    out = torch.empty_like(a)
    _lib.check(_lib.lib().tfb_add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _lib.stream()), "add")
    return out


def block_backward(cfg: TransformerConfig, w, ctx: BlockCtx, dh_out, rope):
    """Backward of block_forward.  Accumulates every weight gradient into ``main_grad``; returns dh_in."""
    Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    B, S = ctx.B, ctx.S
    # ---- FFN ----
    d_act = F.gemm(dh_out, w.down, b_mn=True)
    F.gemm(dh_out, ctx.act, a_mn=True, b_mn=True, out=w.down.main_grad, accumulate=True)
    _bias_grad(w.down_bias, dh_out)
    d_gu = F.glu_bwd(ctx.gu, d_act, cfg.act_kernel) if cfg.gated else F.act_bwd(ctx.gu, d_act, cfg.act_kernel)
    d_f = F.gemm(d_gu, w.gate_up, b_mn=True)
    F.gemm(d_gu, ctx.f, a_mn=True, b_mn=True, out=w.gate_up.main_grad, accumulate=True)
    _bias_grad(w.gate_up_bias, d_gu)
    if cfg.use_parallel_residual:
        dh_mid = dh_out                       # attention branch sees dh_out directly
        d_h_ffn = _norm_bwd(cfg, d_f, ctx.h_in, w.ffn_norm, w.ffn_norm_bias, ctx.st2, dh_out)
    else:
        dh_mid = _norm_bwd(cfg, d_f, ctx.h_mid, w.ffn_norm, w.ffn_norm_bias, ctx.st2, dh_out)
        d_h_ffn = None
    # ---- attention ----
    d_o = F.gemm(dh_mid, w.o, b_mn=True)
    F.gemm(dh_mid, ctx.o, a_mn=True, b_mn=True, out=w.o.main_grad, accumulate=True)
    _bias_grad(w.o_bias, dh_mid)
    d_qkv = torch.empty_like(ctx.qkv)
    F.attn_bwd(ctx.qkv, ctx.qkv, ctx.qkv, ctx.o, d_o, ctx.lse, d_qkv, B, S, Hq, Hkv, D, k_col0=Hq * D,
               v_col0=(Hq + Hkv) * D)
    if rope is not None:
        F.rope_(d_qkv, rope[0], rope[1], Hq + Hkv, D, S, backward=True)
    d_a = F.gemm(d_qkv, w.qkv, b_mn=True)
    F.gemm(d_qkv, ctx.a, a_mn=True, b_mn=True, out=w.qkv.main_grad, accumulate=True)
    _bias_grad(w.qkv_bias, d_qkv)
    dres = d_h_ffn if cfg.use_parallel_residual else dh_mid
    return _norm_bwd(cfg, d_a, ctx.h_in, w.attention_norm, w.attention_norm_bias, ctx.st1, dres)


class _BlockFn(torch.autograd.Function):
    """Autograd node for a whole block (used when the model is driven by torch autograd)."""

    @staticmethod
    def forward(ctx, h_in, blk, B, S, rope, recompute, *params):
        need = any(ctx.needs_input_grad)
        h_out, bctx = block_forward(blk.cfg, blk, h_in, B, S, rope, save=need and not recompute)
        ctx.blk, ctx.bctx, ctx.rope, ctx.recompute = blk, bctx, rope, recompute
        if recompute:
            ctx.saved_h, ctx.BS = h_in, (B, S)
        return h_out

    @staticmethod
    def backward(ctx, dh_out):
        blk = ctx.blk
        bctx = ctx.bctx
        for prm in blk.parameters():
            _ensure_main_grad(prm)
        if ctx.recompute:  # activation checkpointing: rebuild the block's activations from its input
            _, bctx = block_forward(blk.cfg, blk, ctx.saved_h, ctx.BS[0], ctx.BS[1], ctx.rope, save=True)
        dh_in = block_backward(blk.cfg, blk, bctx, dh_out.contiguous(), ctx.rope)
        ctx.bctx = None
        return (dh_in, None, None, None, None, None) + (None,) * len(list(blk.parameters()))


# =================================================================================================
# modules
# =================================================================================================
class DenseBlock(nn.Module):
    """Parameters of one block.  q/k/v and gate/up are stored fused ([out, in], rows concatenated);
    the reference tensor names are exposed as row-slice views by DenseModel.named_tensors()."""

    def __init__(self, cfg: TransformerConfig, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        H, F_, D = cfg.hidden_size, cfg.ffn_hidden_size, cfg.head_dim
        nq, nkv = cfg.num_heads * D, cfg.num_kv_heads * D
        kw = dict(device=device, dtype=dtype)
        ln = cfg.norm_type == "layernorm"
        self.attention_norm = nn.Parameter(torch.ones(H, **kw))
        self.attention_norm_bias = nn.Parameter(torch.zeros(H, **kw)) if ln else None
        self.qkv = nn.Parameter(torch.empty(nq + 2 * nkv, H, **kw))
        self.qkv_bias = nn.Parameter(torch.zeros(nq + 2 * nkv, **kw)) if cfg.attention_bias else None
        self.o = nn.Parameter(torch.empty(H, nq, **kw))
        self.o_bias = nn.Parameter(torch.zeros(H, **kw)) if cfg.attention_bias else None
        self.ffn_norm = nn.Parameter(torch.ones(H, **kw))
        self.ffn_norm_bias = nn.Parameter(torch.zeros(H, **kw)) if ln else None
        self.gate_up = nn.Parameter(torch.empty((2 if cfg.gated else 1) * F_, H, **kw))
        self.gate_up_bias = nn.Parameter(torch.zeros((2 if cfg.gated else 1) * F_, **kw)) if cfg.attention_bias else None
        self.down = nn.Parameter(torch.empty(H, F_, **kw))
        self.down_bias = nn.Parameter(torch.zeros(H, **kw)) if cfg.attention_bias else None


class DenseModel(nn.Module):
    """Decoder-only language model.

    ``forward(ids)`` returns logits [B, S, V] through torch autograd (block-level nodes);
    ``forward_backward(ids, labels)`` is the fused training step used by the trainers: it runs
    forward, the chunked LM-head + cross-entropy, and backward by hand, leaves gradients in
    ``main_grad`` and returns the mean loss (a device scalar, no host sync).
    """

    def __init__(self, cfg: TransformerConfig, device=None, dtype=torch.bfloat16, seed: Optional[int] = 0):
        super().__init__()
        self.cfg = cfg
        H, V = cfg.hidden_size, cfg.vocab_size
        kw = dict(device=device, dtype=dtype)
        self.tok_embeddings = nn.Parameter(torch.empty(V, H, **kw))
        self.pos_embeddings = nn.Parameter(torch.empty(cfg.max_seq_len, H, **kw)) if cfg.position_type == "learned" else None
        self.layers = nn.ModuleList([DenseBlock(cfg, device, dtype) for _ in range(cfg.num_layers)])
        self.norm = nn.Parameter(torch.ones(H, **kw))
        self.norm_bias = nn.Parameter(torch.zeros(H, **kw)) if cfg.norm_type == "layernorm" else None
        self.lm_head = self.tok_embeddings if cfg.tie_embeddings else nn.Parameter(torch.empty(V, H, **kw))
        self.mtp_heads = nn.ParameterList([nn.Parameter(torch.empty(V, H, **kw)) for _ in range(cfg.mtp_num_heads)])
        self.activation_checkpointing = False
        self.loss_chunk_tokens = 9472   # 74 row tiles x 2 column tiles (H=512, 256-wide) = one wave of 148 SMs in the dgrad GEMM
        self._rope = None
        self.flat: Optional[FlatBuffers] = None
        if seed is not None:
            self.init_weights(seed)

    # ------------------------------------------------------------------ init / storage
    def init_weights(self, seed: int = 0):
        """N(0, init_std) for matrices (the BASELINE configs' rule), ones/zeros for norms and biases."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2:
                    p.copy_((torch.randn(p.shape, generator=g) * self.cfg.init_std).to(p.dtype))

    def flatten(self, pad_to: int = 1) -> FlatBuffers:
        """Move all parameters into one flat buffer and attach fp32 ``main_grad`` views."""
        if self.flat is None:
            self.flat = FlatBuffers(self, dtype=self.tok_embeddings.dtype, pad_to=pad_to)
        return self.flat

    def rope(self, device):
        cfg = self.cfg
        if cfg.position_type != "rope":
            return None
        if self._rope is None or self._rope[0].device != device:
            self._rope = F.rope_tables(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta, cfg.rope_scaling_mode,
                                       cfg.rope_scaling_factor, cfg.rope_original_max_seq_len, cfg.yarn_attn_factor,
                                       cfg.yarn_beta_fast, cfg.yarn_beta_slow, device=device)
        return self._rope

    def named_tensors(self):
        """(reference tensor name, tensor view) pairs in the reference's save order (model.cpp:138-166)."""
        cfg = self.cfg
        D = cfg.head_dim
        nq, nkv, Fh = cfg.num_heads * D, cfg.num_kv_heads * D, cfg.ffn_hidden_size
        out = [("tok_embeddings.weight", self.tok_embeddings.data)]
        if self.pos_embeddings is not None:
            out.append(("pos_embeddings.weight", self.pos_embeddings.data))
        for i, l in enumerate(self.layers):
            pre = f"layers.{i}."
            out.append((pre + "attention_norm.weight", l.attention_norm.data))
            if l.attention_norm_bias is not None:
                out.append((pre + "attention_norm.bias", l.attention_norm_bias.data))
            out.append((pre + "ffn_norm.weight", l.ffn_norm.data))
            if l.ffn_norm_bias is not None:
                out.append((pre + "ffn_norm.bias", l.ffn_norm_bias.data))
            out.append((pre + "attention.q_proj.weight", l.qkv.data[:nq]))
            out.append((pre + "attention.k_proj.weight", l.qkv.data[nq: nq + nkv]))
            out.append((pre + "attention.v_proj.weight", l.qkv.data[nq + nkv:]))
            out.append((pre + "attention.o_proj.weight", l.o.data))
            if l.qkv_bias is not None:
                out.append((pre + "attention.q_proj.bias", l.qkv_bias.data[:nq]))
                out.append((pre + "attention.k_proj.bias", l.qkv_bias.data[nq: nq + nkv]))
                out.append((pre + "attention.v_proj.bias", l.qkv_bias.data[nq + nkv:]))
                out.append((pre + "attention.o_proj.bias", l.o_bias.data))
            if cfg.gated:
                out.append((pre + "ffn.gate_proj.weight", l.gate_up.data[:Fh]))
                out.append((pre + "ffn.up_proj.weight", l.gate_up.data[Fh:]))
            else:
                out.append((pre + "ffn.up_proj.weight", l.gate_up.data))
            out.append((pre + "ffn.down_proj.weight", l.down.data))
            if l.gate_up_bias is not None:
                out.append((pre + "ffn.up_proj.bias", l.gate_up_bias.data))
                out.append((pre + "ffn.down_proj.bias", l.down_bias.data))
        out.append(("norm.weight", self.norm.data))
        if self.norm_bias is not None:
            out.append(("norm.bias", self.norm_bias.data))
        if not cfg.tie_embeddings:
            out.append(("lm_head.weight", self.lm_head.data))
        for i, m in enumerate(self.mtp_heads):
            out.append((f"mtp_heads.{i}.weight", m.data))
        return out

    # ------------------------------------------------------------------ multi-token prediction heads
    def mtp_shifted_labels(self, labels, ignore_index: int = -100):
        """Targets of the extra heads: head k (0-based) sees labels moved k + 1 further to the left; the tail of every
        sequence, which has no such token, is ignored.  Returns one flattened [B * S] vector per head."""
        out = []
        for k in range(len(self.mtp_heads)):
            sh = torch.full_like(labels, ignore_index)
            if labels.shape[1] > k + 1:
                sh[:, :-(k + 1)] = labels[:, k + 1:]
            out.append(sh.reshape(-1))
        return out

    def mtp_forward(self, ids):
        """Logits of the extra prediction heads, one [B, S, V] tensor per head (reference: DenseModel::mtp_forward,
        src/model/model.cpp).  Empty when the model has no such heads."""
        B, S = ids.shape
        f = self.hidden_states(ids)
        return [_LinearFn.apply(f, w).view(B, S, -1) for w in self.mtp_heads]

    # ------------------------------------------------------------------ accessors (reference: include/quant/model.h:28-65)
    def get_parameters(self):
        return list(self.parameters())

    def param_count(self) -> int:
        """Distinct parameters (a tied embedding / head counts once)."""
        return sum(p.numel() for p in self.parameters())

    def vocab_size(self) -> int:
        return self.cfg.vocab_size

    def mtp_loss(self, ids, labels, ignore_index: int = -100) -> float:
        """Mean over the extra heads of the cross entropy against the labels moved further left (evaluation; the training
        step folds the same term into its loss when ``mtp_loss_weight`` > 0)."""
        with torch.no_grad():
            heads = self.mtp_forward(ids)
        if not heads:
            return 0.0
        tot = 0.0
        for lg, lab in zip(heads, self.mtp_shifted_labels(labels, ignore_index)):
            tot += float(torch.nn.functional.cross_entropy(lg.float().reshape(-1, lg.shape[-1]), lab, ignore_index=ignore_index))
        return tot / len(heads)

    # ------------------------------------------------------------------ files (reference: DenseModel::save / save_quantized / load)
    def save(self, path, fmt="Q_32"):
        """Write the model as a ``.quant`` container (raw fp32 blocks by default)."""
        from ..quant import codec
        codec.save_model(self, path, fmt)
        return path

    def save_quantized(self, path, fmt="Q_8", per_layer=None):
        """Write the model with its matrices in a block format (``Q_8`` / ``Q_4`` / ``Q_2`` in the reference, any registry
        name here); ``per_layer`` maps tensor-name prefixes to formats."""
        from ..quant import codec
        codec.save_model(self, path, fmt, per_layer)
        return path

    @classmethod
    def load(cls, path, device="cpu", dtype=torch.float32, strict=True):
        """Read a ``.quant`` container into a new model of this class."""
        from ..quant import codec
        return codec.load_model(path, device=device, dtype=dtype, model_cls=cls, strict=strict)

    # ------------------------------------------------------------------ autograd path
    def embed(self, ids):
        B, S = ids.shape
        return F.embedding_fwd(ids.reshape(-1), self.tok_embeddings.data,
                               self.pos_embeddings.data if self.pos_embeddings is not None else None, S)

    def hidden_states(self, ids):
        """Final-norm hidden states [T, H] with torch autograd attached (block-level nodes)."""
        B, S = ids.shape
        rope = self.rope(ids.device)
        h = _EmbedFn.apply(ids, self, self.tok_embeddings)
        for blk in self.layers:
            h = _BlockFn.apply(h, blk, B, S, rope, self.activation_checkpointing, *blk.parameters())
        return _FinalNormFn.apply(h, self, self.norm)

    def forward(self, ids):
        B, S = ids.shape
        f = self.hidden_states(ids)
        logits = _LinearFn.apply(f, self.lm_head)
        return logits.view(B, S, -1)

    @torch.no_grad()
    def head_loss_backward(self, h, lab_f, loss_scale: float = 1.0, ignore_index: int = -100, label_smoothing: float = 0.0,
                           n_valid=None, mtp_labels=None, mtp_weight: float = 0.0):
        """Final norm + chunked LM head + cross entropy on hidden states h [T, H]; accumulates the head's weight
        gradients and returns (mean loss, d loss / d h).  ``n_valid`` overrides the token count the loss is
        averaged over (pipeline micro-batches divide by the whole batch's count).  ``mtp_labels`` (one [T] label vector
        per multi-token-prediction head, already shifted) adds ``mtp_weight`` x the mean of the heads' cross entropies."""
        cfg = self.cfg
        T = h.shape[0]
        f, st = _norm_fwd(cfg, h, self.norm, self.norm_bias)
        # ---- chunked LM head + cross entropy: only one chunk of logits exists at a time ----
        if n_valid is None:
            n_valid = (lab_f != ignore_index).sum().clamp(min=1).float()
        scale = (loss_scale / n_valid).reshape(1)
        d_f = torch.empty_like(f)
        losses = torch.empty(T, dtype=torch.float32, device=f.device)
        W = self.lm_head
        ck = max(128, min(self.loss_chunk_tokens, T))
        for t0 in range(0, T, ck):
            t1 = min(T, t0 + ck)
            logits = F.gemm(f[t0:t1], W.data)
            losses[t0:t1] = F.cross_entropy_fwd_bwd(logits, lab_f[t0:t1], scale, ignore_index, label_smoothing)
            F.gemm(logits, W.data, b_mn=True, out=d_f[t0:t1])
            F.gemm(logits, f[t0:t1], a_mn=True, b_mn=True, out=W.main_grad, accumulate=True)
        loss = losses.sum() / n_valid
        if mtp_labels and mtp_weight > 0:
            # head k predicts the token k + 2 positions ahead from the same normed hidden state
            # (reference: Trainer::mtp_loss, src/trainer/trainer_core.cpp:1098-1125; tails are ignored here, not zero-labelled)
            nh = len(mtp_labels)
            for Wk, lab_k in zip(self.mtp_heads, mtp_labels):
                _ensure_main_grad(Wk)
                nv = (lab_k != ignore_index).sum().clamp(min=1).float()
                sk = (loss_scale * mtp_weight / nh / nv).reshape(1)
                for t0 in range(0, T, ck):
                    t1 = min(T, t0 + ck)
                    logits = F.gemm(f[t0:t1], Wk.data)
                    lk = F.cross_entropy_fwd_bwd(logits, lab_k[t0:t1], sk, ignore_index, label_smoothing)
                    loss = loss + lk.sum() * (mtp_weight / nh) / nv
                    F.gemm(logits, Wk.data, b_mn=True, out=d_f[t0:t1], accumulate=True)
                    F.gemm(logits, f[t0:t1], a_mn=True, b_mn=True, out=Wk.main_grad, accumulate=True)
        dh = _norm_bwd(cfg, d_f, h, self.norm, self.norm_bias, st, None)
        return loss, dh

    # ------------------------------------------------------------------ fused training step
    @torch.no_grad()
    def forward_backward(self, ids, labels, loss_scale: float = 1.0, ignore_index: int = -100,
                         label_smoothing: Optional[float] = None):
        """Forward + backward of the next-token loss.  ``labels`` are already aligned with ``ids``
        (labels[b, s] is the target for position s).  Returns the mean loss as a device scalar."""
        assert self.flat is not None, "call model.flatten() before training"
        if label_smoothing is None:
            label_smoothing = getattr(self, "loss_label_smoothing", 0.0)
        cfg = self.cfg
        B, S = ids.shape
        T = B * S
        rope = self.rope(ids.device)
        ids_f, lab_f = ids.reshape(-1), labels.reshape(-1)
        h = self.embed(ids)
        ckpt = self.activation_checkpointing
        ctxs, inputs = [], []
        for blk in self.layers:
            inputs.append(h)
            h, c = block_forward(cfg, blk, h, B, S, rope, save=not ckpt)
            ctxs.append(c)
        mtp_w = float(getattr(self, "mtp_loss_weight", cfg.mtp_loss_weight) or 0.0)
        mtp_labels = self.mtp_shifted_labels(labels, ignore_index) if (mtp_w > 0 and len(self.mtp_heads)) else None
        loss, dh = self.head_loss_backward(h, lab_f, loss_scale, ignore_index, label_smoothing,
                                           mtp_labels=mtp_labels, mtp_weight=mtp_w)
        for i in range(cfg.num_layers - 1, -1, -1):
            c = ctxs[i]
            if ckpt:
                _, c = block_forward(cfg, self.layers[i], inputs[i], B, S, rope, save=True)
            dh = block_backward(cfg, self.layers[i], c, dh, rope)
            ctxs[i] = None
        F.embedding_bwd(ids_f, dh, self.tok_embeddings.main_grad,
                        self.pos_embeddings.main_grad if self.pos_embeddings is not None else None, S)
        return loss


# =================================================================================================
# small autograd nodes used by the generic path
# =================================================================================================
class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, model, table):
        ctx.model, ctx.ids = model, ids
        return model.embed(ids)

    @staticmethod
    def backward(ctx, dh):
        m = ctx.model
        _ensure_main_grad(m.tok_embeddings)
        if m.pos_embeddings is not None:
            _ensure_main_grad(m.pos_embeddings)
        F.embedding_bwd(ctx.ids.reshape(-1), dh.contiguous(), m.tok_embeddings.main_grad,
                        m.pos_embeddings.main_grad if m.pos_embeddings is not None else None, ctx.ids.shape[1])
        return None, None, None


class _FinalNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, model, w):
        y, st = _norm_fwd(model.cfg, h, model.norm, model.norm_bias)
        ctx.model, ctx.h, ctx.st = model, h, st
        return y

    @staticmethod
    def backward(ctx, dy):
        m = ctx.model
        return _norm_bwd(m.cfg, dy.contiguous(), ctx.h, m.norm, m.norm_bias, ctx.st, None), None, None


class _LinearFn(torch.autograd.Function):
    """y = x W^T with the weight gradient accumulated into W.main_grad."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x)
        ctx.w = w
        return F.gemm(x, w.data)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        w = ctx.w
        dy = dy.contiguous()
        _ensure_main_grad(w)
        F.gemm(dy, x, a_mn=True, b_mn=True, out=w.main_grad, accumulate=True)
        return F.gemm(dy, w.data, b_mn=True), None


def _ensure_main_grad(p):
    if not hasattr(p, "main_grad") or p.main_grad is None:
        p.main_grad = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
