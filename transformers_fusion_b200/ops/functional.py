"""Raw (non-autograd) operators.

Every function dispatches on the device of its first tensor argument: CUDA tensors go to the
sm_100a kernels in ``libtfb_kernels.so``; CPU tensors run the plain PyTorch statement of the same
math, which is both the CPU execution path of the framework and the oracle the GPU tests compare
against.  There is no third path.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import check, ptr, stream

ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2, "silu": 3, "swiglu": 3, "geglu": 2}


def _act_ref(x, act):
    a = ACT[act] if not isinstance(act, int) else act
    if a == 1:
        return torch.relu(x)
    if a == 2:
        return F.gelu(x, approximate="tanh")
    if a == 3:
        return F.silu(x)
    return x


# ---------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------
def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=None, bias=None, residual=None, act=None,
         alpha=1.0, accumulate=False, max_ctas=0):
    """C = act(alpha * A @ B + bias) + residual.

    ``a`` is [M, K] (``a_mn=False``) or stored transposed as [K, M] (``a_mn=True``); ``b`` is the
    weight layout [N, K] (``b_mn=False``) or stored [K, N] (``b_mn=True``).  With
    ``accumulate=True`` (fp32 ``out`` required) the product is added into ``out``.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    Kb = b.shape[0] if b_mn else b.shape[1]
    assert K == Kb, f"reduction dims differ: {K} vs {Kb}"
    if out_dtype is None:
        out_dtype = a.dtype
    if accumulate:
        assert out is not None and out.dtype == torch.float32
        out_dtype = torch.float32
    if not a.is_cuda:
        A = (a.t() if a_mn else a).float()
        B = (b if b_mn else b.t()).float()
        c = alpha * (A @ B)
        if bias is not None:
            c = c + bias.float()
        c = _act_ref(c, act)
        if residual is not None:
            c = c + residual.float()
        if accumulate:
            out.add_(c)
            return out
        if out is not None:
            out.copy_(c.to(out.dtype))
            return out
        return c.to(out_dtype)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    assert out.stride(-1) == 1 and out.shape[0] == M and out.shape[1] == N
    mode = 0 if out.dtype == torch.bfloat16 else (2 if accumulate else 1)
    rc = _lib.lib().tfb_gemm_bf16(a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn),
                                  out.data_ptr(), out.stride(0), M, N, K, ptr(bias), ptr(residual),
                                  residual.stride(0) if residual is not None else 0, float(alpha), ACT[act], mode,
                                  int(max_ctas), _lib.status_word(a.device).data_ptr(), stream())
    check(rc, "gemm_bf16")
    return out


# ---------------------------------------------------------------------------------------------
# normalisation
# ---------------------------------------------------------------------------------------------
def rmsnorm_fwd(x, w, eps, residual=None, want_h=None):
    """Returns (y, h, rstd): h = x + residual (== x when residual is None and want_h is False)."""
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    rows = x2.shape[0]
    if want_h is None:
        want_h = residual is not None
    if not x.is_cuda:
        h = x2.float() + (residual.reshape(-1, H).float() if residual is not None else 0)
        h = h.to(x.dtype)
        hf = h.float()
        rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
        y = (hf * rstd[:, None] * w.float()).to(x.dtype)
        return y.view_as(x), h.view_as(x), rstd
    y = torch.empty_like(x2)
    h = torch.empty_like(x2) if want_h else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    r2 = residual.reshape(-1, H) if residual is not None else None
    check(_lib.lib().tfb_rmsnorm_fwd(x2.data_ptr(), ptr(r2), w.data_ptr(), y.data_ptr(), ptr(h), rstd.data_ptr(), rows,
                                     H, float(eps), stream()), "rmsnorm_fwd")
    return y.view_as(x), (h.view_as(x) if h is not None else x), rstd


def rmsnorm_bwd(dy, h, w, rstd, dw, dres=None):
    """dx = d(rmsnorm)/dh applied to dy, plus dres; accumulates the weight gradient into fp32 ``dw``."""
    H = h.shape[-1]
    dy2, h2 = dy.reshape(-1, H), h.reshape(-1, H)
    rows = h2.shape[0]
    if not h.is_cuda:
        hf, g = h2.float(), dy2.float() * w.float()
        xh = hf * rstd[:, None]
        dw.add_((dy2.float() * xh).sum(0))
        dx = rstd[:, None] * (g - xh * (g * xh).mean(-1, keepdim=True))
        if dres is not None:
            dx = dx + dres.reshape(-1, H).float()
        return dx.to(h.dtype).view_as(h)
    dx = torch.empty_like(h2)
    d2 = dres.reshape(-1, H) if dres is not None else None
    check(_lib.lib().tfb_rmsnorm_bwd(dy2.data_ptr(), h2.data_ptr(), w.data_ptr(), rstd.data_ptr(), ptr(d2),
                                     dx.data_ptr(), dw.data_ptr(), rows, H, stream()), "rmsnorm_bwd")
    return dx.view_as(h)


def layernorm_fwd(x, w, b, eps, residual=None, want_h=None):
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    rows = x2.shape[0]
    if want_h is None:
        want_h = residual is not None
    if not x.is_cuda:
        h = (x2.float() + (residual.reshape(-1, H).float() if residual is not None else 0)).to(x.dtype)
        hf = h.float()
        mean = hf.mean(-1)
        rstd = torch.rsqrt(hf.var(-1, unbiased=False) + eps)
        y = (hf - mean[:, None]) * rstd[:, None] * w.float()
        if b is not None:
            y = y + b.float()
        return y.to(x.dtype).view_as(x), h.view_as(x), rstd, mean
    y = torch.empty_like(x2)
    h = torch.empty_like(x2) if want_h else None
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    r2 = residual.reshape(-1, H) if residual is not None else None
    check(_lib.lib().tfb_layernorm_fwd(x2.data_ptr(), ptr(r2), w.data_ptr(), ptr(b), y.data_ptr(), ptr(h),
                                       rstd.data_ptr(), mean.data_ptr(), rows, H, float(eps), stream()), "layernorm_fwd")
    return y.view_as(x), (h.view_as(x) if h is not None else x), rstd, mean


def layernorm_bwd(dy, h, w, rstd, mean, dw, db, dres=None):
    H = h.shape[-1]
    dy2, h2 = dy.reshape(-1, H), h.reshape(-1, H)
    rows = h2.shape[0]
    if not h.is_cuda:
        xh = (h2.float() - mean[:, None]) * rstd[:, None]
        g = dy2.float() * w.float()
        dw.add_((dy2.float() * xh).sum(0))
        if db is not None:
            db.add_(dy2.float().sum(0))
        dx = rstd[:, None] * (g - xh * (g * xh).mean(-1, keepdim=True) - g.mean(-1, keepdim=True))
        if dres is not None:
            dx = dx + dres.reshape(-1, H).float()
        return dx.to(h.dtype).view_as(h)
    dx = torch.empty_like(h2)
    d2 = dres.reshape(-1, H) if dres is not None else None
    check(_lib.lib().tfb_layernorm_bwd(dy2.data_ptr(), h2.data_ptr(), w.data_ptr(), rstd.data_ptr(), mean.data_ptr(),
                                       ptr(d2), dx.data_ptr(), dw.data_ptr(), ptr(db), rows, H, stream()), "layernorm_bwd")
    return dx.view_as(h)


# ---------------------------------------------------------------------------------------------
# rotary embedding
# ---------------------------------------------------------------------------------------------
def rope_tables(head_dim, max_pos, theta=10000.0, scaling_mode="none", scaling_factor=1.0, original_max=0,
                yarn_attn_factor=1.0, yarn_beta_fast=32.0, yarn_beta_slow=1.0, device="cpu"):
    """cos/sin tables [max_pos, head_dim/2] fp32 for rotate-half RoPE with the reference's scaling modes
    (src/model/transformer.cpp:124-211): none, linear (positions / factor), ntk (theta scaled by
    factor^(d/(d-2))), yarn (per-frequency blend of interpolated and extrapolated frequencies)."""
    half = head_dim // 2
    j = torch.arange(half, dtype=torch.float64)
    mode = (scaling_mode or "none").lower()
    base = float(theta)
    if mode == "ntk" and scaling_factor > 1.0:
        base = base * scaling_factor ** (head_dim / max(head_dim - 2, 1))
    inv = base ** (-2.0 * j / head_dim)
    mscale = 1.0
    if mode == "yarn" and scaling_factor > 1.0:
        orig = float(original_max or max_pos)

        def corr(n_rot):
            return head_dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(theta))
        lo = max(math.floor(corr(yarn_beta_fast)), 0)
        hi = min(math.ceil(corr(yarn_beta_slow)), half - 1)
        ramp = ((j - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        inv = inv / scaling_factor * ramp + inv * (1 - ramp)
        mscale = yarn_attn_factor * (0.1 * math.log(scaling_factor) + 1.0)
    pos = torch.arange(max_pos, dtype=torch.float64)
    if mode == "linear" and scaling_factor > 0:
        pos = pos / scaling_factor
    ang = pos[:, None] * inv[None, :]
    return (ang.cos() * mscale).float().to(device).contiguous(), (ang.sin() * mscale).float().to(device).contiguous()


def rope_(x, cos, sin, n_heads, head_dim, seq_len, pos_offset=0, positions=None, backward=False):
    """In-place rotate-half RoPE on the first ``n_heads`` heads of every row of x [T, ld]."""
    T, ld = x.shape[0], x.stride(0)
    if not x.is_cuda:
        half = head_dim // 2
        if positions is None:
            positions = (torch.arange(T) % seq_len) + pos_offset
        c = cos[positions.long()][:, None, :]
        s = sin[positions.long()][:, None, :] * (-1.0 if backward else 1.0)
        v = x[:, : n_heads * head_dim].reshape(T, n_heads, head_dim).float()
        x1, x2 = v[..., :half], v[..., half:]
        out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
        x[:, : n_heads * head_dim] = out.reshape(T, n_heads * head_dim).to(x.dtype)
        return x
    check(_lib.lib().tfb_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), ptr(positions), T, seq_len, pos_offset,
                              n_heads, head_dim, ld, int(backward), stream()), "rope")
    return x


# ---------------------------------------------------------------------------------------------
# activations
# ---------------------------------------------------------------------------------------------
def glu_fwd(x, act="silu", rows=None):
    """x [M, 2F] = [gate | up] -> act(gate) * up.  ``rows`` (CUDA): a 1-element int32 device tensor; only the first
    ``rows`` rows are computed (the rest of the result is left unwritten)."""
    M, F2 = x.shape
    Fh = F2 // 2
    if not x.is_cuda:
        return (_act_ref(x[:, :Fh].float(), act) * x[:, Fh:].float()).to(x.dtype)
    out = torch.empty((M, Fh), dtype=x.dtype, device=x.device)
    check(_lib.lib().tfb_glu_fwd_rows(x.data_ptr(), out.data_ptr(), M, Fh, ACT[act],
                                      rows.data_ptr() if rows is not None else None, stream()), "glu_fwd")
    return out


def glu_bwd(x, dout, act="silu", rows=None):
    M, F2 = x.shape
    Fh = F2 // 2
    if not x.is_cuda:
        g = x[:, :Fh].float().detach().requires_grad_(True)
        u = x[:, Fh:].float()
        with torch.enable_grad():
            a = _act_ref(g, act)
            (ga,) = torch.autograd.grad(a, g, torch.ones_like(a))
        d = dout.float()
        return torch.cat([d * u * ga, d * a.detach()], 1).to(x.dtype)
    din = torch.empty_like(x)
    check(_lib.lib().tfb_glu_bwd_rows(x.data_ptr(), dout.data_ptr(), din.data_ptr(), M, Fh, ACT[act],
                                      rows.data_ptr() if rows is not None else None, stream()), "glu_bwd")
    return din


def act_fwd(x, act):
    if not x.is_cuda:
        return _act_ref(x.float(), act).to(x.dtype)
    y = torch.empty_like(x)
    check(_lib.lib().tfb_act_fwd(x.data_ptr(), y.data_ptr(), x.numel(), ACT[act], stream()), "act_fwd")
    return y


def act_bwd(x, dy, act):
    if not x.is_cuda:
        xf = x.float().detach().requires_grad_(True)
        with torch.enable_grad():
            a = _act_ref(xf, act)
            (g,) = torch.autograd.grad(a, xf, dy.float())
        return g.to(x.dtype)
    dx = torch.empty_like(x)
    check(_lib.lib().tfb_act_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(), ACT[act], stream()), "act_bwd")
    return dx


# ---------------------------------------------------------------------------------------------
# embedding
# ---------------------------------------------------------------------------------------------
def embedding_fwd(ids, W, pos_table=None, seq_len=0):
    T = ids.numel()
    V, H = W.shape
    if not W.is_cuda:
        out = W[ids.reshape(-1).long()]
        if pos_table is not None:
            out = out + pos_table[(torch.arange(T) % seq_len)]
        return out
    out = torch.empty((T, H), dtype=W.dtype, device=W.device)
    check(_lib.lib().tfb_embedding_fwd(ids.data_ptr(), W.data_ptr(), ptr(pos_table), out.data_ptr(), T, max(seq_len, 1),
                                       H, V, stream()), "embedding_fwd")
    return out


def embedding_bwd(ids, dout, dW, dP=None, seq_len=0):
    """Scatter-add dout rows into the fp32 gradient of the table (and of the position table)."""
    T = ids.numel()
    V, H = dW.shape
    if not dout.is_cuda:
        dW.index_add_(0, ids.reshape(-1).long(), dout.float())
        if dP is not None:
            dP.index_add_(0, torch.arange(T) % seq_len, dout.float())
        return
    check(_lib.lib().tfb_embedding_bwd(ids.data_ptr(), dout.data_ptr(), dW.data_ptr(), ptr(dP), T, max(seq_len, 1), H,
                                       V, stream()), "embedding_bwd")


# ---------------------------------------------------------------------------------------------
# loss / optimiser
# ---------------------------------------------------------------------------------------------
def cross_entropy_fwd_bwd(logits, labels, scale=None, ignore_index=-100, label_smoothing=0.0, z_weight=0.0,
                          want_grad=True):
    """Per-token loss [T] fp32 and, when ``want_grad``, the logit gradient written over ``logits``.

    ``scale`` is a 1-element fp32 tensor on the same device (typically 1 / number of valid tokens)."""
    T, V = logits.shape
    if not logits.is_cuda:
        z = logits.float()
        lse = torch.logsumexp(z, -1)
        valid = labels != ignore_index
        lab = labels.clamp(min=0).long()
        zy = z.gather(1, lab[:, None])[:, 0]
        loss = (1 - label_smoothing) * (lse - zy) + label_smoothing * (lse - z.mean(-1)) + z_weight * lse * lse
        loss = torch.where(valid, loss, torch.zeros_like(loss))
        if want_grad:
            p = torch.softmax(z, -1) * (1 + 2 * z_weight * lse)[:, None]
            p = p - label_smoothing / V
            p.scatter_add_(1, lab[:, None], torch.full((T, 1), -(1 - label_smoothing)))
            s = (scale.float() if scale is not None else torch.ones(())) * valid.float()
            logits.copy_((p * s.reshape(-1, 1)).to(logits.dtype))
        return loss
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    check(_lib.lib().tfb_cross_entropy(logits.data_ptr(), labels.data_ptr(), loss.data_ptr(), None,
                                       logits.data_ptr() if want_grad else None, ptr(scale), T, V, logits.stride(0),
                                       int(ignore_index), float(label_smoothing), float(z_weight), stream()),
          "cross_entropy")
    return loss


def sumsq(x, out):
    """out += sum(x^2) for a flat fp32 tensor."""
    if not x.is_cuda:
        out.add_(x.float().pow(2).sum())
        return out
    check(_lib.lib().tfb_sumsq_f32(x.data_ptr(), x.numel(), out.data_ptr(), stream()), "sumsq")
    return out


def clip_factor(sumsq_t, inv_scale, max_norm, norm_out, clip_out, found_inf=None):
    if not sumsq_t.is_cuda:
        nrm = sumsq_t.sqrt() * inv_scale
        c = torch.tensor(float(inv_scale))
        if not torch.isfinite(nrm):
            c = torch.tensor(0.0)
            if found_inf is not None:
                found_inf.fill_(1)
        elif max_norm > 0 and nrm > max_norm:
            c = c * max_norm / (nrm + 1e-6)
        norm_out.copy_(nrm.reshape(norm_out.shape))
        clip_out.copy_(c.reshape(clip_out.shape))
        return
    check(_lib.lib().tfb_clip_factor(sumsq_t.data_ptr(), float(inv_scale), float(max_norm), norm_out.data_ptr(),
                                     clip_out.data_ptr(), ptr(found_inf), stream()), "clip_factor")


def adamw_(p, g, m, v, p_lp, lr, beta1, beta2, eps, wd, step, gscale=None, zero_grad=True, hyper=None):
    """Fused AdamW over flat fp32 state; refreshes the bf16 copy ``p_lp`` and zeroes ``g``."""
    if not p.is_cuda:
        if hyper is not None:
            lr, bc1, bc2 = (float(x) for x in hyper[:3])
        else:
            bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        gs = gscale.float() if gscale is not None else torch.ones(())
        if gscale is not None and float(gs) == 0.0:
            if zero_grad:
                g.zero_()
            return
        gr = g * gs
        m.mul_(beta1).add_(gr, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gr, gr, value=1 - beta2)
        mh = m / bc1
        vh = v / bc2
        p.sub_(lr * (mh / (vh.sqrt() + eps) + wd * p))
        if zero_grad:
            g.zero_()
        if p_lp is not None:
            p_lp.copy_(p.to(p_lp.dtype))
        return
    check(_lib.lib().tfb_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), ptr(p_lp), p.numel(), float(lr),
                               float(beta1), float(beta2), float(eps), float(wd), int(step), ptr(gscale),
                               int(zero_grad), ptr(hyper), stream()), "adamw")


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------
_lib.register("tfb_attn_fwd", [_lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_p, _lib.c_ll,
                               _lib.c_i, _lib.c_p, _lib.c_ll, _lib.c_p, _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_i,
                               _lib.c_i, _lib.c_f, _lib.c_i, _lib.c_p, _lib.c_p])


_lib.register("tfb_attn_fwd_kv", [_lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_p, _lib.c_ll,
                                  _lib.c_i, _lib.c_p, _lib.c_ll, _lib.c_p, _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_i,
                                  _lib.c_i, _lib.c_f, _lib.c_i, _lib.c_p, _lib.c_p])


def _split_heads(buf, col0, n_heads, D, B, S):
    return buf[:, col0: col0 + n_heads * D].reshape(B, S, n_heads, D).permute(0, 2, 1, 3).float()


def attn_ref(q, k, v, B, S, Hq, Hkv, D, scale, causal, q_col0=0, k_col0=0, v_col0=0, kv_len=None):
    """fp32 reference: returns (o [B*S, Hq*D], lse [B, Hq, S], probabilities).  ``kv_len`` >= S: k / v hold that many
    rows per sequence and the queries are its last S positions."""
    Skv = S if kv_len is None else kv_len
    Q = _split_heads(q, q_col0, Hq, D, B, S)
    K = _split_heads(k, k_col0, Hkv, D, B, Skv).repeat_interleave(Hq // Hkv, 1)
    V = _split_heads(v, v_col0, Hkv, D, B, Skv).repeat_interleave(Hq // Hkv, 1)
    s = (Q @ K.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(torch.ones(S, Skv, dtype=torch.bool, device=s.device).triu(1 + Skv - S), float("-inf"))
    lse = torch.logsumexp(s, -1)
    P = torch.exp(s - lse[..., None])
    o = (P @ V).permute(0, 2, 1, 3).reshape(B * S, Hq * D)
    return o, lse, P


def attn_fwd(q, k, v, B, S, Hq, Hkv, D, scale=None, causal=True, q_col0=0, k_col0=0, v_col0=0, kv_len=None):
    """q/k/v: [B*S, ld] bf16 buffers (may be one fused projection output; see column offsets).
    Returns (o [B*S, Hq*D] bf16, lse [B, Hq, S] fp32).  ``kv_len`` > S: k / v are [B*kv_len, ld] and the S queries are
    the last S positions of each sequence (a prompt suffix attending over a cached prefix and itself)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    Skv = S if kv_len is None else int(kv_len)
    assert Skv >= S
    if not q.is_cuda:
        o, lse, _ = attn_ref(q, k, v, B, S, Hq, Hkv, D, scale, causal, q_col0, k_col0, v_col0, Skv)
        return o.to(q.dtype), lse
    o = torch.empty((B * S, Hq * D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    check(_lib.lib().tfb_attn_fwd_kv(q.data_ptr(), q.stride(0), q_col0, k.data_ptr(), k.stride(0), k_col0, v.data_ptr(),
                                     v.stride(0), v_col0, o.data_ptr(), o.stride(0), lse.data_ptr(), B, S, Skv, Hq, Hkv, D,
                                     float(scale), int(causal), _lib.status_word(q.device).data_ptr(), stream()),
          "attn_fwd")
    return o, lse


_lib.register("tfb_attn_bwd", [_lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_p, _lib.c_ll,
                               _lib.c_i, _lib.c_p, _lib.c_ll, _lib.c_p, _lib.c_ll, _lib.c_p, _lib.c_p,
                               _lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_p, _lib.c_ll,
                               _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_f, _lib.c_i,
                               _lib.c_p, _lib.c_p])


def attn_bwd(q, k, v, o, dout, lse, dqkv, B, S, Hq, Hkv, D, scale=None, causal=True, q_col0=0, k_col0=0, v_col0=0,
             dq_col0=None, dk_col0=None, dv_col0=None):
    """Writes dq / dk / dv into ``dqkv`` ([B*S, ld] bf16) at the given column offsets (defaults: the
    same offsets as q / k / v, i.e. ``dqkv`` mirrors a fused projection output)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    dq_col0 = q_col0 if dq_col0 is None else dq_col0
    dk_col0 = k_col0 if dk_col0 is None else dk_col0
    dv_col0 = v_col0 if dv_col0 is None else dv_col0
    if not q.is_cuda:
        Q = _split_heads(q, q_col0, Hq, D, B, S).requires_grad_(True)
        K = _split_heads(k, k_col0, Hkv, D, B, S).requires_grad_(True)
        V = _split_heads(v, v_col0, Hkv, D, B, S).requires_grad_(True)
        with torch.enable_grad():
            G = Hq // Hkv
            s = (Q @ K.repeat_interleave(G, 1).transpose(-1, -2)) * scale
            if causal:
                s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
            out = (torch.softmax(s, -1) @ V.repeat_interleave(G, 1)).permute(0, 2, 1, 3).reshape(B * S, Hq * D)
            gq, gk, gv = torch.autograd.grad(out, (Q, K, V), dout.float())
        dqkv[:, dq_col0: dq_col0 + Hq * D] = gq.permute(0, 2, 1, 3).reshape(B * S, Hq * D).to(dqkv.dtype)
        dqkv[:, dk_col0: dk_col0 + Hkv * D] = gk.permute(0, 2, 1, 3).reshape(B * S, Hkv * D).to(dqkv.dtype)
        dqkv[:, dv_col0: dv_col0 + Hkv * D] = gv.permute(0, 2, 1, 3).reshape(B * S, Hkv * D).to(dqkv.dtype)
        return dqkv
    delta = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    dp, ldd = dqkv.data_ptr(), dqkv.stride(0)
    check(_lib.lib().tfb_attn_bwd(q.data_ptr(), q.stride(0), q_col0, k.data_ptr(), k.stride(0), k_col0, v.data_ptr(),
                                  v.stride(0), v_col0, o.data_ptr(), o.stride(0), dout.data_ptr(), dout.stride(0),
                                  lse.data_ptr(), delta.data_ptr(), dp, ldd, dq_col0, dp, ldd, dk_col0, dp, ldd,
                                  dv_col0, B, S, Hq, Hkv, D, float(scale), int(causal),
                                  _lib.status_word(q.device).data_ptr(), stream()), "attn_bwd")
    return dqkv
