"""Mixture-of-experts operators: router soft-max + top-k, expert segment planning, token permutation,
grouped expert GEMMs, weighted combine — each with its backward — as one autograd function
(``moe_ffn``) whose data path never leaves the device and never synchronises with the host: the
permuted buffers are sized for the worst case (T*k rows + 128 of padding per expert) and the grouped
GEMMs skip tiles that belong to no expert.

CPU tensors run the PyTorch statement of the same math (also the oracle of the GPU tests).

Reference counterparts: moe::softmax_with_topk / load-balance loss / moe_dispatch_batched
(src/model/moe_core.cpp:98-344), route_topk renormalised (engines/trainer/moe/moe.cpp:54-94),
moe_gather / moe_scatter kernels (src/backend/gpu_compute_cuda.cpp:539-616).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib, functional as F
from ._lib import c_f, c_i, c_ll, c_p, check, ptr, stream

_lib.register("tfb_router_topk", [c_p, c_i, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_p, c_p, c_p])
_lib.register("tfb_router_topk2", [c_p, c_i, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p])
_lib.register("tfb_moe_permute2", [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p])
_lib.register("tfb_moe_zero_pads", [c_p, c_i, c_p, c_p, c_i, c_p, c_i, c_p])
_lib.register("tfb_moe_plan", [c_p, c_i, c_p, c_p, c_p, c_i, c_p, c_p])
_lib.register("tfb_moe_permute", [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p])
_lib.register("tfb_moe_combine", [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p])
_lib.register("tfb_moe_combine_bwd", [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_p])
_lib.register("tfb_moe_permute_bwd", [c_p, c_p, c_p, c_i, c_i, c_i, c_p])


class _Group(C.Structure):
    _fields_ = [("mode", C.c_int), ("num_experts", C.c_int), ("expert_of_mtile", C.c_void_p),
                ("seg_start", C.c_void_p), ("b_expert_stride", C.c_longlong), ("c_expert_stride", C.c_longlong)]


def _grouped_fn():
    fn = _lib.lib().tfb_gemm_bf16_grouped
    fn.argtypes = [c_p, c_ll, c_i, c_p, c_ll, c_i, c_p, c_ll, c_i, c_i, c_i, c_f, c_i, C.POINTER(_Group), c_p, c_p]
    fn.restype = c_i
    return fn


# ---------------------------------------------------------------------------------------------
# routing
# ---------------------------------------------------------------------------------------------
def router_topk(logits, k, renormalize=True):
    """logits [T, E] -> (idx int32 [T,k], w fp32 [T,k], probs fp32 [T,E], counts int32 [E], lse fp32 [T])."""
    return router_topk_stats(logits, k, renormalize)[:5]


def router_topk_stats(logits, k, renormalize=True):
    """router_topk plus the two reductions the auxiliary losses need, produced by the same kernel:
    prob_sums fp32 [E] = sum_t probs[t, e] and lse_sq fp32 [1] = sum_t lse_t^2."""
    T, E = logits.shape
    if not logits.is_cuda:
        z = logits.float()
        probs = torch.softmax(z, -1)
        w, idx = torch.topk(probs, k, dim=-1)
        if renormalize:
            w = w / w.sum(-1, keepdim=True)
        counts = torch.bincount(idx.reshape(-1), minlength=E).int()
        lse = torch.logsumexp(z, -1)
        return idx.int(), w, probs, counts, lse, probs.sum(0), (lse * lse).sum().reshape(1)
    dev = logits.device
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    w = torch.empty((T, k), dtype=torch.float32, device=dev)
    probs = torch.empty((T, E), dtype=torch.float32, device=dev)
    red = torch.zeros(2 * E + 1, dtype=torch.float32, device=dev)        # [counts as int32 | prob_sums | lse_sq], one fill
    counts, prob_sums, lse_sq = red[:E].view(torch.int32), red[E:2 * E], red[2 * E:]
    lse = torch.empty(T, dtype=torch.float32, device=dev)
    check(_lib.lib().tfb_router_topk2(logits.data_ptr(), int(logits.dtype == torch.float32), T, E, k, int(renormalize),
                                      idx.data_ptr(), w.data_ptr(), probs.data_ptr(), counts.data_ptr(), prob_sums.data_ptr(),
                                      lse.data_ptr(), lse_sq.data_ptr(), stream()), "router_topk")
    return idx, w, probs, counts, lse, prob_sums, lse_sq


class Plan:
    """Expert segments padded to 128 rows inside a buffer of ``max_rows`` rows (worst case, no host sync)."""

    def __init__(self, idx, counts, E):
        T, k = idx.shape
        dev = idx.device
        self.T, self.k, self.E = T, k, E
        self.counts = counts
        self.max_rows = (T * k + 127) // 128 * 128 + 128 * E
        self.max_tiles = self.max_rows // 128
        if not idx.is_cuda:
            seg, off = [], 0
            tiles = []
            for e in range(E):
                seg.append(off)
                n = (int(counts[e]) + 127) // 128
                tiles += [e] * n
                off += n * 128
            seg.append(off)
            self.seg_start = torch.tensor(seg, dtype=torch.int32)
            self.expert_of_tile = torch.tensor(tiles + [-1] * (self.max_tiles - len(tiles)), dtype=torch.int32)
            cur = list(seg[:-1])
            row_of = torch.empty(T * k, dtype=torch.int32)
            tok = torch.full((self.max_rows,), -1, dtype=torch.int32)
            flat = idx.reshape(-1).tolist()
            for i, e in enumerate(flat):
                row_of[i] = cur[e]
                tok[cur[e]] = i // k
                cur[e] += 1
            self.row_of, self.token_of_row = row_of.view(T, k), tok
            return
        self.seg_start = torch.empty(E + 1, dtype=torch.int32, device=dev)
        self.cursor = torch.empty(E, dtype=torch.int32, device=dev)
        self.expert_of_tile = torch.empty(self.max_tiles, dtype=torch.int32, device=dev)
        self.total = torch.empty(1, dtype=torch.int32, device=dev)
        self.row_of = torch.empty((T, k), dtype=torch.int32, device=dev)
        self.token_of_row = torch.full((self.max_rows,), -1, dtype=torch.int32, device=dev)
        check(_lib.lib().tfb_moe_plan(counts.data_ptr(), E, self.seg_start.data_ptr(), self.cursor.data_ptr(),
                                      self.expert_of_tile.data_ptr(), self.max_tiles, self.total.data_ptr(), stream()),
              "moe_plan")


def zero_pads(buf, plan: Plan, segments: bool):
    """Clears the rows of an expert buffer [max_rows, H] that carry no assignment: the tail past the last segment and,
    with ``segments``, the padding behind every expert's rows.  (Cheaper than zero-filling the whole buffer, and the
    weight-gradient products sum over padded segments, so those rows must be zero.)"""
    check(_lib.lib().tfb_moe_zero_pads(buf.data_ptr(), buf.shape[1], plan.seg_start.data_ptr(),
                                       plan.counts.data_ptr() if segments else None, plan.E, plan.total.data_ptr(), buf.shape[0],
                                       stream()), "moe_zero_pads")
    return buf


def permute(x, idx, plan: Plan):
    """x [T, H] -> xp [max_rows, H] with every (token, k) row placed in its expert's segment (padding rows 0)."""
    T, H = x.shape
    if not x.is_cuda:
        xp = torch.zeros((plan.max_rows, H), dtype=x.dtype, device=x.device)
        xp[plan.row_of.reshape(-1).long()] = x.repeat_interleave(plan.k, 0)
        return xp
    xp = torch.empty((plan.max_rows, H), dtype=x.dtype, device=x.device)
    check(_lib.lib().tfb_moe_permute2(x.data_ptr(), idx.data_ptr(), plan.cursor.data_ptr(), plan.row_of.data_ptr(),
                                      plan.token_of_row.data_ptr(), xp.data_ptr(), T, plan.k, H, plan.E, stream()), "moe_permute")
    return zero_pads(xp, plan, True)


def permute_bwd(dxp, plan: Plan):
    T, k = plan.T, plan.k
    H = dxp.shape[1]
    if not dxp.is_cuda:
        return dxp[plan.row_of.reshape(-1).long()].view(T, k, H).float().sum(1).to(dxp.dtype)
    dx = torch.empty((T, H), dtype=dxp.dtype, device=dxp.device)
    check(_lib.lib().tfb_moe_permute_bwd(dxp.data_ptr(), plan.row_of.data_ptr(), dx.data_ptr(), T, k, H, stream()),
          "moe_permute_bwd")
    return dx


def combine(yp, w, plan: Plan, residual=None):
    T, k = plan.T, plan.k
    H = yp.shape[1]
    if not yp.is_cuda:
        y = (yp[plan.row_of.reshape(-1).long()].view(T, k, H).float() * w[..., None]).sum(1)
        if residual is not None:
            y = y + residual.float()
        return y.to(yp.dtype)
    y = torch.empty((T, H), dtype=yp.dtype, device=yp.device)
    check(_lib.lib().tfb_moe_combine(yp.data_ptr(), plan.row_of.data_ptr(), w.data_ptr(), y.data_ptr(), ptr(residual),
                                     T, k, H, stream()), "moe_combine")
    return y


def combine_bwd(dy, yp, w, plan: Plan):
    """Returns (dyp [max_rows, H], dw [T, k])."""
    T, k = plan.T, plan.k
    H = yp.shape[1]
    if not dy.is_cuda:
        rows = plan.row_of.reshape(-1).long()
        dyp = torch.zeros_like(yp)
        dyp[rows] = (dy.float().repeat_interleave(k, 0) * w.reshape(-1, 1)).to(yp.dtype)
        dw = (dy.float().repeat_interleave(k, 0) * yp[rows].float()).sum(-1).view(T, k)
        return dyp, dw
    dyp = zero_pads(torch.empty_like(yp), plan, True) if hasattr(plan, "total") else torch.zeros_like(yp)
    dw = torch.empty((T, k), dtype=torch.float32, device=dy.device)
    check(_lib.lib().tfb_moe_combine_bwd(dy.data_ptr(), yp.data_ptr(), plan.row_of.data_ptr(), w.data_ptr(),
                                         dyp.data_ptr(), dw.data_ptr(), T, k, H, stream()), "moe_combine_bwd")
    return dyp, dw


# ---------------------------------------------------------------------------------------------
# grouped GEMMs
# ---------------------------------------------------------------------------------------------
def grouped_gemm(xp, w, plan: Plan, b_mn=False, out=None):
    """xp [rows, K] @ w[e]^T per 128-row tile.  w is [E, N, K] (b_mn False) or [E, K, N] (b_mn True).  ``out``
    (CUDA only): a [rows, N] buffer to write into, e.g. a symmetric-memory buffer that peers read next."""
    rows, K = xp.shape
    E = w.shape[0]
    N = w.shape[2] if b_mn else w.shape[1]
    if not xp.is_cuda:
        out = torch.zeros((rows, N), dtype=xp.dtype)
        for i, e in enumerate(plan.expert_of_tile.tolist()):
            if e >= 0:
                W = w[e].float() if b_mn else w[e].float().t()
                out[i * 128:(i + 1) * 128] = (xp[i * 128:(i + 1) * 128].float() @ W).to(xp.dtype)
        return out
    # tiles past the last segment are skipped by the kernel: only that tail needs clearing (padding rows inside a segment
    # are products of zero rows)
    if out is not None:
        assert out.shape == (rows, N) and out.dtype == xp.dtype and hasattr(plan, "total") and N % 8 == 0
        zero_pads(out, plan, False)
    elif hasattr(plan, "total") and N % 8 == 0:
        out = zero_pads(torch.empty((rows, N), dtype=xp.dtype, device=xp.device), plan, False)
    else:
        out = torch.zeros((rows, N), dtype=xp.dtype, device=xp.device)
    g = _Group(1, E, plan.expert_of_tile.data_ptr(), None, w.stride(0), 0)
    check(_grouped_fn()(xp.data_ptr(), xp.stride(0), 0, w.data_ptr(), w.stride(1), int(b_mn), out.data_ptr(),
                        out.stride(0), rows, N, K, 1.0, 0, C.byref(g), _lib.status_word(xp.device).data_ptr(), stream()),
          "gemm_grouped")
    return out


def grouped_wgrad(dyp, xp, plan: Plan, out):
    """out[e] (fp32 [E, N, K]) += dyp[seg_e]^T @ xp[seg_e] for every expert in one launch."""
    rows, N = dyp.shape
    K = xp.shape[1]
    E = out.shape[0]
    if not dyp.is_cuda:
        seg = plan.seg_start.tolist()
        for e in range(E):
            a, b = seg[e], seg[e + 1]
            if b > a:
                out[e] += dyp[a:b].float().t() @ xp[a:b].float()
        return out
    g = _Group(2, E, None, plan.seg_start.data_ptr(), 0, out.stride(0))
    check(_grouped_fn()(dyp.data_ptr(), dyp.stride(0), 1, xp.data_ptr(), xp.stride(0), 1, out.data_ptr(), out.stride(1),
                        N, K, rows, 1.0, 2, C.byref(g), _lib.status_word(dyp.device).data_ptr(), stream()),
          "gemm_grouped_wgrad")
    return out


# ---------------------------------------------------------------------------------------------
# the whole expert FFN as one autograd node
# ---------------------------------------------------------------------------------------------
class MoEFFN(torch.autograd.Function):
    """y = sum_k w_k * down_e(act(gate_e(x)) * up_e(x)) over the top-k experts of each token.

    Inputs: x [T, H]; router logits [T, E]; gate_up [E, 2F, H]; down [E, H, F].  Returns
    (y, aux) where aux = load-balance loss E * sum_e f_e * P_e + z_weight * mean(lse^2) (differentiable
    through the router probabilities).  Expert weight gradients go to ``main_grad`` when present."""

    @staticmethod
    def forward(ctx, x, logits, gate_up, down, k, renorm, act, lb_weight, z_weight):
        T, H = x.shape
        E = gate_up.shape[0]
        idx, w, probs, counts, lse, prob_sums, lse_sq = router_topk_stats(logits, k, renorm)
        plan = Plan(idx, counts, E)
        xp = permute(x, idx, plan)
        gu = grouped_gemm(xp, gate_up.data, plan)
        a = F.glu_fwd(gu, act)
        yp = grouped_gemm(a, down.data, plan)
        y = combine(yp, w, plan)
        f = counts.float() / float(T * k)
        aux = (lb_weight * E / T) * (f * prob_sums).sum() + (z_weight / T) * lse_sq[0]
        ctx.save_for_backward(x, xp, gu, a, yp, w, probs, idx, lse, f)
        ctx.plan, ctx.gate_up, ctx.down = plan, gate_up, down
        ctx.cfg = (k, renorm, act, lb_weight, z_weight, E)
        ctx.logits_dtype = logits.dtype
        ctx.mark_non_differentiable(idx)
        return y, aux, idx

    @staticmethod
    def backward(ctx, dy, daux, _didx):
        x, xp, gu, a, yp, w, probs, idx, lse, f = ctx.saved_tensors
        plan, gate_up, down = ctx.plan, ctx.gate_up, ctx.down
        k, renorm, act, lb_weight, z_weight, E = ctx.cfg
        T = x.shape[0]
        dy = dy.contiguous()
        dyp, dw = combine_bwd(dy, yp, w, plan)
        for p_ in (gate_up, down):
            if not hasattr(p_, "main_grad") or p_.main_grad is None:
                p_.main_grad = torch.zeros(p_.shape, dtype=torch.float32, device=p_.device)
        da = grouped_gemm(dyp, down.data, plan, b_mn=True)
        grouped_wgrad(dyp, a, plan, down.main_grad)
        dgu = F.glu_bwd(gu, da, act)
        dxp = grouped_gemm(dgu, gate_up.data, plan, b_mn=True)
        grouped_wgrad(dgu, xp, plan, gate_up.main_grad)
        dx = permute_bwd(dxp, plan)
        # ---- router: d(top-k weights)/d(probs) then soft-max backward, plus the auxiliary losses ----
        dprobs = torch.zeros_like(probs)
        li = idx.long()
        sel = probs.gather(1, li)
        if renorm:
            s = sel.sum(-1, keepdim=True)
            dsel = dw / s - (dw * sel).sum(-1, keepdim=True) / (s * s)
        else:
            dsel = dw
        dprobs.scatter_add_(1, li, dsel)
        daux = daux if daux is not None else torch.zeros((), device=x.device)
        dprobs = dprobs + daux * lb_weight * E * f[None, :] / T
        dlogits = probs * (dprobs - (dprobs * probs).sum(-1, keepdim=True))
        dlogits = dlogits + daux * z_weight * (2.0 / T) * lse[:, None] * probs
        return dx, dlogits.to(ctx.logits_dtype), None, None, None, None, None, None, None


def moe_ffn(x, logits, gate_up, down, k=2, renormalize=True, act="silu", lb_weight=0.01, z_weight=0.0):
    return MoEFFN.apply(x, logits, gate_up, down, k, renormalize, act, lb_weight, z_weight)
