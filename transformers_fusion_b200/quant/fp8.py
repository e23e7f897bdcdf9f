"""Block-scaled FP8 (E4M3) quantisation and GEMM.

Activations carry one fp32 scale per 1 x 128 block, weights one per 128 x 128 block (the layout of
the Mixtral-shaped MoE configuration); products are accumulated in fp32 with both scales applied per
128-wide K block.  CUDA tensors use the tcgen05 kernel; CPU tensors use the PyTorch statement below,
which is also the oracle for the GPU tests.

E4M3 conversion parity: quantize_fp8_e4m3 / dequantize (reference src/codec/quant_engines_fp.cpp:17-121:
max finite 448, no infinities, round to nearest even)."""
from __future__ import annotations

import torch

from ..ops import _lib
from ..ops._lib import c_f, c_i, c_ll, c_p, check, ptr, stream

_lib.register("tfb_gemm_fp8_blockscaled", [c_p, c_p, c_p, c_p, c_p, c_ll, c_i, c_i, c_i, c_i, c_p, c_p, c_p])
_lib.register("tfb_quant_fp8_1x128", [c_p, c_p, c_p, c_ll, c_i, c_p])
_lib.register("tfb_quant_fp8_128x128", [c_p, c_p, c_p, c_i, c_i, c_p])

E4M3_MAX = 448.0


def quant_act_1x128(x):
    """x [rows, K] -> (q uint8-viewed e4m3 [rows, K], scale fp32 [rows, ceil(K/128)])."""
    rows, K = x.shape
    kb = (K + 127) // 128
    if not x.is_cuda:
        xp = torch.nn.functional.pad(x.float(), (0, kb * 128 - K)).view(rows, kb, 128)
        amax = xp.abs().amax(-1)
        s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
        q = (xp / s[..., None]).to(torch.float8_e4m3fn).view(rows, kb * 128)[:, :K].contiguous()
        return q.view(torch.uint8), s
    q = torch.empty((rows, K), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, kb), dtype=torch.float32, device=x.device)
    check(_lib.lib().tfb_quant_fp8_1x128(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, K, stream()), "quant_fp8_1x128")
    return q, s


def quant_weight_128x128(w):
    """w [N, K] (or [E, N, K]) -> (q uint8-viewed e4m3, scale fp32 [(E,) ceil(N/128), ceil(K/128)])."""
    if w.dim() == 3:
        qs = [quant_weight_128x128(w[e]) for e in range(w.shape[0])]
        return torch.stack([a for a, _ in qs]), torch.stack([b for _, b in qs])
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    if not w.is_cuda:
        wp = torch.nn.functional.pad(w.float(), (0, kb * 128 - K, 0, nb * 128 - N)).view(nb, 128, kb, 128)
        amax = wp.abs().amax((1, 3))
        s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
        q = (wp / s[:, None, :, None]).to(torch.float8_e4m3fn).view(nb * 128, kb * 128)[:N, :K].contiguous()
        return q.view(torch.uint8), s
    q = torch.empty((N, K), dtype=torch.uint8, device=w.device)
    s = torch.empty((nb, kb), dtype=torch.float32, device=w.device)
    check(_lib.lib().tfb_quant_fp8_128x128(w.data_ptr(), q.data_ptr(), s.data_ptr(), N, K, stream()), "quant_fp8_128x128")
    return q, s


def dequant(q, s, block_rows):
    """fp32 reconstruction; block_rows = 1 for activations, 128 for weights."""
    x = q.view(torch.float8_e4m3fn).float()
    rows, K = x.shape
    sr = s.repeat_interleave(block_rows, 0)[:rows] if block_rows > 1 else s
    return x * sr.repeat_interleave(128, 1)[:, :K]


def gemm_fp8(qa, sa, qb, sb, expert_of_mtile=None, out=None):
    """C [M, N] bf16 = dequant(qa, sa) @ dequant(qb[e], sb[e])^T; ``qb`` is [N, K] or [E, N, K].
    Grouped mode: rows of ``qa`` are expert segments padded to 128; ``expert_of_mtile`` int32 [M/128]."""
    M, K = qa.shape
    grouped = qb.dim() == 3
    E = qb.shape[0] if grouped else 1
    N = qb.shape[-2]
    if not qa.is_cuda:
        A = dequant(qa, sa, 1)
        if not grouped:
            return (A @ dequant(qb, sb, 128).t()).to(torch.bfloat16)
        C = torch.zeros(M, N)
        for i, e in enumerate(expert_of_mtile.tolist()):
            if e >= 0:
                C[i * 128:(i + 1) * 128] = A[i * 128:(i + 1) * 128] @ dequant(qb[e], sb[e], 128).t()
        return C.to(torch.bfloat16)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=qa.device)
        if grouped:
            out.zero_()
    check(_lib.lib().tfb_gemm_fp8_blockscaled(qa.data_ptr(), sa.data_ptr(), qb.data_ptr(), sb.data_ptr(),
                                              out.data_ptr(), out.stride(0), M, N, K, E, ptr(expert_of_mtile),
                                              _lib.status_word(qa.device).data_ptr(), stream()), "gemm_fp8_blockscaled")
    return out
