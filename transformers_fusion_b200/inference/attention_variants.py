"""Stand-alone attention modules with their own projections: multi-query, grouped-query, sliding-window and ALiBi
attention, plus ``compute_logprobs``.  On a GPU the multi-query and grouped-query forms run on the flash-attention
kernel (several query heads per key / value head are what it is tiled for); the windowed and the biased form, which the
kernel's causal mask cannot express, are evaluated as tiled fp32 math (``MemoryEfficientAttention`` carries the
block-sparse long-context form of the window).

Reference counterparts: MultiQueryAttention, GroupedQueryAttention, SlidingWindowAttention, ALiBi, compute_logprobs
(include/quant/inference_opt.h:237-345, src/inference/inference_attention.cpp)."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from ..ops import functional as F


def _init(out_f, in_f, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(out_f, in_f, generator=g) * (1.0 / math.sqrt(in_f))


class GroupedQueryAttention:
    """y = W_o softmax(Q K^T / sqrt(d)) V with ``n_heads`` query heads sharing ``n_kv_heads`` key / value heads.
    ``forward(x)`` is causal self-attention on x [B, S, d_model]; ``forward(q_in, k_in, v_in)`` projects three inputs."""

    def __init__(self, d_model: int, n_heads: int, n_kv_heads: int, device="cpu", dtype=torch.float32, seed: int = 0):
        assert d_model % n_heads == 0 and n_heads % n_kv_heads == 0
        self.d_model, self._n_heads, self._n_kv = d_model, n_heads, n_kv_heads
        self.head_dim = d_model // n_heads
        kv = n_kv_heads * self.head_dim
        mk = lambda o, i, s: _init(o, i, seed + s).to(device=device, dtype=dtype)
        self.w_q, self.w_k, self.w_v, self.w_o = mk(d_model, d_model, 1), mk(kv, d_model, 2), mk(kv, d_model, 3), mk(d_model, d_model, 4)

    def n_heads(self) -> int: return self._n_heads
    def n_kv_heads(self) -> int: return self._n_kv

    def _project(self, q_in, k_in, v_in):
        B, S, _ = q_in.shape
        Sk = k_in.shape[1]
        q = (q_in @ self.w_q.t()).view(B, S, self._n_heads, self.head_dim)
        k = (k_in @ self.w_k.t()).view(B, Sk, self._n_kv, self.head_dim)
        v = (v_in @ self.w_v.t()).view(B, Sk, self._n_kv, self.head_dim)
        return q, k, v

    def _scores_bias(self, S, Sk, device):
        """Additive [heads or 1, S, Sk] term for subclasses (window mask, ALiBi slopes)."""
        return None

    def forward(self, q_in, k_in=None, v_in=None, mask: Optional[torch.Tensor] = None, causal: bool = True):
        k_in = q_in if k_in is None else k_in
        v_in = k_in if v_in is None else v_in
        q, k, v = self._project(q_in, k_in, v_in)
        B, S, Hq, D = q.shape
        Sk = k.shape[1]
        bias = self._scores_bias(S, Sk, q.device)
        if q.is_cuda and bias is None and mask is None and causal and S == Sk and q.dtype == torch.bfloat16 and D in (64, 128):
            qf, kf, vf = q.reshape(B * S, Hq * D), k.reshape(B * S, -1), v.reshape(B * S, -1)
            o, _ = F.attn_fwd(qf.contiguous(), kf.contiguous(), vf.contiguous(), B, S, Hq, self._n_kv, D)
            return (o.view(B, S, Hq * D) @ self.w_o.t())
        g = Hq // self._n_kv
        qh = q.permute(0, 2, 1, 3).float()
        kh = k.permute(0, 2, 1, 3).float().repeat_interleave(g, 1)
        vh = v.permute(0, 2, 1, 3).float().repeat_interleave(g, 1)
        s = qh @ kh.transpose(-1, -2) / math.sqrt(D)
        if causal:
            s = s.masked_fill(torch.ones(S, Sk, dtype=torch.bool, device=s.device).triu(1 + Sk - S), float("-inf"))
        if bias is not None:
            s = s + bias
        if mask is not None:
            s = s + mask.float()
        o = (torch.softmax(s, -1) @ vh).permute(0, 2, 1, 3).reshape(B, S, Hq * D)
        return o.to(q_in.dtype) @ self.w_o.t()

    __call__ = forward


class MultiQueryAttention(GroupedQueryAttention):
    """All query heads share one key / value head."""

    def __init__(self, d_model: int, n_heads: int, d_kv: int = -1, **kw):
        super().__init__(d_model, n_heads, 1, **kw)

    def d_model_(self) -> int: return self.d_model


class SlidingWindowAttention(GroupedQueryAttention):
    """Causal attention in which position i sees positions (i - window, i]."""

    def __init__(self, d_model: int, n_heads: int, window_size: int = 512, **kw):
        super().__init__(d_model, n_heads, n_heads, **kw)
        self.window_size = window_size

    def _scores_bias(self, S, Sk, device):
        i = torch.arange(S, device=device)[:, None] + (Sk - S)
        j = torch.arange(Sk, device=device)[None, :]
        return torch.where(i - j >= self.window_size, float("-inf"), 0.0)[None]


class ALiBi(GroupedQueryAttention):
    """Attention with linear position biases instead of rotary embeddings: head h adds -slope_h * (i - j) to the score of
    query i and key j (slopes 2^(-8 h / n) for n a power of two, interleaved for other head counts)."""

    def __init__(self, n_heads: int, d_model: int = 0, **kw):
        super().__init__(d_model or 64 * n_heads, n_heads, n_heads, **kw)
        self.slopes = torch.tensor(self.compute_slopes(n_heads))

    @staticmethod
    def compute_slopes(n: int) -> List[float]:
        def pow2(m):
            start = 2.0 ** (-8.0 / m)
            return [start ** (i + 1) for i in range(m)]
        if n & (n - 1) == 0:
            return pow2(n)
        m = 1 << (n.bit_length() - 1)
        return pow2(m) + pow2(2 * m)[0::2][: n - m]

    def build_alibi_bias(self, S_q: int, S_k: int, device="cpu") -> torch.Tensor:
        i = torch.arange(S_q, device=device)[:, None] + (S_k - S_q)
        j = torch.arange(S_k, device=device)[None, :]
        return -(i - j).clamp(min=0).float()[None] * self.slopes.to(device)[:, None, None]

    def _scores_bias(self, S, Sk, device):
        return self.build_alibi_bias(S, Sk, device)


def compute_logprobs(logits: torch.Tensor, tokens: Sequence[int]) -> List[List[float]]:
    """Per generated token the full log-probability row: logits [T, V] (row t scores token t) -> T lists of V floats."""
    lp = torch.log_softmax(logits.float().reshape(-1, logits.shape[-1]), -1)
    return lp[: len(tokens)].tolist()
