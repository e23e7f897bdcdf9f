"""Sampling: repetition penalty, temperature, top-k, top-p, greedy — one device kernel per batch of
sequences (``sample``), plus the host statement of the same rules (CPU path / oracle).

Parity: SamplerConfig{temperature .7, top_k 40, top_p .9, repetition_penalty, max_tokens 512} and
Sampler::sample's rule "top-p when p < 1, else top-k" (reference src/inference/sampler.cpp:166-180,
include/quant/sampler.h); ``reference_rule=True`` reproduces that either/or, the default applies both
cuts (top-k, then top-p inside the top-k set).  ReasoningBudget caps 256 / 2048 / 8192."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import _lib
from ..ops._lib import check, stream

REASONING_BUDGET = {"low": 256, "medium": 2048, "high": 8192}


@dataclass
class SamplerConfig:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    repetition_penalty: float = 1.0
    max_tokens: int = 512
    seed: int = 42
    reference_rule: bool = False

    def effective_max_tokens(self, budget: Optional[str] = None) -> int:
        """``max_tokens`` capped by a reasoning budget level ("low" 256 / "medium" 2048 / "high" 8192) when one is given."""
        cap = REASONING_BUDGET.get((budget or "").lower())
        return min(self.max_tokens, cap) if cap else self.max_tokens


class _Desc(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("logits_bf16", C.c_int), ("ld", C.c_longlong), ("work", C.c_void_p),
                ("history", C.c_void_p), ("hist_len", C.c_int), ("temperature", C.c_void_p), ("top_k", C.c_void_p),
                ("top_p", C.c_void_p), ("rep_penalty", C.c_void_p), ("out_ids", C.c_void_p),
                ("out_logprob", C.c_void_p), ("V", C.c_int), ("seed", C.c_ulonglong), ("step", C.c_int)]


def _filtered_probs(logits, temperature, top_k, top_p, rep, history):
    """Host statement: returns the renormalised distribution after all filters (fp32 [V])."""
    z = logits.float().clone()
    if rep != 1.0 and history is not None:
        for tok in set(int(t) for t in history if int(t) >= 0):
            z[tok] = z[tok] / rep if z[tok] > 0 else z[tok] * rep
    if temperature <= 0:
        p = torch.zeros_like(z)
        p[int(torch.argmax(z))] = 1.0
        return p
    z = z / temperature
    keep = torch.ones_like(z, dtype=torch.bool)
    if 0 < top_k < z.numel():
        kth = torch.topk(z, top_k).values[-1]
        keep &= z >= kth
    if top_p < 1.0:
        zz = torch.where(keep, z, torch.full_like(z, float("-inf")))
        p = torch.softmax(zz, -1)
        sp, si = torch.sort(p, descending=True)
        cum = torch.cumsum(sp, 0)
        n = int((cum < top_p).sum().item()) + 1
        k2 = torch.zeros_like(keep)
        k2[si[:n]] = True
        keep &= k2
    z = torch.where(keep, z, torch.full_like(z, float("-inf")))
    return torch.softmax(z, -1)


def sample(logits, temperature, top_k, top_p, rep_penalty=None, history=None, seed=42, step=0, want_logprob=False):
    """logits [B, V] (bf16 or fp32).  temperature / top_k / top_p / rep_penalty: per-row tensors [B]
    (float32 / int32 / float32 / float32) on the same device.  Returns ids int64 [B] (and log-probs)."""
    B, V = logits.shape
    if not logits.is_cuda:
        ids = torch.empty(B, dtype=torch.int64)
        lps = torch.empty(B)
        g = torch.Generator().manual_seed(seed * 1000003 + step)
        for b in range(B):
            p = _filtered_probs(logits[b], float(temperature[b]), int(top_k[b]), float(top_p[b]),
                                float(rep_penalty[b]) if rep_penalty is not None else 1.0,
                                history[b] if history is not None else None)
            ids[b] = int(torch.multinomial(p, 1, generator=g))
            lps[b] = torch.log_softmax(logits[b].float(), -1)[ids[b]]
        return (ids, lps) if want_logprob else ids
    dev = logits.device
    work = torch.empty((B, V), dtype=torch.float32, device=dev)
    ids = torch.empty(B, dtype=torch.int64, device=dev)
    lp = torch.empty(B, dtype=torch.float32, device=dev) if want_logprob else None
    d = _Desc()
    d.logits, d.logits_bf16, d.ld = logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0)
    d.work = work.data_ptr()
    d.history = history.data_ptr() if history is not None else None
    d.hist_len = history.shape[1] if history is not None else 0
    d.temperature, d.top_k, d.top_p = temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr()
    d.rep_penalty = rep_penalty.data_ptr() if rep_penalty is not None else None
    d.out_ids, d.out_logprob = ids.data_ptr(), lp.data_ptr() if lp is not None else None
    d.V, d.seed, d.step = V, seed & 0xFFFFFFFFFFFFFFFF, step
    fn = _lib.lib().tfb_sample
    fn.argtypes, fn.restype = [C.POINTER(_Desc), C.c_int, C.c_void_p], C.c_int
    check(fn(C.byref(d), B, stream()), "sample")
    return (ids, lp) if want_logprob else ids


class Sampler:
    """Per-request sampler with the reference's configuration surface."""

    def __init__(self, cfg: SamplerConfig = SamplerConfig()):
        self.cfg = cfg
        self.step = 0

    def params(self, B, device):
        c = self.cfg
        k = 0 if (c.reference_rule and c.top_p < 1.0) else c.top_k
        return (torch.full((B,), c.temperature, dtype=torch.float32, device=device),
                torch.full((B,), k, dtype=torch.int32, device=device),
                torch.full((B,), c.top_p, dtype=torch.float32, device=device),
                torch.full((B,), c.repetition_penalty, dtype=torch.float32, device=device))

    def __call__(self, logits, history=None):
        t, k, p, r = self.params(logits.shape[0], logits.device)
        self.step += 1
        return sample(logits, t, k, p, r, history, self.cfg.seed, self.step)

    # ---- the single-row verbs of the reference's Sampler (include/quant/sampler.h; src/inference/sampler.cpp)
    def set_seed(self, seed: int):
        self.cfg.seed, self.step = int(seed), 0

    @staticmethod
    def apply_temperature(logits: torch.Tensor, temperature: float) -> torch.Tensor:
        return logits.float() / max(float(temperature), 1e-6)

    @staticmethod
    def apply_repetition_penalty(logits: torch.Tensor, history, penalty: float) -> torch.Tensor:
        """Seen tokens: positive logits divided by the penalty, negative ones multiplied by it."""
        z = logits.float().clone()
        if penalty != 1.0 and history is not None and len(history):
            idx = torch.as_tensor(sorted({int(t) for t in history if 0 <= int(t) < z.shape[-1]}), dtype=torch.long, device=z.device)
            if idx.numel():
                v = z[..., idx]
                z[..., idx] = torch.where(v > 0, v / penalty, v * penalty)
        return z

    @staticmethod
    def greedy(logits: torch.Tensor) -> int:
        return int(logits.reshape(-1, logits.shape[-1])[-1].argmax())

    def _draw(self, logits, temperature, top_k, top_p, history=None):
        row = logits.reshape(-1, logits.shape[-1])[-1:].contiguous()
        dev = row.device
        one = lambda v, dt: torch.full((1,), v, dtype=dt, device=dev)
        hist = None
        if history is not None and len(history) and self.cfg.repetition_penalty != 1.0:
            hist = torch.as_tensor([list(history)], dtype=torch.int32 if row.is_cuda else torch.long, device=dev)
        self.step += 1
        return int(sample(row, one(temperature, torch.float32), one(top_k, torch.int32), one(top_p, torch.float32),
                          one(self.cfg.repetition_penalty, torch.float32), hist, self.cfg.seed, self.step)[0])

    def sample_top_k(self, logits, k: int, temperature: Optional[float] = None) -> int:
        return self._draw(logits, self.cfg.temperature if temperature is None else temperature, k, 1.0)

    def sample_top_p(self, logits, p: float, temperature: Optional[float] = None) -> int:
        return self._draw(logits, self.cfg.temperature if temperature is None else temperature, 0, p)

    def sample(self, logits, history=None) -> int:
        """One token for one row of logits under the configuration (``reference_rule``: top-p when p < 1, else top-k)."""
        c = self.cfg
        if c.temperature <= 0:
            return self.greedy(self.apply_repetition_penalty(logits.reshape(-1, logits.shape[-1])[-1], history, c.repetition_penalty))
        k = 0 if (c.reference_rule and c.top_p < 1.0) else c.top_k
        return self._draw(logits, c.temperature, k, c.top_p, history)
