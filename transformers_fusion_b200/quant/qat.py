"""Quantisation-aware training: fake quantisation with a straight-through estimator, LSQ learned step
sizes, range observers, and the codec round trip ("train through the wire format").

Reference counterparts: fake_quantize / lsq_fake_quantize / observers (src/codec/qat.cpp), STE quantizer
(src/codec/ste_quantizer.cpp), TrainConfig.qat_bits / qat_symmetric / LSQ flags (include/quant/trainer.h:52-58)."""
from __future__ import annotations

import math

import numpy as np
from dataclasses import dataclass

import torch

from ..ops import _lib
from ..ops._lib import c_f, c_i, c_ll, c_p, check, ptr, stream
from . import codec

_lib.register("tfb_fake_quant_block", [c_p, c_p, c_p, c_ll, c_i, c_i, c_i, c_i, c_p])
_lib.register("tfb_lsq_fwd", [c_p, c_p, c_p, c_ll, c_f, c_f, c_i, c_p])
_lib.register("tfb_lsq_bwd", [c_p, c_p, c_p, c_p, c_p, c_ll, c_f, c_f, c_f, c_i, c_p])


def _dt(t):
    assert t.dtype in (torch.bfloat16, torch.float32)
    return 0 if t.dtype == torch.bfloat16 else 1


def fake_quant_block(x: torch.Tensor, bits=8, block=256, symmetric=True, out=None, return_scales=False):
    """Quantise-dequantise with one scale (and zero point) per ``block`` consecutive elements."""
    x = x.contiguous()
    out = torch.empty_like(x) if out is None else out
    n = x.numel()
    nb = (n + block - 1) // block
    if x.is_cuda:
        sc = torch.empty(nb, dtype=torch.float32, device=x.device) if return_scales else None
        check(_lib.lib().tfb_fake_quant_block(x.data_ptr(), out.data_ptr(), ptr(sc), n, block, bits, int(symmetric), _dt(x),
                                              stream()), "fake_quant_block")
        return (out, sc) if return_scales else out
    f = torch.zeros(nb * block, dtype=torch.float32)
    f[:n] = x.reshape(-1).float()
    f = f.view(nb, block)
    valid = torch.arange(nb * block).view(nb, block) < n
    if symmetric:
        qmax = float((1 << (bits - 1)) - 1)
        amax = f.abs().amax(1, keepdim=True)
        s = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
        q = torch.clamp(torch.round(f * (1.0 / s)), -qmax, qmax) * s
    else:
        levels = float((1 << bits) - 1)
        lo = torch.where(valid, f, torch.full_like(f, float("inf"))).amin(1, keepdim=True)
        hi = torch.where(valid, f, torch.full_like(f, float("-inf"))).amax(1, keepdim=True)
        s = torch.where(hi > lo, (hi - lo) / levels, torch.ones_like(hi))
        q = torch.clamp(torch.round((f - lo) * (1.0 / s)), 0, levels) * s + lo
    out.copy_(q.reshape(-1)[:n].view(x.shape).to(x.dtype))
    return (out, s[:, 0]) if return_scales else out


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bits, block, symmetric):
        return fake_quant_block(x, bits, block, symmetric)

    @staticmethod
    def backward(ctx, dy):
        return dy, None, None, None


def fake_quantize(x, bits=8, block=256, symmetric=True):
    """Differentiable fake quantisation (identity gradient)."""
    return _FakeQuantSTE.apply(x, bits, block, symmetric)


class _LSQ(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, step, bits, symmetric):
        qn, qp = (-(2 ** (bits - 1)), 2 ** (bits - 1) - 1) if symmetric else (0, 2 ** bits - 1)
        ctx.q = (float(qn), float(qp))
        ctx.save_for_backward(x, step)
        if x.is_cuda:
            x = x.contiguous()
            y = torch.empty_like(x)
            check(_lib.lib().tfb_lsq_fwd(x.data_ptr(), step.data_ptr(), y.data_ptr(), x.numel(), float(qn), float(qp), _dt(x), stream()),
                  "lsq_fwd")
            return y
        s = step.float().clamp(min=1e-12)
        return (torch.clamp(torch.round(x.float() / s), qn, qp) * s).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, step = ctx.saved_tensors
        qn, qp = ctx.q
        gs = 1.0 / math.sqrt(max(1.0, x.numel() * qp))
        if x.is_cuda:
            x, dy = x.contiguous(), dy.contiguous()
            dx = torch.empty_like(x)
            ds = torch.zeros(1, dtype=torch.float32, device=x.device)
            check(_lib.lib().tfb_lsq_bwd(x.data_ptr(), dy.data_ptr(), step.data_ptr(), dx.data_ptr(), ds.data_ptr(), x.numel(), qn, qp,
                                         gs, _dt(x), stream()), "lsq_bwd")
            return dx, ds.view(step.shape).to(step.dtype), None, None
        s = step.float().clamp(min=1e-12)
        r = x.float() / s
        inside = (r > qn) & (r < qp)
        dsv = torch.where(r <= qn, torch.full_like(r, qn), torch.where(r >= qp, torch.full_like(r, qp), torch.round(r) - r))
        return (dy.float() * inside).to(x.dtype), ((dy.float() * dsv).sum() * gs).view(step.shape).to(step.dtype), None, None


def lsq_fake_quantize(x, step, bits=8, symmetric=True):
    """Learned-step-size quantisation (Esser et al.): ``step`` is a 1-element fp32 parameter."""
    return _LSQ.apply(x, step, bits, symmetric)


def lsq_init_step(x, bits=8, symmetric=True):
    qp = 2 ** (bits - 1) - 1 if symmetric else 2 ** bits - 1
    return (2.0 * x.float().abs().mean() / math.sqrt(qp)).reshape(1).clone()


@dataclass
class QuantParams:
    scale: float = 1.0
    zero_point: int = 0
    qmin: int = -127
    qmax: int = 127

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        return (x.float() / self.scale + self.zero_point).round().clamp(self.qmin, self.qmax)

    def dequantize(self, q: torch.Tensor) -> torch.Tensor:
        return (q.float() - self.zero_point) * self.scale


class MinMaxObserver:
    def __init__(self):
        self.lo, self.hi = float("inf"), float("-inf")

    def observe(self, x):
        self.lo, self.hi = min(self.lo, float(x.min())), max(self.hi, float(x.max()))

    def qparams(self, bits=8, symmetric=True):
        if symmetric:
            return max(abs(self.lo), abs(self.hi)) / ((1 << (bits - 1)) - 1) or 1.0, 0.0
        s = (self.hi - self.lo) / ((1 << bits) - 1) or 1.0
        return s, self.lo

    # ---- the reference's observer interface (include/quant/qat.h:120-145)
    def has_data(self) -> bool: return self.lo <= self.hi
    def min_val(self) -> float: return self.lo if self.has_data() else 0.0
    def max_val(self) -> float: return self.hi if self.has_data() else 0.0
    def type(self) -> str: return {"MinMaxObserver": "MinMax", "MovingAverageObserver": "MovingAverage", "PercentileObserver": "Percentile"}.get(type(self).__name__, type(self).__name__)

    def reset(self):
        self.lo, self.hi = float("inf"), float("-inf")
        if hasattr(self, "init"):
            self.init = False

    def calc_qparams(self, bits=8, symmetric=True) -> "QuantParams":
        """Scale, integer zero point and integer range for the observed values; scale 1 before anything was observed."""
        if symmetric:
            qmin, qmax = -(1 << (bits - 1)) + 1, (1 << (bits - 1)) - 1
        else:
            qmin, qmax = 0, (1 << bits) - 1
        if not self.has_data():
            return QuantParams(1.0, 0, qmin, qmax)
        if symmetric:
            return QuantParams(max(abs(self.lo), abs(self.hi)) / qmax or 1.0, 0, qmin, qmax)
        lo, hi = min(self.lo, 0.0), max(self.hi, 0.0)            # the range must contain 0 so that 0 is exactly representable
        s = (hi - lo) / (qmax - qmin) or 1.0
        return QuantParams(s, int(min(max(round(qmin - lo / s), qmin), qmax)), qmin, qmax)


class MovingAverageObserver(MinMaxObserver):
    def __init__(self, momentum=0.9):
        super().__init__()
        self.m, self.init = momentum, False

    def observe(self, x):
        lo, hi = float(x.min()), float(x.max())
        if not self.init:
            self.lo, self.hi, self.init = lo, hi, True
        else:
            self.lo = self.m * self.lo + (1 - self.m) * lo
            self.hi = self.m * self.hi + (1 - self.m) * hi


class PercentileObserver(MinMaxObserver):
    def __init__(self, pct=99.99):
        super().__init__()
        self.pct = pct

    def observe(self, x):
        f = x.float().reshape(-1)
        if f.numel() > 1 << 20:
            f = f[torch.randint(0, f.numel(), (1 << 20,), device=f.device)]
        k = max(1, int(f.numel() * (1 - self.pct / 100.0)))
        self.hi = max(self.hi, float(f.topk(k).values[-1]))
        self.lo = min(self.lo, float((-f).topk(k).values[-1] * -1))


@torch.no_grad()
def ste_roundtrip_(t: torch.Tensor, fmt, block=256, mask=None):
    """Replace ``t`` by its decode(encode(t)) through a wire format (exactly what a saved checkpoint will
    hold).  ``mask`` (bool per block) restricts the round trip to selected blocks.  Formats with a plain
    absmax grid (Q_8 bits or more are approximated on device when ``t`` is a CUDA tensor and exactness is not
    needed) go through the codec on the host."""
    f = codec.parse_format(fmt) if isinstance(fmt, str) else int(fmt)
    a = t.detach().float().cpu().contiguous().numpy().reshape(-1)
    out = a.copy()
    for b, o in enumerate(range(0, a.size, block)):
        if mask is not None and not bool(mask[b]):
            continue
        seg = a[o:o + block]
        out[o:o + block] = codec.dequantize_block(f, codec.quantize_block(f, seg), seg.size)
    t.copy_(torch.from_numpy(out).view(t.shape).to(t.dtype))
    return t


class QATState:
    """Per-model QAT hook used by the trainer: fake-quantises every matrix weight before the forward pass
    (the fp32 master copy keeps the unquantised value, so the update is the straight-through estimator)."""

    def __init__(self, bits=8, symmetric=True, block=256, min_numel=1024):
        self.bits, self.symmetric, self.block, self.min_numel = bits, symmetric, block, min_numel

    @torch.no_grad()
    def apply_(self, model):
        for p in model.parameters():
            if p.dim() >= 2 and p.numel() >= self.min_numel:
                fake_quant_block(p.data, self.bits, self.block, self.symmetric, out=p.data)
