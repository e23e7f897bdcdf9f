"""Quantisation-aware training: fake quantisation with a straight-through estimator, LSQ learned step
sizes, range observers, and the codec round trip ("train through the wire format").

Reference counterparts: fake_quantize / lsq_fake_quantize / observers (src/codec/qat.cpp), STE quantizer
(src/codec/ste_quantizer.cpp), TrainConfig.qat_bits / qat_symmetric / LSQ flags (include/quant/trainer.h:52-58)."""
from __future__ import annotations

import math

import numpy as np
from dataclasses import dataclass
from typing import Optional

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


MovingAverageMinMaxObserver = MovingAverageObserver
Observer = MinMaxObserver          # the interface every observer follows: observe / calc_qparams / reset / type


class KLDivergenceObserver(MinMaxObserver):
    """Histogram calibration: the clipping threshold is the one whose quantised histogram is closest (Kullback-Leibler) to
    the observed one, which ignores rare outliers that a min / max range would spend its levels on.  Falls back to the
    observed range when the histogram is degenerate.  Reference counterpart: KLDivergenceObserver
    (include/quant/qat.h:164-183)."""

    def __init__(self, bins: int = 2048, quantized_bins: int = 128):
        super().__init__()
        self.bins, self.qbins = bins, quantized_bins
        self.hist = torch.zeros(bins, dtype=torch.float64)
        self.hmax = 0.0

    def type(self) -> str: return "KLDivergence"

    def reset(self):
        super().reset()
        self.hist.zero_()
        self.hmax = 0.0

    def observe(self, x):
        f = x.detach().float().reshape(-1).cpu()
        super().observe(f)
        amax = float(f.abs().max())
        if amax > self.hmax:                                       # widen the histogram: re-bin what is already there
            if self.hmax > 0 and float(self.hist.sum()) > 0:
                centres = (torch.arange(self.bins, dtype=torch.float64) + 0.5) * (self.hmax / self.bins)
                idx = (centres / amax * self.bins).long().clamp(max=self.bins - 1)
                self.hist = torch.zeros_like(self.hist).index_add_(0, idx, self.hist)
            self.hmax = amax
        if self.hmax > 0:
            self.hist += torch.histc(f.abs(), self.bins, 0.0, self.hmax).double()

    def compute_kl_threshold(self, bits: int = 8) -> float:
        levels = min(self.qbins, 1 << (bits - 1))
        total = float(self.hist.sum())
        if total <= 0 or self.hmax <= 0:
            return 0.0
        best, best_t = float("inf"), self.hmax
        for i in range(levels, self.bins + 1, max(1, self.bins // 256)):
            p = self.hist[:i].clone()
            p[-1] += self.hist[i:].sum()                           # clipped mass lands in the last kept bin
            edges = torch.linspace(0, i, levels + 1).long()
            q = torch.zeros(i, dtype=torch.float64)
            for a, b in zip(edges[:-1].tolist(), edges[1:].tolist()):
                seg = self.hist[a:b]
                nz = seg > 0
                if nz.any():
                    q[a:b][nz] = seg.sum() / nz.sum()
            pn, qn = p / p.sum(), q / q.sum().clamp(min=1e-30)
            m = pn > 0
            kl = float((pn[m] * (pn[m] / qn[m].clamp(min=1e-30)).log()).sum())
            if kl < best:
                best, best_t = kl, (i / self.bins) * self.hmax
        return best_t

    def calc_qparams(self, bits=8, symmetric=True) -> QuantParams:
        t = self.compute_kl_threshold(bits)
        if t <= 0:
            return super().calc_qparams(bits, symmetric)
        lo, hi = self.lo, self.hi
        self.lo, self.hi = max(lo, -t), min(hi, t)
        try:
            return super().calc_qparams(bits, symmetric)
        finally:
            self.lo, self.hi = lo, hi


@dataclass
class QATConfig:
    bits: int = 8
    symmetric: bool = True
    per_channel: bool = False
    narrow_range: bool = False
    init_scale: float = 1.0
    use_lsq: bool = False
    lsq_grad_scale: float = 1.0


def get_qrange(cfg_or_bits, symmetric: bool = True, narrow: bool = False):
    """(qmin, qmax) of a configuration (or of bits / symmetric / narrow given one by one)."""
    if isinstance(cfg_or_bits, QATConfig):
        cfg_or_bits, symmetric, narrow = cfg_or_bits.bits, cfg_or_bits.symmetric, cfg_or_bits.narrow_range
    b = int(cfg_or_bits)
    if not symmetric:
        return 0, (1 << b) - 1
    return -(1 << (b - 1)) + (1 if narrow else 0), (1 << (b - 1)) - 1


class _PerTensorSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, qmin, qmax):
        s = max(float(scale), 1e-12)
        return (torch.clamp(torch.round(x.float() / s), qmin, qmax) * s).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        return dy, None, None, None


def ste_fake_quantize(x, scale: float, qmin: int, qmax: int):
    """clamp(round(x / scale), qmin, qmax) * scale with one scale for the whole tensor; the gradient passes unchanged."""
    return _PerTensorSTE.apply(x, scale, qmin, qmax)


def fake_quantize_per_tensor(x, scale: float, bits: int = 8, symmetric: bool = True):
    return ste_fake_quantize(x, scale, *get_qrange(bits, symmetric))


def fake_quantize_with_observer(x, obs, bits: int = 8, symmetric: bool = True):
    """Feed ``x`` to the observer, then quantise it with the observer's current parameters (zero point included)."""
    obs.observe(x.detach())
    qp = obs.calc_qparams(bits, symmetric)
    if qp.zero_point == 0:
        return ste_fake_quantize(x, qp.scale, qp.qmin, qp.qmax)
    return x + (qp.dequantize(qp.quantize(x.detach())).to(x.dtype) - x).detach()


class LSQQuantizer:
    """Per-tensor fake quantisation whose step size is a trainable parameter (``scale_param_tensor()`` goes to the
    optimizer).  Reference counterpart: LSQQuantizer (include/quant/qat.h:84-109)."""

    def __init__(self, cfg: Optional[QATConfig] = None):
        self.cfg = cfg or QATConfig(use_lsq=True)
        self._qmin, self._qmax = get_qrange(self.cfg)
        self._step = torch.nn.Parameter(torch.tensor([max(self.cfg.init_scale, 1e-6)], dtype=torch.float32))

    def config(self) -> QATConfig: return self.cfg
    def qmin(self) -> int: return self._qmin
    def qmax(self) -> int: return self._qmax
    def scale(self) -> float: return float(self._step.detach())
    def scale_param_tensor(self) -> torch.nn.Parameter: return self._step
    def quant_params(self) -> QuantParams: return QuantParams(self.scale(), 0, self._qmin, self._qmax)

    def set_scale(self, s: float):
        with torch.no_grad():
            self._step.fill_(max(float(s), 1e-6))

    def init_from(self, x: torch.Tensor):
        """The usual LSQ start: 2 mean|x| / sqrt(qmax)."""
        self.set_scale(float(lsq_init_step(x, self.cfg.bits, self.cfg.symmetric)))
        return self

    def forward(self, x: torch.Tensor, scale_param: Optional[torch.Tensor] = None) -> torch.Tensor:
        step = self._step if scale_param is None else scale_param
        return lsq_fake_quantize(x, step.to(x.device), self.cfg.bits, self.cfg.symmetric)

    __call__ = forward

    def compute_scale_grad(self, x: torch.Tensor, grad_output: torch.Tensor) -> float:
        """dL/dstep for given dL/dy, by the LSQ rule (the rounding residual inside the range, the clip level outside),
        scaled by ``lsq_grad_scale`` / sqrt(numel * qmax)."""
        s = max(self.scale(), 1e-12)
        r = x.detach().float() / s
        qn, qp = float(get_qrange(self.cfg.bits, self.cfg.symmetric)[0]), float(self._qmax)
        d = torch.where(r <= qn, torch.full_like(r, qn), torch.where(r >= qp, torch.full_like(r, qp), torch.round(r) - r))
        return float((grad_output.detach().float() * d).sum()) * self.cfg.lsq_grad_scale / math.sqrt(max(1.0, x.numel() * qp))


class QATContext:
    """A switch the training loop consults: ``maybe_quantize`` is the identity while disabled.  Reference counterpart:
    QATContext (include/quant/qat.h:214-232)."""

    def __init__(self, cfg: Optional[QATConfig] = None):
        self.cfg, self._on = cfg or QATConfig(), False

    def enable(self): self._on = True
    def disable(self): self._on = False
    def enabled(self) -> bool: return self._on
    def config(self) -> QATConfig: return self.cfg
    def set_config(self, c: QATConfig): self.cfg = c

    def maybe_quantize(self, x, obs=None):
        if not self._on:
            return x
        if obs is not None:
            return fake_quantize_with_observer(x, obs, self.cfg.bits, self.cfg.symmetric)
        qmin, qmax = get_qrange(self.cfg)
        amax = float(x.detach().abs().max())
        return ste_fake_quantize(x, (amax / qmax) if amax > 0 else self.cfg.init_scale, qmin, qmax)

    def maybe_lsq_quantize(self, x, scale_param):
        return lsq_fake_quantize(x, scale_param, self.cfg.bits, self.cfg.symmetric) if self._on else x


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


class STEQuantizer:
    """Straight-through quantisation of weights to one of the container's formats: forward returns exactly what a saved
    checkpoint in that format would decode to, backward passes the gradient unchanged.  Reference counterpart: STEQuantizer
    (include/quant/ste_quantizer.h:10-58)."""

    def __init__(self, target_format="Q_1"):
        self.set_target_format(target_format)

    def set_target_format(self, fmt):
        self._fmt = codec.parse_format(fmt) if isinstance(fmt, str) else int(fmt)

    def target_format(self) -> int: return self._fmt

    def bits_for_format(self, fmt=None) -> int:
        return max(1, int(math.ceil(codec.format_bpw(self._fmt if fmt is None else fmt) - 1e-9)))

    def forward(self, w: torch.Tensor, block: int = 256) -> torch.Tensor:
        q = ste_roundtrip_(w.detach().clone(), self._fmt, block)
        return w + (q - w).detach()

    __call__ = forward

    def forward_mixed(self, w: torch.Tensor, per_block_formats, block_size: int = 256) -> torch.Tensor:
        """A different format for every block of ``block_size`` consecutive weights (the last block may be shorter)."""
        flat = w.detach().float().reshape(-1).cpu().contiguous().numpy()
        nb = (flat.size + block_size - 1) // block_size
        if len(per_block_formats) != nb:
            raise ValueError(f"{nb} blocks need {nb} formats, got {len(per_block_formats)}")
        out = flat.copy()
        for b, f in enumerate(per_block_formats):
            f = codec.parse_format(f) if isinstance(f, str) else int(f)
            seg = flat[b * block_size:(b + 1) * block_size]
            out[b * block_size:(b + 1) * block_size] = codec.dequantize_block(f, codec.quantize_block(f, seg), seg.size)
        q = torch.from_numpy(out).view(w.shape).to(w.dtype).to(w.device)
        return w + (q - w).detach()

    def quantize_with_codebook(self, w: torch.Tensor, codebook) -> torch.Tensor:
        """Snap to the nearest entry of a scalar codebook (after scaling by the tensor's absmax); an untrained codebook is
        trained on ``w`` first.  ``codebook``: an object with ``centroids`` and ``train`` (quant.engines.Codebook)."""
        amax = w.detach().abs().max().clamp(min=1e-30)
        u = (w.detach().float() / amax).reshape(-1)
        if not getattr(codebook, "trained", False):
            codebook.train(u)
            codebook.trained = True
        c = codebook.centroids.to(u.device)
        q = (c[torch.bucketize(u.contiguous(), (c[1:] + c[:-1]) / 2)] * amax).view(w.shape).to(w.dtype)
        return w + (q - w).detach()

    @staticmethod
    def find_scale(x: torch.Tensor) -> float:
        return float(x.detach().abs().max())

    def quantize_Q1(self, src: torch.Tensor):
        """(codes uint8 in {0, 1, 2} for -1 / 0 / +1, scale): ternary with the mean magnitude of the kept weights as scale."""
        x = src.detach().float().reshape(-1)
        thr = 0.7 * x.abs().mean()
        sign = torch.where(x.abs() > thr, x.sign(), torch.zeros_like(x))
        kept = sign != 0
        scale = float(x[kept].abs().mean()) if bool(kept.any()) else 1.0
        return (sign + 1).to(torch.uint8), scale

    def quantize_quant(self, src: torch.Tensor):
        """(4-bit codes uint8 in 0 .. 15, scale) on the symmetric absmax grid with levels -7 .. 7 (code 8 is zero)."""
        x = src.detach().float().reshape(-1)
        scale = self.find_scale(x) / 7.0 or 1.0
        return (torch.clamp(torch.round(x / scale), -7, 7) + 8).to(torch.uint8), scale

    def fake_quantize_qat(self, w: torch.Tensor, scale_override: float = 0.0) -> torch.Tensor:
        bits = min(16, max(2, self.bits_for_format()))
        qmin, qmax = get_qrange(bits, True, True)
        scale = scale_override if scale_override > 0 else (self.find_scale(w) / qmax or 1.0)
        return ste_fake_quantize(w, scale, qmin, qmax)

    def lsq_quantize(self, w: torch.Tensor, scale_param: torch.Tensor) -> torch.Tensor:
        return lsq_fake_quantize(w, scale_param, min(16, max(2, self.bits_for_format())), True)

    def fake_quantize_with_observer(self, w: torch.Tensor, obs, bits: int = 0) -> torch.Tensor:
        return fake_quantize_with_observer(w, obs, bits or min(16, max(2, self.bits_for_format())), True)
