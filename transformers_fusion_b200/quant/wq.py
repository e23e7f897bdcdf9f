"""Weight-only quantised linear layers served by the fused-dequant GEMM (csrc/kernels/gemm_wq.cu).

``pack_weight(w, fmt, group)`` quantises a [N, K] matrix into one of the device formats (int8, int4, mxfp8 = e4m3 with
power-of-two scales per 32, fp4 = e2m1, ternary) and lays codes and scales out tile-major (128 rows x 64 k per tile);
``gemm_wq(x, pw)`` multiplies activations with it without ever materialising the bf16 weights in HBM; ``QuantLinear`` is
the module form; ``from_quant_tensor`` picks the device format closest to a ``.quant`` wire format, so a checkpoint
quantised with ``quant_quantize`` can be served at its own bit width.

Reference counterparts: src/kernel/kernel_quant8.cpp / kernel_quant4.cpp / kernel_tl.cpp (CPU quantised matmuls),
INT8Inference / FP8Inference (src/inference/inference_lowprec.cpp), quant engines (src/codec/quant_engines_*.cpp)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import _lib
from ..ops._lib import c_i, c_ll, c_p, check, ptr, stream

FORMATS = {"int8": 0, "int4": 1, "mxfp8": 2, "fp8": 2, "fp4": 3, "mxfp4": 3, "ternary": 4}
BITS = {0: 8, 1: 4, 2: 8, 3: 4, 4: 2}
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])

_lib.register("tfb_gemm_wq", [c_p, c_ll, c_p, c_p, c_i, c_i, c_p, c_ll, c_i, c_i, c_i, c_p, c_i, c_i, c_p, c_p])
_lib.register("tfb_wq_finalize", [c_p, c_ll, c_p, c_ll, c_i, c_i, c_i, c_p])
_lib.register("tfb_wq_dequant", [c_p, c_p, c_i, c_i, c_p, c_ll, c_i, c_i, c_p])


@dataclass
class PackedWeight:
    codes: torch.Tensor       # uint8, tile-major
    scales: torch.Tensor      # bf16, tile-major
    fmt: int
    group: int
    N: int                    # logical rows / cols
    K: int
    Np: int                   # padded
    Kp: int

    @property
    def bits_per_weight(self):
        return BITS[self.fmt] + 16.0 / self.group


def _quantise(w: torch.Tensor, fmt: int, group: int, pow2_scales: bool, given_scales=None):
    """w [Np, Kp] fp32 -> (codes uint8 [Np, Kp] one code per element, scales fp32 [Np, Kp / group], dequantised fp32).
    ``given_scales`` [Np, Kp / group]: use these instead of deriving them from the data (transcodes of streams that
    carry their own scale)."""
    Np, Kp = w.shape
    g = w.view(Np, Kp // group, group)
    amax = g.abs().amax(-1, keepdim=True).clamp(min=1e-30)
    qmax = {0: 127.0, 1: 7.0, 2: 448.0, 3: 6.0, 4: 1.0}[fmt]
    s = amax / qmax
    if fmt == 4:
        s = g.abs().mean(-1, keepdim=True).clamp(min=1e-30) * 1.0    # ternary: scale = mean |w| (threshold at half of it)
    if given_scales is not None:
        s = given_scales.reshape(Np, Kp // group, 1).float().clamp(min=1e-30)
    elif pow2_scales:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    s = s.to(torch.bfloat16).float()                                  # the kernel sees bf16 scales
    x = g / s
    if fmt == 0:
        c = torch.clamp(torch.round(x), -127, 127)
        deq, codes = c * s, (c.to(torch.int16) & 255).to(torch.uint8)
    elif fmt == 1:
        c = torch.clamp(torch.round(x), -8, 7)
        deq, codes = c * s, (c + 8).to(torch.uint8)
    elif fmt == 2:
        c = torch.clamp(x, -448, 448).to(torch.float8_e4m3fn)
        deq, codes = c.float() * s, c.view(torch.uint8)
    elif fmt == 3:
        mag = x.abs().clamp(max=6.0)
        idx = (mag.unsqueeze(-1) - _E2M1.to(w.device)).abs().argmin(-1)
        sign = (x < 0).to(torch.uint8)
        deq = _E2M1.to(w.device)[idx] * torch.where(x < 0, -1.0, 1.0) * s
        codes = (idx.to(torch.uint8) | (sign << 3))
    else:
        c = torch.where(x > 0.5, 1.0, torch.where(x < -0.5, -1.0, 0.0))
        deq, codes = c * s, (c + 1).to(torch.uint8)
    return codes.view(Np, Kp), s.view(Np, Kp // group), deq.reshape(Np, Kp)


def pack_weight(w: torch.Tensor, fmt="int8", group: int = 64, pow2_scales: Optional[bool] = None,
                row_scales: Optional[torch.Tensor] = None) -> PackedWeight:
    """``row_scales`` [N]: one scale per row, used for every group of that row instead of scales derived from the data."""
    f = FORMATS[fmt] if isinstance(fmt, str) else int(fmt)
    assert group in (32, 64)
    if pow2_scales is None:
        pow2_scales = isinstance(fmt, str) and fmt.startswith("mx")
    N, K = w.shape
    Np, Kp = (N + 127) // 128 * 128, (K + 63) // 64 * 64
    wp = torch.zeros((Np, Kp), dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    given = None
    if row_scales is not None:
        given = torch.ones((Np, Kp // group), dtype=torch.float32, device=w.device)
        given[:N] = row_scales.float().reshape(N, 1)
    codes, scales, _ = _quantise(wp, f, group, pow2_scales, given)
    # pack codes along k
    # order inside a 32-bit word (see gemm_wq.cu): 4-bit: nibble j = element 2j, nibble j + 4 = element 2j + 1 (j < 4);
    # 2-bit: field j = element 2j, field j + 8 = element 2j + 1 (j < 8)
    if f in (1, 3):
        c = codes.view(Np, Kp // 8, 8)
        e = lambda i: c[..., i]
        codes = torch.stack([e(0) | (e(2) << 4), e(4) | (e(6) << 4), e(1) | (e(3) << 4), e(5) | (e(7) << 4)], -1).reshape(Np, Kp // 2)
    elif f == 4:
        c = codes.view(Np, Kp // 16, 16)
        byte = lambda a: c[..., a[0]] | (c[..., a[1]] << 2) | (c[..., a[2]] << 4) | (c[..., a[3]] << 6)
        codes = torch.stack([byte((0, 2, 4, 6)), byte((8, 10, 12, 14)), byte((1, 3, 5, 7)), byte((9, 11, 13, 15))], -1).reshape(Np, Kp // 4)
    rb = codes.shape[1] * 64 // Kp                       # bytes per row per k-block
    NB, KB = Np // 128, Kp // 64
    U = min(16, rb // 2)                                 # unit-major inside a tile: unit u of row r at (u * 128 + r) * U
    ct = codes.view(NB, 128, KB, rb // U, U).permute(0, 2, 3, 1, 4).contiguous()
    st = scales.view(NB, 128, KB, 64 // group).permute(0, 2, 1, 3).contiguous().to(torch.bfloat16)
    return PackedWeight(ct.view(-1), st.view(-1), f, group, N, K, Np, Kp)


def dequant(pw: PackedWeight) -> torch.Tensor:
    """fp32 [N, K] image of a packed weight (the oracle of the kernel)."""
    NB, KB = pw.Np // 128, pw.Kp // 64
    rb = {0: 64, 1: 32, 2: 64, 3: 32, 4: 16}[pw.fmt]
    U = min(16, rb // 2)
    c = pw.codes.view(NB, KB, rb // U, 128, U).permute(0, 3, 1, 2, 4).reshape(pw.Np, KB * rb)
    s = pw.scales.view(NB, KB, 128, 64 // pw.group).permute(0, 2, 1, 3).reshape(pw.Np, pw.Kp // pw.group).float()
    if pw.fmt in (1, 3):
        b = c.view(pw.Np, pw.Kp // 8, 4)
        lo, hi = b & 15, b >> 4                       # nibbles 0, 2, 4, 6 / 1, 3, 5, 7 of the word
        nib = torch.stack([lo, hi], -1).reshape(pw.Np, pw.Kp // 8, 8)          # nibble order 0..7
        c = torch.stack([nib[..., 0], nib[..., 4], nib[..., 1], nib[..., 5], nib[..., 2], nib[..., 6], nib[..., 3], nib[..., 7]],
                        -1).reshape(pw.Np, pw.Kp)
    elif pw.fmt == 4:
        b = c.view(pw.Np, pw.Kp // 16, 4)
        fld = torch.stack([b & 3, (b >> 2) & 3, (b >> 4) & 3, b >> 6], -1).reshape(pw.Np, pw.Kp // 16, 16)   # field order 0..15
        c = torch.stack([fld[..., j // 2 + 8 * (j % 2)] for j in range(16)], -1).reshape(pw.Np, pw.Kp)
    if pw.fmt == 0:
        v = c.view(torch.int8).float()
    elif pw.fmt == 1:
        v = c.float() - 8
    elif pw.fmt == 2:
        v = c.view(torch.float8_e4m3fn).float()
    elif pw.fmt == 3:
        v = _E2M1.to(c.device)[(c & 7).long()] * torch.where((c & 8) > 0, -1.0, 1.0)
    else:
        v = c.float() - 1
    return (v.view(pw.Np, pw.Kp // pw.group, pw.group) * s.unsqueeze(-1)).view(pw.Np, pw.Kp)[: pw.N, : pw.K]


_SCRATCH = {}
LARGE_M = 2048    # from here on a bf16 image in scratch + the plain bf16 GEMM beats dequantising every tile once per M-tile


def dequant_bf16(pw: PackedWeight) -> torch.Tensor:
    """Row-major bf16 image [Np, Kp] of a packed weight in a per-device scratch buffer shared by all weights of that
    size or smaller (overwritten by the next call)."""
    dev = pw.codes.device
    n = pw.Np * pw.Kp
    buf = _SCRATCH.get(dev)
    if buf is None or buf.numel() < n:
        buf = _SCRATCH[dev] = torch.empty(n, dtype=torch.bfloat16, device=dev)
    out = buf[:n].view(pw.Np, pw.Kp)
    check(_lib.lib().tfb_wq_dequant(pw.codes.data_ptr(), pw.scales.data_ptr(), pw.fmt, pw.group, out.data_ptr(), pw.Kp, pw.Np, pw.Kp,
                                    stream()), "wq_dequant")
    return out


_SPLIT_WS = {}


def gemm_wq(x: torch.Tensor, pw: PackedWeight, bias: Optional[torch.Tensor] = None, splits: int = 0,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y [M, N] = x [M, K] @ dequant(pw)^T (+ bias).  bf16 in / out.  M <= 16 (decode): fused-dequant kernel with the deep
    ring and split-K; M < 2048: fused-dequant kernel with 128-row tiles; larger: bf16 image in scratch + bf16 GEMM.
    ``out`` [M, N] bf16: where the result goes (e.g. the staging buffer of a collective)."""
    y = _gemm_wq(x, pw, bias, splits, out)
    if out is not None and y is not out:
        out.copy_(y)
        return out
    return y


def _gemm_wq(x, pw, bias, splits, dst):
    M, K = x.shape
    if not x.is_cuda:
        y = x.float() @ dequant(pw).t()
        return (y + (bias.float() if bias is not None else 0)).to(x.dtype)
    assert x.dtype == torch.bfloat16
    if M >= LARGE_M and splits == 0:
        from ..ops import functional as F
        if K != pw.Kp:
            xp = torch.zeros((M, pw.Kp), dtype=x.dtype, device=x.device)
            xp[:, :K] = x
            x = xp
        bp = None
        if bias is not None:
            bp = torch.zeros(pw.Np, dtype=torch.bfloat16, device=x.device)
            bp[: pw.N] = bias
        return F.gemm(x.contiguous(), dequant_bf16(pw), bias=bp)[:, : pw.N]
    if K != pw.Kp:
        xp = torch.zeros((M, pw.Kp), dtype=x.dtype, device=x.device)
        xp[:, :K] = x
        x = xp
    x = x.contiguous()
    tiles = ((M + 127) // 128) * (pw.Np // 128)
    use_split = splits > 1 or (splits == 0 and tiles * 2 <= 148 and pw.Kp >= 512)
    if use_split:
        # the fp32 workspace of this shape is kept zeroed between uses: the finalize kernel clears what it reads
        key = (x.device, torch.cuda.current_stream(x.device).cuda_stream, M, pw.Np)
        out = _SPLIT_WS.get(key)
        if out is None:
            out = _SPLIT_WS[key] = torch.zeros((M, pw.Np), dtype=torch.float32, device=x.device)
    elif dst is not None and pw.Np == pw.N and dst.is_contiguous() and dst.dtype == torch.bfloat16:
        out = dst
    else:
        out = torch.empty((M, pw.Np), dtype=torch.bfloat16, device=x.device)
    bp = None
    if bias is not None:
        bp = torch.zeros(pw.Np, dtype=torch.bfloat16, device=x.device)
        bp[: pw.N] = bias
    rc = _lib.lib().tfb_gemm_wq(x.data_ptr(), x.stride(0), pw.codes.data_ptr(), pw.scales.data_ptr(), pw.fmt, pw.group, out.data_ptr(),
                                out.stride(0), M, pw.Np, pw.Kp, ptr(bp), splits if use_split else 1, int(use_split),
                                _lib.status_word(x.device).data_ptr(), stream())
    if rc < 1:
        check(rc, "gemm_wq")
    if out.dtype == torch.bfloat16:
        return out if out is dst else out[:, : pw.N]
    # the fp32 split-K sums are rounded straight into the caller's buffer (or a new one) and the workspace is cleared
    if dst is None or dst.dtype != torch.bfloat16 or dst.stride(-1) != 1 or dst.stride(0) % 4 or dst.data_ptr() % 8 or pw.N % 4:
        y = torch.empty((M, pw.N), dtype=torch.bfloat16, device=x.device) if pw.N % 4 == 0 else None
        if y is None:                          # odd widths: plain cast, explicit clear
            y = out[:, : pw.N].to(torch.bfloat16)
            out.zero_()
            return y
    else:
        y = dst
    check(_lib.lib().tfb_wq_finalize(out.data_ptr(), out.stride(0), y.data_ptr(), y.stride(0), M, pw.N, pw.Np, stream()),
          "wq_finalize")
    return y


class QuantLinear(torch.nn.Module):
    def __init__(self, weight: torch.Tensor, fmt="int8", group=64, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.pw = pack_weight(weight, fmt, group)
        self.bias = bias

    def forward(self, x):
        shp = x.shape
        return gemm_wq(x.reshape(-1, shp[-1]), self.pw, self.bias).view(*shp[:-1], self.pw.N)

    def extra_repr(self):
        return f"N={self.pw.N}, K={self.pw.K}, {self.pw.bits_per_weight:.2f} bits/weight"


def device_format_for(wire_format_name: str):
    """Device format that serves a ``.quant`` wire format at (about) its own width: (fmt, group)."""
    n = wire_format_name.upper()
    bits = int("".join(ch for ch in n.split("_K")[0].replace("Q_G_", "").replace("Q_MX_", "").replace("Q_", "").split("_")[0] if ch.isdigit()) or 32)
    if bits <= 2:
        return "ternary", 32
    if bits <= 4:
        return ("int4", 32) if "G" in n else ("fp4", 32)
    if bits <= 8:
        return ("mxfp8", 32) if "MX" in n else ("int8", 64)
    return None, 0                                  # 12 bits and up: keep bf16


def quantize_model_linears(model, fmt="int8", group=64, min_numel=1 << 14):
    """{parameter name: PackedWeight} for every matrix of the model's blocks (norms, embeddings and the head stay bf16)."""
    out = {}
    for i, l in enumerate(model.layers):
        for name in ("qkv", "o", "gate_up", "down"):
            w = getattr(l, name).data
            if w.numel() >= min_numel:
                out[f"layers.{i}.{name}"] = pack_weight(w, fmt, group)
    return out
