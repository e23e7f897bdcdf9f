"""Codebooks and per-width quantisation engines (tensor level, on the tensor's own device).

* ``Codebook(bits)``        - scalar codebook with 2^bits fp32 centroids: Lloyd training (quantile init), nearest-centroid
  ``quantize``, ``dequantize``, EMA update from assignments, (de)serialisation.  ``CodebookQ3/Q4/Q6/Q8/Q12`` fix the width.
* ``VectorQuantizer``       - k-means codebook over d-dimensional sub-vectors with straight-through forward.
* ``Q8Engine / Q4Engine / Q2Engine`` - codebook + per-block scale with optional stochastic rounding between neighbours.
* ``QuantEngine``           - ternary {-1, 0, +1} x per-block (128) scale, 2-bit packed, ``quant_gemm``.
* ``TernaryLUT``            - the reference's TL1 / TL2 row streams of ternary weights (2 bits each: 00 = -1, 01 = 0, 10 = +1;
  rows of ceil(K / 4) bytes, or 3 bytes per 12 weights) with its lookup-table product (activations rounded to int8 per row,
  pair sums saturating at int8 in TL1) and the transcode into the packed ternary form of the fused-dequant GEMM.
* ``Q1Engine``              - sign x mean |w|.   ``Q16Engine / Q32Engine`` - fp16 round trip / identity.
* fp8: ``fp8_quantize(x, "e4m3" | "e5m2")`` (max 448, no infinities / max 57344), per-channel variants, ``fp8_quant_gemm``.
* ``quant_error`` (MSE) and ``quant_snr`` (dB).
* ``quant8_quantize_tensor`` - the engines/quant facade: asymmetric uint8 affine or symmetric absmax.

Reference counterparts: src/kernel/kernel_tl.cpp (TL1 :12-89, TL2 :91-186), src/codec/codebook.cpp, vector_quantizer.cpp, quant_engines_{core,fp,quant,quant1,quant2,quant4,quant8}.cpp,
include/quant/quant_engines.h, engines/quant/quantize.cpp."""
from __future__ import annotations

import math
import struct
from typing import Optional, Tuple

import torch
from dataclasses import dataclass


def quant_error(a, b) -> float:
    return float(((a.float() - b.float()) ** 2).mean())


def quant_snr(a, b) -> float:
    n = float(((a.float() - b.float()) ** 2).sum())
    return float("inf") if n == 0 else 10.0 * math.log10(float((a.float() ** 2).sum()) / n)


class Codebook:
    def __init__(self, bits: int, device="cpu"):
        self.bits, self.K = bits, 1 << bits
        p = (torch.arange(self.K, dtype=torch.float64) + 0.5) / self.K
        c = torch.erfinv(2 * p - 1) * math.sqrt(2.0)
        self.centroids = (c / c.abs().max()).float().to(device)

    def train(self, data: torch.Tensor, iters: int = 30, max_samples: int = 1 << 20):
        """Lloyd's algorithm from a quantile initialisation."""
        x = data.detach().float().reshape(-1)
        if x.numel() > max_samples:
            x = x[torch.randint(0, x.numel(), (max_samples,), device=x.device)]
        q = (torch.arange(self.K, device=x.device, dtype=torch.float32) + 0.5) / self.K
        c = torch.quantile(x[: min(x.numel(), 1 << 18)], q)
        cur = torch.sort(self.centroids.to(x.device)).values

        def mse(cc):
            return float(((cc[torch.bucketize(x, (cc[1:] + cc[:-1]) / 2)] - x) ** 2).mean())
        if mse(cur) < mse(c):             # Lloyd only ever lowers the error, so start from the better of the two
            c = cur
        for _ in range(iters):
            idx = torch.bucketize(x, (c[1:] + c[:-1]) / 2)
            s = torch.zeros(self.K, device=x.device).index_add_(0, idx, x)
            n = torch.zeros(self.K, device=x.device).index_add_(0, idx, torch.ones_like(x))
            new = torch.where(n > 0, s / n.clamp(min=1), c)
            new, _ = torch.sort(new)
            if float((new - c).abs().max()) < 1e-7:
                c = new
                break
            c = new
        self.centroids = c
        return self

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        c = self.centroids.to(x.device)
        idx = torch.bucketize(x.float().contiguous(), (c[1:] + c[:-1]) / 2)
        return idx.to(torch.uint8 if self.bits <= 8 else torch.int16)

    def dequantize(self, idx: torch.Tensor) -> torch.Tensor:
        return self.centroids.to(idx.device)[idx.long()]

    def ema_update(self, data: torch.Tensor, assign: torch.Tensor, lr: float):
        """Move every centroid towards the mean of the values assigned to it."""
        x, a = data.float().reshape(-1), assign.long().reshape(-1)
        s = torch.zeros(self.K, device=x.device).index_add_(0, a, x)
        n = torch.zeros(self.K, device=x.device).index_add_(0, a, torch.ones_like(x))
        c = self.centroids.to(x.device)
        self.centroids = torch.where(n > 0, (1 - lr) * c + lr * s / n.clamp(min=1), c)

    def serialize(self) -> bytes:
        fmt = "<f" if self.bits >= 8 else "<e"
        body = b"".join(struct.pack(fmt, float(v)) for v in self.centroids.cpu())
        return struct.pack("<BI", self.bits, self.K) + body

    @classmethod
    def deserialize(cls, raw: bytes):
        bits, K = struct.unpack_from("<BI", raw, 0)
        cb = cls(bits)
        fmt, sz = ("<f", 4) if bits >= 8 else ("<e", 2)
        cb.centroids = torch.tensor([struct.unpack_from(fmt, raw, 5 + i * sz)[0] for i in range(K)])
        return cb

    def serialized_size(self):
        return 5 + self.K * (4 if self.bits >= 8 else 2)


def CodebookQ3(device="cpu"): return Codebook(3, device)
def CodebookQ4(device="cpu"): return Codebook(4, device)
def CodebookQ6(device="cpu"): return Codebook(6, device)
def CodebookQ8(device="cpu"): return Codebook(8, device)
def CodebookQ12(device="cpu"): return Codebook(12, device)


@dataclass
class VQConfig:
    codebook_size: int = 256
    embedding_dim: int = 64
    commitment_weight: float = 0.25
    ema_decay: float = 0.99
    codebook_init_std: float = 1.0
    use_ema: bool = True


@dataclass
class VQResult:
    quantized: torch.Tensor
    indices: torch.Tensor
    commitment_loss: float
    codebook_loss: float


class VectorQuantizer:
    """Learned vector codebook (reference: include/quant/vector_quantizer.h:36-80).  ``train`` fits it with Lloyd iterations;
    ``update_ema`` / ``update_codebook_grad`` are the two online updates used while the encoder that feeds it is training."""

    def __init__(self, num_codes=256, dim: int = 64, device="cpu", seed=0):
        if isinstance(num_codes, VQConfig):
            self.cfg = num_codes
        else:
            self.cfg = VQConfig(codebook_size=num_codes, embedding_dim=dim)
        g = torch.Generator().manual_seed(seed)
        self.codes = (torch.randn(self.cfg.codebook_size, self.cfg.embedding_dim, generator=g) * self.cfg.codebook_init_std).to(device)
        self.dim = self.cfg.embedding_dim
        self._counts = torch.zeros(self.cfg.codebook_size, device=device)       # EMA cluster sizes
        self._sums = self.codes.clone() * 0                                    # EMA cluster sums
        self._hits = torch.zeros(self.cfg.codebook_size, device=device)        # raw assignment counts, for the usage statistics
        self._last_idx = None

    def config(self) -> VQConfig: return self.cfg
    def codebook(self) -> torch.Tensor: return self.codes

    def quantize(self, embeddings: torch.Tensor) -> VQResult:
        """The reference's forward: nearest code per vector plus the two losses (the codebook loss is 0 under EMA updates)."""
        x = embeddings.detach().float()
        idx = self.encode(x)
        q = self.decode(idx, x.shape)
        self._last_idx = idx
        self._hits.index_add_(0, idx.to(self._hits.device), torch.ones(idx.numel(), device=self._hits.device))
        mse = float(((q - x) ** 2).mean())
        return VQResult(q.to(embeddings.dtype), idx.reshape(embeddings.shape[:-1]), mse, 0.0 if self.cfg.use_ema else mse)

    def backward(self, grad_output: torch.Tensor) -> torch.Tensor:
        """Straight-through: the encoder receives the gradient of the quantised output unchanged."""
        return grad_output

    def update_ema(self, embeddings: torch.Tensor, indices: torch.Tensor):
        x = embeddings.detach().float().reshape(-1, self.dim).to(self.codes.device)
        idx = indices.reshape(-1).long().to(self.codes.device)
        d = self.cfg.ema_decay
        n = torch.zeros_like(self._counts).index_add_(0, idx, torch.ones(idx.numel(), device=x.device))
        s = torch.zeros_like(self._sums).index_add_(0, idx, x)
        self._counts.mul_(d).add_(n, alpha=1 - d)
        self._sums.mul_(d).add_(s, alpha=1 - d)
        # Laplace smoothing keeps a code that lost all its members from dividing by zero; it stays where it was instead
        tot = self._counts.sum()
        K = self._counts.numel()
        sm = (self._counts + 1e-5) / (tot + K * 1e-5) * tot
        live = self._counts > 1e-8
        self.codes = torch.where(live[:, None], self._sums / sm[:, None].clamp(min=1e-12), self.codes)

    def update_codebook_grad(self, grad_quantized: torch.Tensor, indices: torch.Tensor, lr: float = 1.0):
        """Gradient form (``use_ema`` off): every code moves against the summed gradient of the positions assigned to it."""
        g = grad_quantized.detach().float().reshape(-1, self.dim).to(self.codes.device)
        idx = indices.reshape(-1).long().to(self.codes.device)
        self.codes = self.codes - lr * torch.zeros_like(self.codes).index_add_(0, idx, g)

    def usage_rate(self) -> float:
        """Fraction of the codes that have been chosen at least once since construction."""
        return float((self._hits > 0).float().mean())

    def perplexity(self) -> float:
        """exp(entropy) of the assignment distribution: the effective number of codes in use."""
        tot = self._hits.sum()
        if tot <= 0:
            return 0.0
        p = self._hits / tot
        return float(torch.exp(-(p[p > 0] * p[p > 0].log()).sum()))

    def train(self, data: torch.Tensor, iters=20):
        x = data.detach().float().reshape(-1, self.dim)
        K = self.codes.shape[0]
        # farthest-first initialisation: every new code is the sample farthest from the codes chosen so far
        sub = x[: min(x.shape[0], 1 << 16)]
        codes = [sub[0]]
        dmin = ((sub - codes[0]) ** 2).sum(1)
        for _ in range(K - 1):
            codes.append(sub[int(dmin.argmax())])
            dmin = torch.minimum(dmin, ((sub - codes[-1]) ** 2).sum(1))
        self.codes = torch.stack(codes).clone()
        for _ in range(iters):
            idx = torch.cdist(x, self.codes).argmin(1)
            s = torch.zeros_like(self.codes).index_add_(0, idx, x)
            n = torch.zeros(K, device=x.device).index_add_(0, idx, torch.ones(x.shape[0], device=x.device))
            self.codes = torch.where(n[:, None] > 0, s / n[:, None].clamp(min=1), self.codes)
        return self

    def encode(self, x):
        return torch.cdist(x.float().reshape(-1, self.dim), self.codes.to(x.device)).argmin(1)

    def decode(self, idx, shape=None):
        y = self.codes.to(idx.device)[idx]
        return y.reshape(shape) if shape is not None else y

    def forward(self, x):
        """(quantised with straight-through gradient, indices, commitment loss)."""
        idx = self.encode(x)
        q = self.decode(idx, x.shape).to(x.dtype)
        return x + (q - x).detach(), idx, ((q.detach() - x) ** 2).mean()


class _ScalarVQ:
    """Scalar codebook quantiser with online (EMA) centroid updates: the form used for the few most sensitive weights
    (reference: Q8VectorQuantizer / Q4VectorQuantizer, include/quant/vector_quantizer.h:84-140)."""
    SIZE = 256
    DTYPE = torch.float32

    def __init__(self, initial_codebook=None, ema_decay: float = 0.99):
        if initial_codebook is None:
            cb = torch.linspace(-1.0, 1.0, self.SIZE)
        else:
            cb = torch.as_tensor(initial_codebook)
            cb = cb.view(torch.float16).float() if cb.dtype in (torch.uint16, torch.int16) else cb.float()
            if cb.numel() != self.SIZE:
                raise ValueError(f"the codebook needs {self.SIZE} entries")
        self._cb = cb.to(self.DTYPE).clone()
        self.decay = ema_decay
        self._sum = torch.zeros(self.SIZE)
        self._cnt = torch.zeros(self.SIZE)

    def codebook(self) -> torch.Tensor: return self._cb

    def find_nearest(self, value: float) -> int:
        return int((self._cb.float() - float(value)).abs().argmin())

    def _nearest(self, w: torch.Tensor) -> torch.Tensor:
        c, order = self._cb.float().sort()
        x = w.detach().float().reshape(-1)
        pos = torch.bucketize(x.contiguous(), (c[1:] + c[:-1]) / 2)
        return order[pos]

    def _indices(self, stored: torch.Tensor, n: int) -> torch.Tensor:
        return stored.reshape(-1)[:n].long()

    def quantize(self, weights: torch.Tensor) -> torch.Tensor:
        return self._nearest(weights).to(torch.uint8)

    def dequantize(self, indices: torch.Tensor, n: Optional[int] = None) -> torch.Tensor:
        n = indices.numel() if n is None else n
        return self._cb.float()[self._indices(indices, n)]

    def update_ema(self, weights: torch.Tensor, indices: torch.Tensor, n: Optional[int] = None):
        x = weights.detach().float().reshape(-1)
        idx = self._indices(indices, x.numel() if n is None else n)
        x = x[: idx.numel()]
        d = self.decay
        self._cnt.mul_(d).add_(torch.zeros(self.SIZE).index_add_(0, idx, torch.ones(idx.numel())), alpha=1 - d)
        self._sum.mul_(d).add_(torch.zeros(self.SIZE).index_add_(0, idx, x), alpha=1 - d)
        live = self._cnt > 1e-8
        self._cb = torch.where(live, self._sum / self._cnt.clamp(min=1e-12), self._cb.float()).to(self.DTYPE)


class Q8VectorQuantizer(_ScalarVQ):
    """256 fp32 entries; one byte per weight."""


class Q4VectorQuantizer(_ScalarVQ):
    """16 fp16 entries; two indices per byte, the even position in the low nibble."""
    SIZE = 16
    DTYPE = torch.float16

    def quantize(self, weights: torch.Tensor) -> torch.Tensor:
        idx = self._nearest(weights).to(torch.uint8)
        if idx.numel() % 2:
            idx = torch.cat([idx, idx.new_zeros(1)])
        return idx[0::2] | (idx[1::2] << 4)

    def _indices(self, stored: torch.Tensor, n: int) -> torch.Tensor:
        p = stored.reshape(-1)
        return torch.stack([p & 0xF, p >> 4], 1).reshape(-1)[:n].long()

    def dequantize(self, packed: torch.Tensor, n: Optional[int] = None) -> torch.Tensor:
        return super().dequantize(packed, 2 * packed.numel() if n is None else n)

    @staticmethod
    def fp16_to_float(h: int) -> float:
        return float(torch.tensor([h], dtype=torch.int32).to(torch.int16).view(torch.float16)[0])

    @staticmethod
    def float_to_fp16(f: float) -> int:
        return int(torch.tensor([f], dtype=torch.float16).view(torch.int16)[0]) & 0xFFFF


@dataclass
class AudioCodebookConfig:
    num_quantizers: int = 8
    codebook_size: int = 1024
    embedding_dim: int = 128
    commitment_weight: float = 0.25
    ema_decay: float = 0.99


class AudioCodebook:
    """Residual vector quantisation (EnCodec / DAC style): each layer quantises what the layers before it left over, so the
    sum of the chosen entries approaches the input as layers are added.  Reference counterpart: AudioCodebook
    (include/quant/vector_quantizer.h:150-190)."""

    def __init__(self, cfg: Optional[AudioCodebookConfig] = None, seed: int = 0):
        self.cfg = cfg or AudioCodebookConfig()
        c = self.cfg
        self._q = [VectorQuantizer(VQConfig(c.codebook_size, c.embedding_dim, c.commitment_weight, c.ema_decay), seed=seed + i)
                   for i in range(c.num_quantizers)]
        self._commit = self._cbloss = 0.0

    def quantizers(self) -> list: return self._q
    def total_commitment_loss(self) -> float: return self._commit
    def total_codebook_loss(self) -> float: return self._cbloss

    def fit(self, features: torch.Tensor, iters: int = 10):
        """Lloyd-fit every layer on the residual the earlier layers leave."""
        r = features.detach().float().reshape(-1, self.cfg.embedding_dim)
        for q in self._q:
            q.train(r, iters)
            r = r - q.decode(q.encode(r))
        return self

    def encode(self, features: torch.Tensor, update: bool = False) -> torch.Tensor:
        """features [batch, seq, dim] -> indices [num_quantizers, batch, seq]; ``update`` also moves every layer's codebook
        toward its inputs (EMA)."""
        lead = features.shape[:-1]
        r = features.detach().float().reshape(-1, self.cfg.embedding_dim)
        out, self._commit, self._cbloss = [], 0.0, 0.0
        for q in self._q:
            res = q.quantize(r)
            if update:
                q.update_ema(r, res.indices)
            self._commit += self.cfg.commitment_weight * res.commitment_loss
            self._cbloss += res.codebook_loss
            out.append(res.indices.reshape(lead))
            r = r - res.quantized.float()
        return torch.stack(out)

    def decode(self, indices: torch.Tensor) -> torch.Tensor:
        """indices [num_quantizers (or fewer: a coarser reconstruction), batch, seq] -> features [batch, seq, dim]."""
        y = 0
        for q, idx in zip(self._q, indices):
            y = y + q.decode(idx.reshape(-1).long()).float()
        return y.view(*indices.shape[1:], self.cfg.embedding_dim)


class _CodebookEngine:
    bits = 8

    def __init__(self, block_size: int = 256, stochastic: bool = False, seed: int = 0):
        self.cb = Codebook(self.bits)
        self.block, self.stochastic = block_size, stochastic
        self.gen = torch.Generator().manual_seed(seed)

    def train_codebook(self, data):
        x = data.detach().float().reshape(-1)
        self.cb.train(x / x.abs().max().clamp(min=1e-30))
        return self

    def train_codebook_per_block(self, data, block_size=None, lloyd_iters=30):
        bs = block_size or self.block
        x = data.detach().float().reshape(-1)
        n = x.numel() // bs * bs
        blk = x[:n].view(-1, bs)
        self.cb.train((blk / blk.abs().amax(1, keepdim=True).clamp(min=1e-30)).reshape(-1), lloyd_iters)
        return self

    def quantize(self, w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(indices uint8 [n], per-block scales [nblocks])."""
        x = w.detach().float().reshape(-1)
        nb = (x.numel() + self.block - 1) // self.block
        pad = torch.zeros(nb * self.block, device=x.device)
        pad[: x.numel()] = x
        blk = pad.view(nb, self.block)
        s = blk.abs().amax(1).clamp(min=1e-30)
        u = blk / s[:, None]
        c = self.cb.centroids.to(x.device)
        idx = torch.bucketize(u.contiguous(), (c[1:] + c[:-1]) / 2)
        if self.stochastic:
            lo = torch.where(c[idx] > u, (idx - 1).clamp(min=0), idx)
            hi = (lo + 1).clamp(max=self.cb.K - 1)
            span = (c[hi] - c[lo]).clamp(min=1e-12)
            p_hi = ((u - c[lo]) / span).clamp(0, 1)
            r = torch.rand(u.shape, generator=self.gen).to(x.device)
            idx = torch.where(r < p_hi, hi, lo)
        return idx.view(-1)[: x.numel()].to(torch.uint8), s

    def dequantize(self, idx, scales, n=None):
        n = n or idx.numel()
        nb = scales.numel()
        pad = torch.zeros(nb * self.block, dtype=torch.long, device=idx.device)
        pad[: idx.numel()] = idx.long()
        v = self.cb.centroids.to(idx.device)[pad].view(nb, self.block) * scales[:, None]
        return v.view(-1)[:n]

    def roundtrip(self, w):
        i, s = self.quantize(w)
        return self.dequantize(i, s, w.numel()).view(w.shape)

    # ---- the reference's verbs (include/quant/quant_engines.h: Q8Engine / Q4Engine / Q2Engine)
    def codebook(self) -> torch.Tensor:
        return self.cb.centroids

    def enable_stochastic_rounding(self, enable: bool, temperature: float = 1.0):
        self.stochastic, self.stoch_temperature = bool(enable), float(temperature)

    def quantize_per_block(self, data, block_size: Optional[int] = None):
        """(indices, per-block absmax scales) with blocks of ``block_size`` (default: the engine's block)."""
        old, self.block = self.block, block_size or self.block
        try:
            return self.quantize(data)
        finally:
            self.block = old

    def dequantize_per_block(self, indices, scales, n: Optional[int] = None, block_size: Optional[int] = None):
        old, self.block = self.block, block_size or self.block
        try:
            return self.dequantize(indices, scales, n)
        finally:
            self.block = old

    def quantize_tensor(self, data) -> torch.Tensor:
        """Codebook indices of a tensor scaled by its own absmax (one scale for the whole tensor, kept in
        ``last_tensor_scale``): the plain, block-free form."""
        x = data.detach().float().reshape(-1)
        self.last_tensor_scale = float(x.abs().max().clamp(min=1e-30))
        return self.cb.quantize(x / self.last_tensor_scale).to(torch.uint8)

    def dequant_tensor(self, indices, n: Optional[int] = None, scale: Optional[float] = None) -> torch.Tensor:
        v = self.cb.dequantize(indices.long()) * (self.last_tensor_scale if scale is None else scale)
        return v[: n or v.numel()]

    def quant_gemm(self, a, b_idx, M: int, N: int, K: int, scales=None) -> torch.Tensor:
        """a [M, K] @ W^T where W [N, K] is given by its codebook indices: per-block scales when ``scales`` is passed
        (the output of ``quantize``), else the tensor-wide scale of ``quantize_tensor``."""
        w = self.dequantize(b_idx, scales, N * K) if scales is not None else self.dequant_tensor(b_idx, N * K)
        return a.float().reshape(M, K) @ w.view(N, K).t()

    def quantize_per_channel(self, t, channel_dim: int = 0):
        """(indices shaped like ``t``, one absmax scale per slice along ``channel_dim``)."""
        x = t.detach().float().movedim(channel_dim, 0)
        s = x.reshape(x.shape[0], -1).abs().amax(1).clamp(min=1e-30)
        q = self.cb.quantize((x / s.view([-1] + [1] * (x.dim() - 1))).reshape(-1)).view(x.shape).to(torch.uint8)
        return q.movedim(0, channel_dim), s

    def dequantize_per_channel(self, q, scales, channel_dim: int = 0):
        shp = [1] * q.dim()
        shp[channel_dim] = -1
        return self.cb.dequantize(q.long().reshape(-1)).view(q.shape) * scales.view(shp)

    quant_error = staticmethod(quant_error)
    quant_snr = staticmethod(quant_snr)


class Q8Engine(_CodebookEngine):
    bits = 8


class Q4Engine(_CodebookEngine):
    bits = 4


class Q2Engine(_CodebookEngine):
    bits = 2


class QuantEngine:
    """Ternary weights: per block of 128, scale = mean |w|, code = sign(w) where |w| > scale / 2 else 0; 2 bits packed."""

    def __init__(self, block_size=128):
        self.block = block_size

    def quantize(self, w) -> Tuple[torch.Tensor, torch.Tensor]:
        x = w.detach().float().reshape(-1)
        nb = (x.numel() + self.block - 1) // self.block
        pad = torch.zeros(nb * self.block, device=x.device)
        pad[: x.numel()] = x
        blk = pad.view(nb, self.block)
        s = blk.abs().mean(1).clamp(min=1e-30)
        t = torch.where(blk > 0.5 * s[:, None], 2, torch.where(blk < -0.5 * s[:, None], 0, 1)).to(torch.uint8).view(-1)
        t = torch.nn.functional.pad(t, (0, (-t.numel()) % 4))
        packed = t[0::4] | (t[1::4] << 2) | (t[2::4] << 4) | (t[3::4] << 6)
        return packed, s

    def dequantize(self, packed, scales, n):
        t = torch.stack([packed & 3, (packed >> 2) & 3, (packed >> 4) & 3, packed >> 6], -1).reshape(-1).float() - 1
        nb = scales.numel()
        return (t[: nb * self.block].view(nb, self.block) * scales[:, None]).view(-1)[:n]

    quantize_batch = quantize

    def dequantize_batch(self, q):
        return self.dequantize(q[0], q[1], q[0].numel() * 4)

    def quant_gemm(self, a, b_packed, b_scales, M, N, K):
        """a [M, K] @ dequant(b)[N, K]^T."""
        b = self.dequantize(b_packed, b_scales, N * K).view(N, K)
        return a.float().view(M, K) @ b.t()

    def quantize_per_channel(self, t, channel_dim=0):
        x = t.detach().float().transpose(0, channel_dim).contiguous()
        s = x.reshape(x.shape[0], -1).abs().mean(1).clamp(min=1e-30)
        shp = [-1] + [1] * (x.dim() - 1)
        q = torch.where(x > 0.5 * s.view(shp), 1, torch.where(x < -0.5 * s.view(shp), -1, 0)).to(torch.int8)
        return q.transpose(0, channel_dim), s

    def dequantize_per_channel(self, q, scales, channel_dim=0):
        shp = [1] * q.dim()
        shp[channel_dim] = -1
        return q.float() * scales.view(shp)

    quant_error = staticmethod(quant_error)
    quant_snr = staticmethod(quant_snr)


class TernaryLUT:
    """Row streams of ternary weights in the reference's two lookup-table layouts.

    ``kind`` 1 (TL1): a row of K weights is ceil(K / 4) bytes, weight i in bits 2 (i % 4) .. of byte i / 4; the product
    looks pairs of weights up in a 9-entry table of int8 activation sums, each entry saturated to [-128, 127].
    ``kind`` 2 (TL2): 12 weights per 3 bytes (rows padded to whole 3-byte groups), triples looked up in 27-entry tables;
    sums are kept in 32 bits.  Both quantise every activation row to int8 with scale 127 / max |a| and divide the integer
    dot product by that scale."""

    CODE = {-1: 0, 0: 1, 1: 2}

    def __init__(self, kind: int = 1):
        assert kind in (1, 2)
        self.kind = kind

    def row_bytes(self, K: int) -> int:
        return (K + 3) // 4 if self.kind == 1 else (K + 11) // 12 * 3

    def pack(self, t: torch.Tensor) -> torch.Tensor:
        """t [rows, K] with values in {-1, 0, +1} -> uint8 [rows, row_bytes(K)] (padding weights are zeros: code 01)."""
        rows, K = t.shape
        rb = self.row_bytes(K)
        codes = torch.ones((rows, rb * 4), dtype=torch.uint8, device=t.device)
        codes[:, :K] = (t.to(torch.int16) + 1).to(torch.uint8)
        c = codes.view(rows, rb, 4)
        return c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)

    def unpack(self, packed: torch.Tensor, K: int) -> torch.Tensor:
        """uint8 [rows, row_bytes(K)] -> int8 [rows, K]; the unused code 11 reads as +1, as in the reference's decoder."""
        rows = packed.shape[0]
        c = torch.stack([packed & 3, (packed >> 2) & 3, (packed >> 4) & 3, packed >> 6], -1).reshape(rows, -1)[:, :K]
        return torch.where(c == 0, -1, torch.where(c == 1, 0, 1)).to(torch.int8)

    def gemm(self, packed: torch.Tensor, a: torch.Tensor, K: int) -> torch.Tensor:
        """out [rows_w, rows_a] = ternary rows x activation rows with the reference's integer arithmetic (see the class
        docstring); ``a`` is [rows_a, K] floating point."""
        w = self.unpack(packed, K).to(torch.int32)
        af = a.detach().float()
        scale = 127.0 / af.abs().amax(-1).clamp(min=1e-10)
        ai = torch.round(af * scale[:, None]).to(torch.int32)
        if self.kind == 2:
            tot = w.to(torch.float64) @ ai.to(torch.float64).t()
            return (tot / scale[None, :].double()).float()
        Kp = K - (K % 2)
        # pair sums saturate like the int8 table entries they stand for
        ps = (w[:, None, 0:Kp:2] * ai[None, :, 0:Kp:2] + w[:, None, 1:Kp:2] * ai[None, :, 1:Kp:2]).clamp(-128, 127)
        tot = ps.sum(-1)
        if K % 2:
            tot = tot + w[:, None, K - 1] * ai[None, :, K - 1]
        return tot.float() / scale[None, :]

    def to_packed_weight(self, packed: torch.Tensor, K: int, scale=1.0, group: int = 32):
        """The stream as a ``quant.wq.PackedWeight`` (device ternary format: codes x one scale per group) for the
        fused-dequant GEMM; ``scale``: a number or a per-row tensor that the ternary values are multiplied by."""
        from . import wq
        w = self.unpack(packed, K).float()
        s = torch.as_tensor(scale, dtype=torch.float32, device=w.device)
        s = s if s.dim() == 1 else s.expand(w.shape[0])
        return wq.pack_weight(w * s[:, None], "ternary", group, row_scales=s)


class Q1Engine:
    """One bit per weight: sign, with one scale (mean |w|) per tensor or per channel; 8 signs per byte."""

    def quantize(self, w):
        x = w.detach().float().reshape(-1)
        scale = float(x.abs().mean())
        bits = (x >= 0).to(torch.uint8)
        bits = torch.nn.functional.pad(bits, (0, (-bits.numel()) % 8)).view(-1, 8)
        packed = (bits << torch.arange(8, device=x.device, dtype=torch.uint8)).sum(1).to(torch.uint8)
        return packed, scale

    def dequantize(self, packed, scale, n):
        bits = ((packed[:, None] >> torch.arange(8, device=packed.device, dtype=torch.uint8)) & 1).reshape(-1)[:n]
        return (bits.float() * 2 - 1) * scale

    def quant_gemm(self, a, b_packed, b_scale, M, N, K):
        return a.float().view(M, K) @ self.dequantize(b_packed, b_scale, N * K).view(N, K).t()

    def quantize_per_channel(self, t, channel_dim=0):
        x = t.detach().float().transpose(0, channel_dim)
        s = x.reshape(x.shape[0], -1).abs().mean(1)
        return torch.where(x >= 0, 1, -1).to(torch.int8).transpose(0, channel_dim), s

    def dequantize_per_channel(self, q, scales, channel_dim=0):
        shp = [1] * q.dim()
        shp[channel_dim] = -1
        return q.float() * scales.view(shp)

    quantize_batch = quantize

    def dequantize_batch(self, q):
        """``q``: the (packed, scale) pair of ``quantize``; every bit of the packed bytes is decoded."""
        return self.dequantize(q[0], q[1], q[0].numel() * 8)

    quant_error = staticmethod(quant_error)
    quant_snr = staticmethod(quant_snr)


class _FloatEngine:
    """Engines whose "quantisation" is a cast: the same verbs as the integer engines, for code written against them."""
    dtype = torch.float32

    def quantize(self, w):
        return w.detach().to(self.dtype).clone()

    def dequantize(self, q, n: Optional[int] = None):
        v = q.float()
        return v.reshape(-1)[:n] if n else v

    quantize_batch = quantize

    def dequantize_batch(self, q):
        return q.float()

    def quant_gemm(self, a, b_packed, M: int, N: int, K: int):
        return a.float().reshape(M, K) @ b_packed.float().reshape(N, K).t()

    def quantize_per_channel(self, t, channel_dim: int = 0):
        """(cast tensor, unit scales): a cast needs no scale; the scales exist so that callers can treat all engines alike."""
        return self.quantize(t), torch.ones(t.shape[channel_dim], device=t.device)

    def dequantize_per_channel(self, q, scales, channel_dim: int = 0):
        shp = [1] * q.dim()
        shp[channel_dim] = -1
        return q.float() * scales.view(shp)

    quant_error = staticmethod(quant_error)
    quant_snr = staticmethod(quant_snr)


class Q16Engine(_FloatEngine):
    dtype = torch.float16


class Q32Engine(_FloatEngine):
    dtype = torch.float32


_FP8 = {"e4m3": (torch.float8_e4m3fn, 448.0), "e5m2": (torch.float8_e5m2, 57344.0)}


def fp8_quantize(x: torch.Tensor, kind="e4m3", per_channel_dim: Optional[int] = None):
    """(fp8 tensor, scale): x ~ fp8 * scale with the scale mapping the (per-channel) absmax onto the format's maximum."""
    dt, mx = _FP8[kind]
    f = x.detach().float()
    if per_channel_dim is None:
        s = f.abs().max().clamp(min=1e-30) / mx
    else:
        dims = [d for d in range(f.dim()) if d != per_channel_dim]
        s = f.abs().amax(dims, keepdim=True).clamp(min=1e-30) / mx
    return (f / s).clamp(-mx, mx).to(dt), s


def fp8_dequantize(q, scale):
    return q.float() * scale


def fp8_quant_gemm(a, b, kind="e4m3"):
    """a [M, K] @ b [N, K]^T with both operands rounded to fp8 (per-tensor scales); the block-scaled tensor-core version
    lives in quant/fp8.py."""
    qa, sa = fp8_quantize(a, kind)
    qb, sb = fp8_quantize(b, kind)
    return (qa.float() @ qb.float().t()) * (sa * sb)


def quant8_quantize_tensor(t: torch.Tensor, symmetric=False):
    """uint8 affine (scale, zero point) or int8 absmax quantisation of a whole tensor: (q, scale, zero_point)."""
    f = t.detach().float()
    if symmetric:
        s = float(f.abs().max()) / 127.0 or 1.0
        return torch.clamp(torch.round(f / s), -127, 127).to(torch.int8), s, 0
    lo, hi = float(f.min()), float(f.max())
    s = (hi - lo) / 255.0 or 1.0
    zp = int(round(-lo / s))
    return torch.clamp(torch.round(f / s) + zp, 0, 255).to(torch.uint8), s, zp


def quant8_dequantize_tensor(q, scale, zero_point=0):
    return (q.float() - zero_point) * scale


# ---- the reference's fp8 function names (include/quant/quant_engines.h:9-26), both encodings ------------------------------
def _fp8_family(kind):
    dt, mx = _FP8[kind]

    def quantize(val: float) -> int:
        """Bits of one value rounded to the format (saturating at its largest finite value)."""
        return int(torch.tensor([max(-mx, min(mx, float(val)))]).to(dt).view(torch.uint8)[0])

    def dequantize(bits: int) -> float:
        return float(torch.tensor([bits], dtype=torch.uint8).view(dt).float()[0])

    def quantize_tensor(data) -> torch.Tensor:
        return torch.as_tensor(data).float().clamp(-mx, mx).to(dt).view(torch.uint8)

    def dequant_tensor(bits: torch.Tensor, n: Optional[int] = None) -> torch.Tensor:
        v = bits.view(dt).float()
        return v.reshape(-1)[:n] if n else v

    def quant_gemm(a, b_q: torch.Tensor, M: int, N: int, K: int) -> torch.Tensor:
        return a.float().reshape(M, K) @ dequant_tensor(b_q).reshape(N, K).t()

    def quantize_per_channel(t, channel_dim: int = 0):
        q, s = fp8_quantize(t, kind, channel_dim)
        return q.view(torch.uint8), s

    def dequantize_per_channel(q, scales, channel_dim: int = 0):
        return q.view(dt).float() * scales

    return dict(quantize=quantize, dequantize=dequantize, quantize_tensor=quantize_tensor, dequant_tensor=dequant_tensor,
                quant_gemm=quant_gemm, quantize_per_channel=quantize_per_channel, dequantize_per_channel=dequantize_per_channel,
                quant_error=quant_error, quant_snr=quant_snr)


for _kind in ("e4m3", "e5m2"):
    for _name, _fn in _fp8_family(_kind).items():
        globals()[f"fp8_{_kind}_{_name}"] = _fn


def compute_quant_mse(original, reconstructed) -> float:
    return float((original.float() - reconstructed.float()).pow(2).mean())


compute_quant_error = quant_error
compute_quant_snr = quant_snr
