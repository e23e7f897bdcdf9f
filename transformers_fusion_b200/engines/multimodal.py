"""Multimodal engine helpers: turning images, waveforms and clips into token rows, training blocks for the alignment head and
the Perceiver with throughput accounting, sensor and 3-D preprocessing, and the fusion primitives.  Everything here is
tensor code that runs on whatever device its inputs live on.

Reference counterparts: engines/trainer/multimodal/dense/codecs.h:10-85 (PatchEmbed, AudioFramer, VideoSampler, AlignTrainer,
PerceiverTrainer, TokProbe) and modalities.h:12-110 (Modality, Sensor3D, FusionMath)."""
from __future__ import annotations

import enum
import math
import time
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as TF


@dataclass
class CodecStats:
    steps: int = 0
    tokens: int = 0
    tok_per_sec: float = 0.0
    last_loss: float = 0.0


class _Timed:
    def __init__(self):
        self._stats, self._t0 = CodecStats(), time.perf_counter()

    def stats(self) -> CodecStats: return self._stats

    def _account(self, tokens: int, loss: float) -> float:
        s = self._stats
        s.steps, s.tokens, s.last_loss = s.steps + 1, s.tokens + int(tokens), float(loss)
        s.tok_per_sec = s.tokens / max(time.perf_counter() - self._t0, 1e-9)
        return s.last_loss


def _fit_dim(x: torch.Tensor, dim: int) -> torch.Tensor:
    """Bring the last dimension to ``dim`` without learned weights: longer rows are average-pooled, shorter ones tiled."""
    d = x.shape[-1]
    if d == dim:
        return x
    if d > dim:
        return TF.adaptive_avg_pool1d(x.reshape(-1, 1, d), dim).reshape(*x.shape[:-1], dim)
    reps = (dim + d - 1) // d
    return x.repeat(*([1] * (x.dim() - 1)), reps)[..., :dim]


@dataclass
class PatchEmbed:
    """image [C, H, W] -> tokens [N, dim]: non-overlapping ``patch`` x ``patch`` tiles, flattened and fitted to ``dim``."""
    patch: int = 16
    dim: int = 512

    def embed(self, image: torch.Tensor) -> torch.Tensor:
        C, H, W = image.shape
        p = self.patch
        x = image[:, : H // p * p, : W // p * p].float()
        tiles = x.unfold(1, p, p).unfold(2, p, p)                              # [C, H/p, W/p, p, p]
        return _fit_dim(tiles.permute(1, 2, 0, 3, 4).reshape(-1, C * p * p), self.dim)


@dataclass
class AudioFramer:
    """waveform [C, T] -> frames [F, dim]: channels averaged, Hann-windowed frames of ``win`` samples every ``hop``."""
    win: int = 400
    hop: int = 160
    dim: int = 512

    def frame(self, waveform: torch.Tensor) -> torch.Tensor:
        w = waveform.float().mean(0) if waveform.dim() == 2 else waveform.float()
        if w.numel() < self.win:
            w = TF.pad(w, (0, self.win - w.numel()))
        fr = w.unfold(0, self.win, self.hop) * torch.hann_window(self.win, device=w.device)
        return _fit_dim(fr, self.dim)


@dataclass
class VideoSampler:
    """frames [T, C, H, W] -> clips [K, dim]: the frames are split into K equal runs, each averaged over time."""
    clips: int = 8
    dim: int = 512

    def sample(self, frames: torch.Tensor) -> torch.Tensor:
        T = frames.shape[0]
        k = min(self.clips, T)
        edges = torch.linspace(0, T, k + 1).round().long().tolist()
        rows = [frames[a:max(b, a + 1)].float().mean(0).reshape(-1) for a, b in zip(edges[:-1], edges[1:])]
        return _fit_dim(torch.stack(rows), self.dim)


class AlignTrainer(_Timed):
    """Contrastive training of an alignment head (an ``nn.Module`` with ``contrastive_loss(a, b)``) on paired embeddings."""

    def __init__(self, aligner, tokenizer=None, lr: float = 1e-3):
        super().__init__()
        self.aligner, self.tok = aligner, tokenizer
        ps = [p for p in aligner.parameters() if p.requires_grad]
        self.opt = torch.optim.AdamW(ps, lr=lr) if ps else None

    def train_step(self, image_emb: torch.Tensor, text_emb: torch.Tensor) -> float:
        loss = self.aligner.contrastive_loss(image_emb, text_emb)
        if self.opt is not None and loss.requires_grad:
            self.opt.zero_grad(set_to_none=True)
            loss.backward()
            self.opt.step()
        return self._account(image_emb.shape[0] + text_emb.shape[0], float(loss.detach()))


class PerceiverTrainer(_Timed):
    """Regression training of a Perceiver: mean squared error between its latent outputs and the labels."""

    def __init__(self, model, tokenizer=None, lr: float = 1e-3):
        super().__init__()
        self.model, self.tok = model, tokenizer
        self.opt = torch.optim.AdamW(model.parameters(), lr=lr)

    @staticmethod
    def mse(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return (a.float() - b.float()).pow(2).mean()

    def train_step(self, inputs: torch.Tensor, queries: Optional[torch.Tensor], labels: torch.Tensor) -> float:
        out = self.model(inputs, queries) if queries is not None else self.model(inputs)
        loss = self.mse(out, labels)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        return self._account(inputs.shape[-2] * (inputs.shape[0] if inputs.dim() == 3 else 1), float(loss.detach()))


class TokProbe:
    """Coverage checks of a multimodal tokenizer."""

    @staticmethod
    def roundtrip(tok, text: str) -> int:
        """Number of characters at which decode(encode(text)) differs from the text (0 = exact)."""
        back = tok.decode(tok.encode(text)) if hasattr(tok, "decode") else tok.text.decode(tok.text.encode(text))
        return sum(a != b for a, b in zip(text, back)) + abs(len(text) - len(back))

    @staticmethod
    def image_ids(tok, image: torch.Tensor) -> List[int]: return tok.encode_image(image)

    @staticmethod
    def audio_ids(tok, audio: torch.Tensor) -> List[int]: return tok.encode_audio(audio)


class Modality(enum.IntEnum):
    TEXT = 0
    IMAGE = 1
    AUDIO = 2
    VIDEO = 3
    OCR = 4
    SPEECH = 5
    CAPTION = 6
    VQA = 7
    TTI = 8
    TTS = 9
    MEL = 10
    FEAT = 11
    TOKENIZER = 12
    ENCODER = 13
    ALIGN = 14
    PERCEIVER = 15
    POINT3D = 16
    DEPTH = 17
    THERMAL = 18
    MULTISPECTRAL = 19
    HYPERSPECTRAL = 20
    SAR = 21
    LIDAR = 22
    RADAR = 23
    IMU = 24
    GPS = 25


NUM_MODALITIES = len(Modality)


def modality_name(m) -> str:
    return Modality(int(m)).name.lower()


class Sensor3D:
    """Preprocessing of 3-D and sensor inputs into dense tensors a tower can consume."""

    @staticmethod
    def voxelize(points: torch.Tensor, D: int, H: int, W: int) -> torch.Tensor:
        """points [N, 3] -> occupancy counts [D, H, W] over the points' bounding box."""
        p = points.float()
        lo, hi = p.amin(0), p.amax(0)
        u = (p - lo) / (hi - lo).clamp(min=1e-12)
        dims = torch.tensor([D, H, W], device=p.device)
        idx = (u * dims).long().clamp(min=0)
        idx = torch.minimum(idx, dims - 1)
        flat = (idx[:, 0] * H + idx[:, 1]) * W + idx[:, 2]
        return torch.bincount(flat, minlength=D * H * W).float().view(D, H, W)

    @staticmethod
    def depth_to_normals(depth: torch.Tensor) -> torch.Tensor:
        """depth [H, W] -> unit normals [H, W, 3] from central differences (one-sided at the border)."""
        d = depth.float()
        gy, gx = torch.gradient(d)
        n = torch.stack([-gx, -gy, torch.ones_like(d)], -1)
        return n / n.norm(dim=-1, keepdim=True)

    @staticmethod
    def normalize_thermal(thermal: torch.Tensor) -> torch.Tensor:
        t = thermal.float()
        return (t - t.min()) / (t.max() - t.min()).clamp(min=1e-12)

    @staticmethod
    def spectral_index(ms: torch.Tensor, red: int, nir: int) -> torch.Tensor:
        """Normalised difference (NDVI-style) of two bands of ms [C, H, W]."""
        r, n = ms[red].float(), ms[nir].float()
        return (n - r) / (n + r).abs().clamp(min=1e-12)

    @staticmethod
    def hs_pca3(hs: torch.Tensor) -> torch.Tensor:
        """hs [C, H, W] -> the three leading principal components per pixel [3, H, W]."""
        C, H, W = hs.shape
        x = hs.float().reshape(C, -1)
        x = x - x.mean(1, keepdim=True)
        _, vec = torch.linalg.eigh(x @ x.t() / max(1, x.shape[1] - 1))
        k = min(3, C)
        comp = vec[:, -k:].flip(1).t() @ x                                     # leading component first
        return TF.pad(comp, (0, 0, 0, 3 - k)).view(3, H, W)

    @staticmethod
    def sar_to_db(sar: torch.Tensor) -> torch.Tensor:
        return 20.0 * torch.log10(sar.float().abs().clamp(min=1e-12))

    @staticmethod
    def lidar_to_xyz(rng: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
        """range [N], angles [N, 2] (azimuth, elevation in radians) -> xyz [N, 3]."""
        r, az, el = rng.float(), angles[:, 0].float(), angles[:, 1].float()
        return torch.stack([r * el.cos() * az.cos(), r * el.cos() * az.sin(), r * el.sin()], -1)

    @staticmethod
    def radar_speed(radar: torch.Tensor) -> torch.Tensor:
        return torch.hypot(radar[:, 2].float(), radar[:, 3].float())

    @staticmethod
    def imu_tilt(imu: torch.Tensor) -> torch.Tensor:
        """imu [N, 6] (ax, ay, az, gx, gy, gz) -> (roll, pitch) [N, 2] in radians from the accelerometer."""
        ax, ay, az = imu[:, 0].float(), imu[:, 1].float(), imu[:, 2].float()
        return torch.stack([torch.atan2(ay, az), torch.atan2(-ax, torch.sqrt(ay * ay + az * az))], -1)

    @staticmethod
    def gps_local(gps: torch.Tensor, lat0: float, lon0: float) -> torch.Tensor:
        """gps [N, 2] (latitude, longitude in degrees) -> metres east / north of (lat0, lon0), equirectangular."""
        R = 6371000.0
        lat, lon = torch.deg2rad(gps[:, 0].double()), torch.deg2rad(gps[:, 1].double())
        east = (lon - math.radians(lon0)) * math.cos(math.radians(lat0)) * R
        north = (lat - math.radians(lat0)) * R
        return torch.stack([east, north], -1).float()


class FusionMath:
    """Parameter-free cross-modal combination primitives."""

    @staticmethod
    def concat_last(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return torch.cat([a, b], -1)

    @staticmethod
    def gated_sum(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """g a + (1 - g) b with the gate g = sigmoid(mean of a - mean of b) per row: the stream with the larger mean
        activation dominates."""
        g = torch.sigmoid(a.float().mean(-1, keepdim=True) - b.float().mean(-1, keepdim=True))
        return (g * a.float() + (1 - g) * b.float()).to(a.dtype)

    @staticmethod
    def align_matrix(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """Cosine similarity of every row of a [Na, D] with every row of b [Nb, D]."""
        return TF.normalize(a.float(), dim=-1) @ TF.normalize(b.float(), dim=-1).t()

    @staticmethod
    def perceiver_step(latents: torch.Tensor, inputs: torch.Tensor, heads: int = 4) -> torch.Tensor:
        """One weight-free cross-attention read: latents [L, D] query inputs [N, D] (keys = values = inputs) and the result
        is added to the latents."""
        L, D = latents.shape
        h = heads if D % heads == 0 else 1
        q = latents.float().view(L, h, D // h).transpose(0, 1)
        kv = inputs.float().view(-1, h, D // h).transpose(0, 1)
        out = TF.scaled_dot_product_attention(q[None], kv[None], kv[None])[0]
        return (latents.float() + out.transpose(0, 1).reshape(L, D)).to(latents.dtype)
