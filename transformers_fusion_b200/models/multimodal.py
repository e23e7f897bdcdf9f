"""Multimodal encoders, fusion and task heads.

Vision (patch embedding + transformer), audio (mel spectrogram, strided 1-D convolutional front end + transformer), text
tower, cross-attention blocks, the shared fusion encoder, contrastive alignment, Perceiver resampling, modality-specific
mixture-of-experts layers and thin task heads (classification, CTC speech recognition, OCR, video, captioning, VQA,
text-to-image token decoding, Griffin-Lim audio synthesis).  Linear layers run on the framework's GEMM kernel and attention
on its flash-attention kernel whenever the tensors are bf16 on a CUDA device and no autograd graph is being recorded;
otherwise they take the equivalent torch path (which is also their test oracle).

Reference counterparts: include/quant/multimodal_cross_attn.h (PatchEmbedding :70, VisionTransformer :81, Conv1DExtractor
:127, AudioTransformer :137, CrossAttentionBlock :182, ModalityFusionEncoder :215, ContrastiveAlignmentHead :256,
MultimodalCrossAttention :274), include/quant/multimodal.h (task heads, MelSpectrogram, Perceiver, modality MoEs, fusion),
image.h / audio.h / video.h / vision.h / ocr.h / text.h / embeddings.h."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F


# ================================================================================================ building blocks
class TFLinear(nn.Module):
    def __init__(self, in_f, out_f, bias=True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_f, in_f))
        self.bias = nn.Parameter(torch.zeros(out_f)) if bias else None
        nn.init.normal_(self.weight, std=math.sqrt(2.0 / (in_f + out_f)))

    def forward(self, x):
        fast = x.is_cuda and x.dtype == torch.bfloat16 and not (torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad))
        if fast:
            shp = x.shape
            y = F.gemm(x.reshape(-1, shp[-1]).contiguous(), self.weight.data.to(torch.bfloat16),
                       bias=self.bias.data.to(torch.bfloat16) if self.bias is not None else None)
            return y.view(*shp[:-1], -1)
        return TF.linear(x, self.weight.to(x.dtype), self.bias.to(x.dtype) if self.bias is not None else None)


def attention(q, k, v, num_heads, causal=False):
    """q [B, Sq, H], k / v [B, Sk, H] -> [B, Sq, H]."""
    B, Sq, H = q.shape
    Sk, D = k.shape[1], H // num_heads
    fast = q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and Sq == Sk and not torch.is_grad_enabled()
    if fast:
        o, _ = F.attn_fwd(q.reshape(B * Sq, H).contiguous(), k.reshape(B * Sk, H).contiguous(), v.reshape(B * Sk, H).contiguous(),
                          B, Sq, num_heads, num_heads, D, causal=causal)
        return o.view(B, Sq, H)
    qh, kh, vh = (t.view(B, -1, num_heads, D).transpose(1, 2) for t in (q, k, v))
    return TF.scaled_dot_product_attention(qh, kh, vh, is_causal=causal).transpose(1, 2).reshape(B, Sq, H)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        f = x.float()
        return (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


class EncoderBlock(nn.Module):
    def __init__(self, dim, heads, mlp_dim, rms=True, eps=1e-5):
        super().__init__()
        self.heads = heads
        self.n1 = RMSNorm(dim, eps) if rms else nn.LayerNorm(dim, eps)
        self.n2 = RMSNorm(dim, eps) if rms else nn.LayerNorm(dim, eps)
        self.qkv, self.o = TFLinear(dim, 3 * dim), TFLinear(dim, dim)
        self.up, self.down = TFLinear(dim, mlp_dim), TFLinear(mlp_dim, dim)

    def forward(self, x, causal=False):
        q, k, v = self.qkv(self.n1(x)).chunk(3, -1)
        x = x + self.o(attention(q, k, v, self.heads, causal))
        return x + self.down(TF.gelu(self.up(self.n2(x)), approximate="tanh"))


@dataclass
class ViTConfig:
    image_size: int = 224
    patch_size: int = 16
    in_channels: int = 3
    hidden_dim: int = 768
    num_heads: int = 12
    num_layers: int = 12
    mlp_dim: int = 3072
    dropout: float = 0.1


class PatchEmbedding(nn.Module):
    """Non-overlapping patches flattened and projected: [B, C, H, W] -> [B, (H/p)(W/p), hidden]."""

    def __init__(self, cfg: ViTConfig):
        super().__init__()
        self.p = cfg.patch_size
        self.proj = TFLinear(cfg.in_channels * cfg.patch_size ** 2, cfg.hidden_dim)

    def forward(self, img):
        B, C, H, W = img.shape
        p = self.p
        x = img.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)
        return self.proj(x)


class _TowerAPI:
    """The reference's encoder verbs on every tower (include/quant/{vision,audio,video,text}.h): ``init`` (re-)draws the
    weights, ``is_initialized`` says whether weights exist, ``encode`` returns pooled features, ``hidden_size`` their width."""

    def init(self, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for p_ in self.parameters():
                if p_.dim() >= 2:
                    p_.copy_((torch.randn(p_.shape, generator=g) * (1.0 / math.sqrt(p_.shape[-1]))).to(p_.dtype))
        self._initialized = True
        return self

    def is_initialized(self) -> bool:
        return getattr(self, "_initialized", True) and any(True for _ in self.parameters())

    def hidden_size(self) -> int:
        c = getattr(self, "cfg", None)
        for name in ("hidden_dim", "shared_hidden", "hidden"):
            if c is not None and hasattr(c, name):
                return int(getattr(c, name))
        return int(getattr(self, "dim", 0))

    d_model = hidden_size

    @torch.no_grad()
    def encode(self, x, *args, **kw):
        """Pooled features [B, hidden] of a batch (a single unbatched item gets a batch dimension)."""
        out = self(x, *args, **kw)
        out = out[0] if isinstance(out, tuple) else out
        return out if out.dim() == 2 else out.mean(1)


class VisionTransformer(_TowerAPI, nn.Module):
    def __init__(self, cfg: Optional[ViTConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or ViTConfig()
        n = (cfg.image_size // cfg.patch_size) ** 2
        self.patch = PatchEmbedding(cfg)
        self.cls = nn.Parameter(torch.zeros(1, 1, cfg.hidden_dim))
        self.pos = nn.Parameter(torch.randn(1, n + 1, cfg.hidden_dim) * 0.02)
        self.blocks = nn.ModuleList(EncoderBlock(cfg.hidden_dim, cfg.num_heads, cfg.mlp_dim, rms=False) for _ in range(cfg.num_layers))
        self.norm = nn.LayerNorm(cfg.hidden_dim)

    def forward(self, img, return_tokens=False):
        x = self.patch(img)
        x = torch.cat([self.cls.to(x.dtype).expand(x.shape[0], -1, -1), x], 1) + self.pos.to(x.dtype)[:, : x.shape[1] + 1]
        for b in self.blocks:
            x = b(x)
        x = self.norm(x)
        return x if return_tokens else x[:, 0]

    def config(self) -> ViTConfig: return self.cfg
    def patch_embed(self, img): return self.patch(img)

    @torch.no_grad()
    def get_patch_features(self, img):
        """Per-patch features [B, patches, hidden] (the class token is left out)."""
        return self(img, return_tokens=True)[:, 1:]


@dataclass
class AudioEncoderConfig:
    input_dim: int = 80
    hidden_dim: int = 384
    num_heads: int = 6
    num_layers: int = 6
    kernel_size: int = 31
    dropout: float = 0.1


class Conv1DExtractor(nn.Module):
    """Two strided 1-D convolutions over time (4x down-sampling): [B, T, n_mels] -> [B, T/4, hidden]."""

    def __init__(self, in_dim, hidden, kernel_size=3):
        super().__init__()
        self.c1 = nn.Conv1d(in_dim, hidden, kernel_size, stride=2, padding=kernel_size // 2)
        self.c2 = nn.Conv1d(hidden, hidden, kernel_size, stride=2, padding=kernel_size // 2)

    def forward(self, x):
        y = TF.gelu(self.c1(x.transpose(1, 2).float()))
        return TF.gelu(self.c2(y)).transpose(1, 2).to(x.dtype)


class AudioTransformer(_TowerAPI, nn.Module):
    def __init__(self, cfg: Optional[AudioEncoderConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or AudioEncoderConfig()
        self.front = Conv1DExtractor(cfg.input_dim, cfg.hidden_dim, 3)
        self.blocks = nn.ModuleList(EncoderBlock(cfg.hidden_dim, cfg.num_heads, 4 * cfg.hidden_dim) for _ in range(cfg.num_layers))
        self.norm = RMSNorm(cfg.hidden_dim)

    @staticmethod
    def _sinusoid(n, d, device, dtype):
        pos = torch.arange(n, device=device).float()[:, None]
        i = torch.arange(0, d, 2, device=device).float()[None]
        ang = pos / (10000 ** (i / d))
        return torch.cat([ang.sin(), ang.cos()], -1)[:, :d].to(dtype)

    def forward(self, mel, return_tokens=True):
        x = self.front(mel)
        x = x + self._sinusoid(x.shape[1], x.shape[2], x.device, x.dtype)
        for b in self.blocks:
            x = b(x)
        x = self.norm(x)
        return x if return_tokens else x.mean(1)

    def config(self) -> AudioEncoderConfig: return self.cfg
    def n_mels(self) -> int: return self.cfg.input_dim
    def sample_rate(self) -> int: return int(getattr(self.cfg, "sample_rate", 16000))


@dataclass
class CrossAttentionLayerConfig:
    hidden_size: int = 768
    num_heads: int = 8
    head_dim: int = 96
    dropout_rate: float = 0.1
    use_rms_norm: bool = True
    norm_eps: float = 1e-5


class CrossAttentionBlock(nn.Module):
    """Queries from one modality attend over keys / values of another; pre-norm, residual, followed by an MLP."""

    def __init__(self, cfg: Optional[CrossAttentionLayerConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or CrossAttentionLayerConfig()
        inner = cfg.num_heads * cfg.head_dim
        Norm = (lambda d: RMSNorm(d, cfg.norm_eps)) if cfg.use_rms_norm else (lambda d: nn.LayerNorm(d, cfg.norm_eps))
        self.nq, self.nkv, self.nm = Norm(cfg.hidden_size), Norm(cfg.hidden_size), Norm(cfg.hidden_size)
        self.q, self.k, self.v = TFLinear(cfg.hidden_size, inner, False), TFLinear(cfg.hidden_size, inner, False), TFLinear(cfg.hidden_size, inner, False)
        self.o = TFLinear(inner, cfg.hidden_size, False)
        self.up, self.down = TFLinear(cfg.hidden_size, 4 * cfg.hidden_size), TFLinear(4 * cfg.hidden_size, cfg.hidden_size)

    def forward(self, x, context, context_mask=None):
        c = self.cfg
        B, Sq, _ = x.shape
        q = self.q(self.nq(x)).view(B, Sq, c.num_heads, c.head_dim).transpose(1, 2)
        ctx = self.nkv(context)
        k = self.k(ctx).view(B, -1, c.num_heads, c.head_dim).transpose(1, 2)
        v = self.v(ctx).view(B, -1, c.num_heads, c.head_dim).transpose(1, 2)
        mask = None if context_mask is None else context_mask[:, None, None, :].bool()
        a = TF.scaled_dot_product_attention(q, k, v, attn_mask=mask).transpose(1, 2).reshape(B, Sq, -1)
        x = x + self.o(a)
        return x + self.down(TF.gelu(self.up(self.nm(x)), approximate="tanh"))

    def forward_self_attn(self, x, mask=None):
        """The block applied to a sequence that attends to itself."""
        return self.forward(x, x, mask)


@dataclass
class MultimodalEncoderConfig:
    image_patch_size: int = 16
    image_size: int = 224
    image_channels: int = 3
    image_embed_dim: int = 768
    image_num_layers: int = 12
    image_num_heads: int = 12
    audio_sample_rate: int = 16000
    audio_n_mels: int = 80
    audio_frame_size: int = 400
    audio_hop_size: int = 160
    audio_embed_dim: int = 384
    audio_num_layers: int = 6
    audio_num_heads: int = 6
    text_vocab_size: int = 32000
    text_embed_dim: int = 768
    text_max_len: int = 2048
    text_num_layers: int = 12
    text_num_heads: int = 12
    shared_hidden: int = 768
    shared_num_heads: int = 12
    shared_num_layers: int = 4
    modality_dropout: float = 0.1


class TextEncoder(_TowerAPI, nn.Module):
    def __init__(self, vocab, dim, layers, heads, max_len=2048, causal=False):
        super().__init__()
        self.emb, self.dim = nn.Embedding(vocab, dim), dim
        self.pos = nn.Parameter(torch.randn(1, max_len, dim) * 0.02)
        self.blocks = nn.ModuleList(EncoderBlock(dim, heads, 4 * dim) for _ in range(layers))
        self.norm, self.causal = RMSNorm(dim), causal

    def forward(self, ids, return_tokens=True):
        x = self.emb(ids) + self.pos[:, : ids.shape[1]]
        for b in self.blocks:
            x = b(x, self.causal)
        x = self.norm(x)
        return x if return_tokens else x.mean(1)


class ModalityProjection(nn.Module):
    def __init__(self, in_dim, out_dim):
        super().__init__()
        self.proj, self.norm = TFLinear(in_dim, out_dim), RMSNorm(out_dim)

    def forward(self, x):
        return self.norm(self.proj(x))

    project = forward
    project_vision = project_audio = project_text = forward      # one projection per instance: the names say what it is used for


class ModalityFusionEncoder(nn.Module):
    """Projects every modality's tokens into the shared width, tags them with a learned modality embedding, concatenates
    them and runs the shared transformer; modalities that are absent (None) are simply left out."""

    MODALITIES = ("image", "audio", "text")

    def __init__(self, cfg: Optional[MultimodalEncoderConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or MultimodalEncoderConfig()
        dims = {"image": cfg.image_embed_dim, "audio": cfg.audio_embed_dim, "text": cfg.text_embed_dim}
        self.proj = nn.ModuleDict({m: ModalityProjection(d, cfg.shared_hidden) for m, d in dims.items()})
        self.tag = nn.ParameterDict({m: nn.Parameter(torch.randn(1, 1, cfg.shared_hidden) * 0.02) for m in dims})
        self.blocks = nn.ModuleList(EncoderBlock(cfg.shared_hidden, cfg.shared_num_heads, 4 * cfg.shared_hidden)
                                    for _ in range(cfg.shared_num_layers))
        self.norm = RMSNorm(cfg.shared_hidden)

    def forward(self, image=None, audio=None, text=None):
        parts, spans, o = [], {}, 0
        for name, t in (("image", image), ("audio", audio), ("text", text)):
            if t is None:
                continue
            if self.training and self.cfg.modality_dropout > 0 and len(parts) > 0 and torch.rand(()) < self.cfg.modality_dropout:
                continue
            p = self.proj[name](t) + self.tag[name].to(t.dtype)
            parts.append(p)
            spans[name] = (o, o + p.shape[1])
            o += p.shape[1]
        x = torch.cat(parts, 1)
        for b in self.blocks:
            x = b(x)
        return self.norm(x), spans

    # ---- named fusion modes (reference: ModalityFusionEncoder, include/quant/multimodal_cross_attn.h)
    def fuse(self, image=None, audio=None, text=None):
        """Fused token sequence [B, tokens, hidden] (early fusion, the module's forward)."""
        return self(image, audio, text)[0]

    fuse_early = fuse

    def fuse_late(self, image=None, audio=None, text=None):
        """Late fusion: every modality runs through the shared transformer on its own and the pooled results are
        averaged -> [B, hidden]."""
        pooled = []
        for name, t in (("image", image), ("audio", audio), ("text", text)):
            if t is not None:
                pooled.append(self(**{name: t})[0].mean(1))
        return torch.stack(pooled).mean(0)

    def get_per_modality_features(self, image=None, audio=None, text=None):
        """{modality: pooled features [B, hidden]} read from the early-fused sequence."""
        x, spans = self(image, audio, text)
        return {m: x[:, a:b].mean(1) for m, (a, b) in spans.items()}

    def apply_modality_dropout(self, feats: dict, p: Optional[float] = None, generator=None) -> dict:
        """Drop whole modalities with probability ``p`` (at least one always survives): {name: tensor or None}."""
        p = self.cfg.modality_dropout if p is None else p
        names = [m for m, t in feats.items() if t is not None]
        keep = [m for m in names if float(torch.rand((), generator=generator)) >= p]
        if not keep and names:
            keep = [names[int(torch.randint(len(names), (), generator=generator))]]
        return {m: (t if m in keep else None) for m, t in feats.items()}


class ContrastiveAlignmentHead(nn.Module):
    """CLIP-style symmetric InfoNCE between two pooled embeddings with a learned temperature."""

    def __init__(self, dim_a, dim_b, proj_dim=256, init_temperature=0.07):
        super().__init__()
        self.pa, self.pb = TFLinear(dim_a, proj_dim, False), TFLinear(dim_b, proj_dim, False)
        self.logit_scale = nn.Parameter(torch.tensor(math.log(1.0 / init_temperature)))

    def embed(self, a, b):
        return TF.normalize(self.pa(a).float(), dim=-1), TF.normalize(self.pb(b).float(), dim=-1)

    def similarity(self, a, b):
        ea, eb = self.embed(a, b)
        return self.logit_scale.exp().clamp(max=100.0) * ea @ eb.t()

    def forward(self, a, b):
        s = self.similarity(a, b)
        t = torch.arange(s.shape[0], device=s.device)
        return 0.5 * (TF.cross_entropy(s, t) + TF.cross_entropy(s.t(), t))

    # ---- the reference's names (include/quant/multimodal_cross_attn.h: ContrastiveAlignmentHead)
    def project(self, x, which: str = "a"):
        return TF.normalize((self.pa if which == "a" else self.pb)(x).float(), dim=-1)

    def align_features(self, a, b):
        return self.embed(a, b)

    compute_clip_loss = forward

    def compute_infonce_loss(self, a, b):
        """One-directional InfoNCE: each row of ``a`` must pick its own row of ``b``."""
        s = self.similarity(a, b)
        return TF.cross_entropy(s, torch.arange(s.shape[0], device=s.device))

    def get_temperature(self) -> float:
        return float(1.0 / self.logit_scale.exp())

    def set_temperature(self, t: float):
        with torch.no_grad():
            self.logit_scale.fill_(math.log(1.0 / max(float(t), 1e-4)))


class MultimodalCrossAttention(nn.Module):
    """Towers + fusion encoder + text-queries-image/audio cross attention + alignment heads."""

    def __init__(self, cfg: Optional[MultimodalEncoderConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or MultimodalEncoderConfig()
        self.vision = VisionTransformer(ViTConfig(cfg.image_size, cfg.image_patch_size, cfg.image_channels, cfg.image_embed_dim,
                                                  cfg.image_num_heads, cfg.image_num_layers, 4 * cfg.image_embed_dim))
        self.audio = AudioTransformer(AudioEncoderConfig(cfg.audio_n_mels, cfg.audio_embed_dim, cfg.audio_num_heads, cfg.audio_num_layers))
        self.text = TextEncoder(cfg.text_vocab_size, cfg.text_embed_dim, cfg.text_num_layers, cfg.text_num_heads, cfg.text_max_len)
        self.fusion = ModalityFusionEncoder(cfg)
        self.xattn = CrossAttentionBlock(CrossAttentionLayerConfig(cfg.shared_hidden, cfg.shared_num_heads, cfg.shared_hidden // cfg.shared_num_heads))
        self.align_it = ContrastiveAlignmentHead(cfg.image_embed_dim, cfg.text_embed_dim)
        self.align_at = ContrastiveAlignmentHead(cfg.audio_embed_dim, cfg.text_embed_dim)

    def forward(self, image=None, mel=None, text_ids=None):
        iv = self.vision(image, return_tokens=True) if image is not None else None
        av = self.audio(mel) if mel is not None else None
        tv = self.text(text_ids) if text_ids is not None else None
        fused, spans = self.fusion(iv, av, tv)
        out = {"fused": fused, "spans": spans}
        if tv is not None and "text" in spans and len(spans) > 1:
            lo, hi = spans["text"]
            ctx = torch.cat([fused[:, a:b] for m, (a, b) in spans.items() if m != "text"], 1)
            out["text_grounded"] = self.xattn(fused[:, lo:hi], ctx)
        if iv is not None and tv is not None:
            out["loss_image_text"] = self.align_it(iv[:, 0], tv.mean(1))
        if av is not None and tv is not None:
            out["loss_audio_text"] = self.align_at(av.mean(1), tv.mean(1))
        return out


def _mmca_api():
    """High-level verbs of the joint model (reference: MultimodalCrossAttention, include/quant/multimodal_cross_attn.h)."""
    M = MultimodalCrossAttention

    def config(self): return self.cfg
    def vision_encoder(self): return self.vision
    def audio_encoder(self): return self.audio
    def text_embedding(self): return self.text
    def contrastive_head(self, pair: str = "image_text"): return self.align_it if pair == "image_text" else self.align_at

    @torch.no_grad()
    def encode_image(self, image): return self.vision(image, return_tokens=False)

    @torch.no_grad()
    def encode_audio(self, mel): return self.audio(mel, return_tokens=False)

    @torch.no_grad()
    def encode_text(self, text_ids): return self.text(text_ids, return_tokens=False)

    def forward_text_image(self, text_ids, image):
        """Text tokens grounded in the image: [B, text tokens, shared hidden]."""
        return self(image=image, text_ids=text_ids)["text_grounded"]

    def forward_text_audio(self, text_ids, mel):
        return self(mel=mel, text_ids=text_ids)["text_grounded"]

    def add_image_tokens(self, image):
        """Shared-width tokens of an image, tagged as image tokens (what the fusion encoder concatenates)."""
        return self.fusion.proj["image"](self.vision(image, return_tokens=True)) + self.fusion.tag["image"]

    def add_audio_tokens(self, mel):
        return self.fusion.proj["audio"](self.audio(mel)) + self.fusion.tag["audio"]

    def add_text_tokens(self, text_ids):
        return self.fusion.proj["text"](self.text(text_ids)) + self.fusion.tag["text"]

    @torch.no_grad()
    def retrieve_images(self, text_ids, images, top_k: int = 5):
        """Indices and similarities of the images that match one text best (alignment-head similarity)."""
        sim = self.align_it.similarity(self.encode_image(images), self.encode_text(text_ids))[:, 0]
        v, i = sim.topk(min(top_k, sim.numel()))
        return i.tolist(), v.tolist()

    @torch.no_grad()
    def retrieve_text(self, image, texts_ids, top_k: int = 5):
        sim = self.align_it.similarity(self.encode_image(image), self.encode_text(texts_ids))[0]
        v, i = sim.topk(min(top_k, sim.numel()))
        return i.tolist(), v.tolist()

    def _vocab_logits(self, grounded):
        """Grounded text states scored against the text tower's embedding table (tied read-out through the fusion's text
        projection): [B, T, vocab]."""
        table = self.fusion.proj["text"](self.text.emb.weight[None])[0]
        return grounded @ table.t()

    @torch.no_grad()
    def generate_caption(self, image, bos: int = 1, eos: int = 2, max_tokens: int = 16):
        """Greedy caption ids for ONE image [1, C, H, W]: the next token is read from the last grounded text state."""
        ids = [bos]
        for _ in range(max_tokens):
            g = self.forward_text_image(torch.tensor([ids], device=image.device), image)
            nxt = int(self._vocab_logits(g)[0, -1].argmax())
            ids.append(nxt)
            if nxt == eos:
                break
        return ids[1:]

    @torch.no_grad()
    def visual_question_answer(self, image, question_ids, max_tokens: int = 8, eos: int = 2):
        """Greedy answer ids that continue the question, grounded in the image."""
        ids = list(question_ids[0].tolist() if torch.is_tensor(question_ids) else question_ids)
        out = []
        for _ in range(max_tokens):
            g = self.forward_text_image(torch.tensor([ids + out], device=image.device), image)
            nxt = int(self._vocab_logits(g)[0, -1].argmax())
            out.append(nxt)
            if nxt == eos:
                break
        return out

    for name, fn in list(locals().items()):
        if callable(fn) and name not in ("M",):
            setattr(M, name, fn)


_mmca_api()


class CrossModalAttention(CrossAttentionBlock):
    pass


class Perceiver(nn.Module):
    """A fixed number of learned queries cross-attend over an arbitrarily long input: [B, N, H] -> [B, num_queries, H]."""

    def __init__(self, hidden, num_queries, num_heads):
        super().__init__()
        self.heads = num_heads
        self.queries = nn.Parameter(torch.randn(1, num_queries, hidden) * 0.02)
        self.q, self.k, self.v, self.o = (TFLinear(hidden, hidden, False) for _ in range(4))

    def forward(self, x, queries=None):
        B, H = x.shape[0], x.shape[2]
        q = self.q((queries if queries is not None else self.queries.to(x.dtype)).expand(B, -1, -1))
        D = H // self.heads
        qh = q.view(B, -1, self.heads, D).transpose(1, 2)
        kh = self.k(x).view(B, -1, self.heads, D).transpose(1, 2)
        vh = self.v(x).view(B, -1, self.heads, D).transpose(1, 2)
        return self.o(TF.scaled_dot_product_attention(qh, kh, vh).transpose(1, 2).reshape(B, -1, H))


# ================================================================================================ audio front end
class MelSpectrogram:
    """Log-mel spectrogram: Hann-windowed STFT -> power -> triangular mel filter bank -> log."""

    def __init__(self, sample_rate=22050, n_mels=80, n_fft=400, hop=160):
        self.sr, self.n_mels, self.n_fft, self.hop = sample_rate, n_mels, n_fft, hop
        self.fb = self.mel_filterbank(n_mels, n_fft, sample_rate)

    @staticmethod
    def mel_filterbank(n_filters, fft_size, sample_rate):
        hz2mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)
        mel2hz = lambda m: 700.0 * (10 ** (m / 2595.0) - 1.0)
        pts = torch.tensor([mel2hz(m) for m in torch.linspace(hz2mel(0.0), hz2mel(sample_rate / 2), n_filters + 2).tolist()])
        bins = torch.linspace(0, sample_rate / 2, fft_size // 2 + 1)
        fb = torch.zeros(n_filters, fft_size // 2 + 1)
        for i in range(n_filters):
            l, c, r = pts[i], pts[i + 1], pts[i + 2]
            fb[i] = torch.clamp(torch.minimum((bins - l) / (c - l), (r - bins) / (r - c)), min=0)
        return fb

    def init(self, sample_rate: Optional[int] = None, n_mels: Optional[int] = None):
        """Rebuild the filter bank for another sample rate / number of bands."""
        self.sr, self.n_mels = sample_rate or self.sr, n_mels or self.n_mels
        self.fb = self.mel_filterbank(self.n_mels, self.n_fft, self.sr)
        return self

    def is_initialized(self) -> bool: return self.fb is not None
    def feature_length(self, num_samples: int) -> int: return 1 + num_samples // self.hop

    def extract(self, waveform):
        """The reference's name for ``compute``; a 1-D waveform is treated as one channel."""
        w = torch.as_tensor(waveform)
        return self.compute(w[None] if w.dim() == 1 else w)

    def compute(self, waveform):
        """waveform [channels, samples] -> [channels, frames, n_mels]."""
        w = waveform.float()
        spec = torch.stft(w, self.n_fft, self.hop, window=torch.hann_window(self.n_fft, device=w.device), return_complex=True)
        power = spec.abs() ** 2
        mel = torch.einsum("mf,cft->ctm", self.fb.to(w.device), power)
        return torch.log(mel.clamp(min=1e-10))


class AudioFeatureExtractor:
    def __init__(self, encoder: AudioTransformer, mel: Optional[MelSpectrogram] = None):
        self.encoder = encoder
        self.mel = mel or MelSpectrogram(16000, encoder.cfg.input_dim)

    @torch.no_grad()
    def extract(self, audio):
        return self.encoder(self.mel.compute(audio), return_tokens=False)

    def init(self, sample_rate: Optional[int] = None):
        self.mel.init(sample_rate, self.encoder.cfg.input_dim)
        return self

    def is_initialized(self) -> bool: return self.mel.is_initialized() and self.encoder.is_initialized()


class AudioSynthesizer:
    """Griffin-Lim phase reconstruction from a log-mel spectrogram (pseudo-inverse of the filter bank)."""

    def __init__(self, mel: Optional[MelSpectrogram] = None, iters=16):
        self.mel, self.iters = mel or MelSpectrogram(), iters

    def synthesize(self, log_mel):
        """[frames, n_mels] -> waveform [samples]."""
        m = self.mel
        mag = torch.sqrt(torch.clamp(torch.linalg.pinv(m.fb) @ log_mel.float().exp().t(), min=0))       # [freq, frames]
        win = torch.hann_window(m.n_fft)
        phase = torch.exp(2j * math.pi * torch.rand(mag.shape, generator=torch.Generator().manual_seed(0)))
        for _ in range(self.iters):
            wav = torch.istft(mag * phase, m.n_fft, m.hop, window=win)
            spec = torch.stft(wav, m.n_fft, m.hop, window=win, return_complex=True)
            phase = spec / spec.abs().clamp(min=1e-8)
            if phase.shape[1] != mag.shape[1]:
                phase = TF.pad(torch.view_as_real(phase), (0, 0, 0, mag.shape[1] - phase.shape[1])) if phase.shape[1] < mag.shape[1] else phase[:, : mag.shape[1]]
                phase = torch.view_as_complex(phase.contiguous()) if not torch.is_complex(phase) else phase
        return torch.istft(mag * phase, m.n_fft, m.hop, window=win)


# ================================================================================================ modality MoEs / fusion
class _ModalityMoE(nn.Module):
    def __init__(self, hidden, num_experts=4, expert_hidden=None, top_k=2):
        super().__init__()
        from ..ops import moe as M
        self.M, self.k = M, top_k
        Fh = expert_hidden or 2 * hidden
        self.router = nn.Parameter(torch.randn(num_experts, hidden) * 0.02)
        self.gate_up = nn.Parameter(torch.randn(num_experts, 2 * Fh, hidden) * 0.02)
        self.down = nn.Parameter(torch.randn(num_experts, hidden, Fh) * 0.02)

    def forward(self, x):
        shp = x.shape
        t = x.reshape(-1, shp[-1])
        logits = (t.float() @ self.router.float().t())
        y, aux, _ = self.M.moe_ffn(t, logits, self.gate_up.to(t.dtype), self.down.to(t.dtype), self.k, True, "silu", 0.01, 0.0)
        self.last_aux = aux
        return x + y.view(shp)


class VisionMoE(_ModalityMoE):
    pass


class AudioMoE(_ModalityMoE):
    pass


class VisionTextMoE(nn.Module):
    """Separate expert pools per modality plus a shared pool applied to the concatenation."""

    def __init__(self, hidden, num_experts=4):
        super().__init__()
        self.vision, self.text, self.shared = _ModalityMoE(hidden, num_experts), _ModalityMoE(hidden, num_experts), _ModalityMoE(hidden, num_experts)

    def forward(self, vision_tokens, text_tokens):
        v, t = self.vision(vision_tokens), self.text(text_tokens)
        both = self.shared(torch.cat([v, t], 1))
        return both[:, : v.shape[1]], both[:, v.shape[1]:]


class AudioTextMoE(VisionTextMoE):
    pass


class AllModalityMoE(nn.Module):
    def __init__(self, hidden, num_experts=4):
        super().__init__()
        self.pools = nn.ModuleDict({m: _ModalityMoE(hidden, num_experts) for m in ("image", "audio", "text")})
        self.shared = _ModalityMoE(hidden, num_experts)

    def forward(self, **tokens):
        outs = {m: self.pools[m](t) for m, t in tokens.items() if t is not None}
        cat = self.shared(torch.cat(list(outs.values()), 1))
        o, res = 0, {}
        for m, t in outs.items():
            res[m] = cat[:, o:o + t.shape[1]]
            o += t.shape[1]
        return res


@dataclass
class FusionConfig:
    hidden: int = 768
    num_heads: int = 12
    mode: str = "cross_attention"        # concat | gated | cross_attention


class CrossAttentionFusion(nn.Module):
    def __init__(self, hidden, heads):
        super().__init__()
        self.block = CrossAttentionBlock(CrossAttentionLayerConfig(hidden, heads, hidden // heads))

    def forward(self, a, b):
        return self.block(a, b)


class MultimodalFusion(nn.Module):
    def __init__(self, cfg: Optional[FusionConfig] = None):
        super().__init__()
        self.cfg = cfg = cfg or FusionConfig()
        self.xattn = CrossAttentionFusion(cfg.hidden, cfg.num_heads)
        self.gate = TFLinear(2 * cfg.hidden, cfg.hidden)
        self.cat = TFLinear(2 * cfg.hidden, cfg.hidden)

    def forward(self, a, b):
        if self.cfg.mode == "cross_attention":
            return self.xattn(a, b)
        pooled = b.mean(1, keepdim=True).expand_as(a)
        both = torch.cat([a, pooled], -1)
        if self.cfg.mode == "gated":
            g = torch.sigmoid(self.gate(both))
            return g * a + (1 - g) * pooled
        return self.cat(both)


def _fusion_api():
    """Named fusions (reference: MultimodalFusion, include/quant/multimodal.h): pairs, all three, weighted."""
    Fz = MultimodalFusion

    def fuse_vision_text(self, vision, text): return self(text, vision)        # text queries the image
    def fuse_audio_text(self, audio, text): return self(text, audio)
    def fuse_vision_audio(self, vision, audio): return self(vision, audio)

    def compute_fusion_weights(self, *streams):
        """Soft-max over the streams of their mean activation energy: the louder stream gets the larger weight."""
        e = torch.stack([s_.float().pow(2).mean() for s_ in streams])
        return torch.softmax(e / e.mean().clamp(min=1e-12), 0)

    def fuse_weighted(self, streams, weights=None):
        """Weighted sum of pooled streams -> [B, hidden]."""
        w = self.compute_fusion_weights(*streams) if weights is None else torch.as_tensor(weights, dtype=torch.float32)
        return sum(wi * s_.mean(1).float() for wi, s_ in zip(w, streams))

    def fuse_all(self, vision, audio, text):
        """Text grounded first in the image, then in the audio: [B, text tokens, hidden]."""
        return self(self(text, vision), audio)

    def fuse_all_multistream(self, vision, audio, text):
        """Every stream grounded in the two others; returns the three grounded streams."""
        va = torch.cat([vision, audio], 1)
        return self(vision, torch.cat([audio, text], 1)), self(audio, torch.cat([vision, text], 1)), self(text, va)

    def param_count(self): return sum(p_.numel() for p_ in self.parameters())

    for name, fn in list(locals().items()):
        if callable(fn) and name != "Fz":
            setattr(Fz, name, fn)


_fusion_api()


class CrossModalAlignment(ContrastiveAlignmentHead):
    def contrastive_loss(self, a, b):
        return self.forward(a, b)

    def align(self, a, b):
        return self.similarity(a, b)


class ModalityEncoder(nn.Module):
    """Uniform wrapper: ``encode(x)`` returns pooled features of whatever tower it holds."""

    def __init__(self, tower):
        super().__init__()
        self.tower = tower

    def encode(self, x):
        out = self.tower(x)
        return out if out.dim() == 2 else out.mean(1)


class MultiModalTokenizer:
    """One id space for text tokens and discrete image / audio codes: text ids first, then ``image_codes`` image ids,
    then ``audio_codes`` audio ids, each modality bracketed by begin / end markers."""

    def __init__(self, text_tokenizer=None, image_codes=8192, audio_codes=1024):
        from ..tokenizer import ByteTokenizer
        self.text = text_tokenizer or ByteTokenizer()
        self.tv = self.text.vocab_size
        self.image_base, self.audio_base = self.tv + 4, self.tv + 4 + image_codes
        self.BOI, self.EOI, self.BOA, self.EOA = self.tv, self.tv + 1, self.tv + 2, self.tv + 3
        self.vocab_size = self.audio_base + audio_codes

    def encode(self, text="", image_codes: Sequence[int] = (), audio_codes: Sequence[int] = ()):
        ids = list(self.text.encode(text)) if text else []
        if len(image_codes):
            ids += [self.BOI] + [self.image_base + int(c) for c in image_codes] + [self.EOI]
        if len(audio_codes):
            ids += [self.BOA] + [self.audio_base + int(c) for c in audio_codes] + [self.EOA]
        return ids

    def image_token_id(self, code: int = 0) -> int: return self.image_base + int(code)
    def audio_token_id(self, code: int = 0) -> int: return self.audio_base + int(code)

    def encode_image(self, image, grid: int = 8, levels: Optional[int] = None) -> List[int]:
        """Discrete codes of an image without a learned codebook: the mean brightness of each cell of a ``grid`` x ``grid``
        partition, quantised to the image-code range, bracketed by the image markers."""
        img = image.data if isinstance(image, Image) else torch.as_tensor(image).float()
        img = img.mean(0, keepdim=True) if img.dim() == 3 else img[None]
        cells = TF.adaptive_avg_pool2d(img[None], grid)[0, 0].reshape(-1)
        n = levels or (self.audio_base - self.image_base)
        lo, hi = float(cells.min()), float(cells.max())
        codes = ((cells - lo) / max(hi - lo, 1e-12) * (n - 1)).round().long().tolist()
        return self.encode("", image_codes=codes)

    def encode_audio(self, mel_or_wave, frames: int = 16) -> List[int]:
        """Discrete codes of a log-mel spectrogram [frames, mels] (or a waveform): the mean energy of ``frames`` equal
        time slices, quantised to the audio-code range."""
        x = torch.as_tensor(mel_or_wave).float()
        x = x.abs()[:, None] if x.dim() == 1 else x
        sl = TF.adaptive_avg_pool1d(x.mean(1)[None, None], frames)[0, 0]
        n = self.vocab_size - self.audio_base
        lo, hi = float(sl.min()), float(sl.max())
        codes = ((sl - lo) / max(hi - lo, 1e-12) * (n - 1)).round().long().tolist()
        return self.encode("", audio_codes=codes)

    def decode(self, ids):
        text = self.text.decode([i for i in ids if i < self.tv])
        img = [i - self.image_base for i in ids if self.image_base <= i < self.audio_base]
        aud = [i - self.audio_base for i in ids if i >= self.audio_base]
        return {"text": text, "image_codes": img, "audio_codes": aud}


# ================================================================================================ task heads
class ImageNetClassifier(nn.Module):
    def __init__(self, vit: VisionTransformer, num_classes=1000):
        super().__init__()
        self.vit, self.head = vit, TFLinear(vit.cfg.hidden_dim, num_classes)

    def forward(self, img):
        return self.head(self.vit(img))

    @torch.no_grad()
    def classify(self, img, top_k=5):
        p = torch.softmax(self.forward(img).float(), -1)
        v, i = p.topk(top_k, -1)
        return [[(int(a), float(b)) for a, b in zip(ii, vv)] for ii, vv in zip(i, v)]

    @torch.no_grad()
    def evaluate(self, images, labels, top_k: int = 5) -> dict:
        """{top1, top5 (top-``top_k``) accuracy} on a labelled batch."""
        lg = self.forward(images).float()
        lab = torch.as_tensor(labels, device=lg.device)
        top = lg.topk(min(top_k, lg.shape[-1]), -1).indices
        return {"top1": float((top[:, 0] == lab).float().mean()), f"top{top_k}": float((top == lab[:, None]).any(-1).float().mean())}


ImageClassifier = ImageNetClassifier


def ctc_greedy_decode(log_probs, blank=0):
    """[T, V] -> token ids with repeats merged and blanks removed."""
    out, prev = [], None
    for t in log_probs.argmax(-1).tolist():
        if t != prev and t != blank:
            out.append(t)
        prev = t
    return out


class SpeechRecognizer(nn.Module):
    def __init__(self, encoder: AudioTransformer, vocab_size, blank=0):
        super().__init__()
        self.enc, self.head, self.blank = encoder, TFLinear(encoder.cfg.hidden_dim, vocab_size), blank

    def forward(self, mel):
        return torch.log_softmax(self.head(self.enc(mel)).float(), -1)

    def loss(self, mel, targets, target_lengths):
        lp = self.forward(mel).transpose(0, 1)
        il = torch.full((mel.shape[0],), lp.shape[0], dtype=torch.long)
        return TF.ctc_loss(lp, targets, il, target_lengths, blank=self.blank, zero_infinity=True)

    @torch.no_grad()
    def transcribe(self, mel):
        return [ctc_greedy_decode(lp, self.blank) for lp in self.forward(mel)]


@dataclass
class OCRBox:
    x: int
    y: int
    w: int
    h: int
    text: str = ""
    confidence: float = 0.0


class OCREngine(_TowerAPI, nn.Module):
    """Line recogniser: the image is cut into column strips (patch columns), encoded, and decoded with CTC."""

    def __init__(self, vit: VisionTransformer, vocab_size, blank=0):
        super().__init__()
        self.vit, self.head, self.blank = vit, TFLinear(vit.cfg.hidden_dim, vocab_size), blank

    def forward(self, img):
        tok = self.vit(img, return_tokens=True)[:, 1:]
        g = img.shape[-1] // self.vit.cfg.patch_size
        cols = tok.view(tok.shape[0], -1, g, tok.shape[-1]).mean(1)          # average over patch rows -> one feature per column
        return torch.log_softmax(self.head(cols).float(), -1)

    @torch.no_grad()
    def recognize(self, img, decode=lambda ids: "".join(chr(i) for i in ids)):
        out = []
        for b, lp in enumerate(self.forward(img)):
            ids = ctc_greedy_decode(lp, self.blank)
            out.append(OCRBox(0, 0, img.shape[-1], img.shape[-2], decode(ids), float(lp.max(-1).values.exp().mean())))
        return out


OCRPipeline = OCREngine


class VideoEncoder(_TowerAPI, nn.Module):
    """Frames through the image tower, then a temporal transformer over the per-frame features."""

    def __init__(self, vit: VisionTransformer, temporal_layers=2):
        super().__init__()
        d = vit.cfg.hidden_dim
        self.vit, self.dim = vit, d
        self.temporal = nn.ModuleList(EncoderBlock(d, vit.cfg.num_heads, 4 * d) for _ in range(temporal_layers))

    def forward(self, video):
        B, T = video.shape[:2]
        f = self.vit(video.flatten(0, 1)).view(B, T, -1)
        for b in self.temporal:
            f = b(f)
        return f


class VideoUnderstanding(nn.Module):
    def __init__(self, encoder: VideoEncoder, num_classes):
        super().__init__()
        self.enc, self.head = encoder, TFLinear(encoder.vit.cfg.hidden_dim, num_classes)

    def forward(self, video):
        return self.head(self.enc(video).mean(1))

    @torch.no_grad()
    def describe(self, video, class_names: Optional[Sequence[str]] = None, top_k: int = 3) -> str:
        """One line per clip naming the most likely classes with their probabilities."""
        p = torch.softmax(self.forward(video).float(), -1)
        v, i = p.topk(min(top_k, p.shape[-1]), -1)
        name = lambda c: class_names[c] if class_names else f"class {c}"
        return "\n".join(", ".join(f"{name(int(c))} ({float(q):.2f})" for c, q in zip(ii, vv)) for ii, vv in zip(i, v))


class ImageCaptioning(nn.Module):
    """Image tokens as a prefix (projected to the language model's width) of a causal text decoder."""

    def __init__(self, vit: VisionTransformer, vocab_size, dim=None, layers=2, heads=4, max_len=128):
        super().__init__()
        dim = dim or vit.cfg.hidden_dim
        self.vit, self.proj = vit, TFLinear(vit.cfg.hidden_dim, dim)
        self.dec = TextEncoder(vocab_size, dim, layers, heads, max_len, causal=True)
        self.head = TFLinear(dim, vocab_size, False)
        self.max_len = max_len

    def forward(self, img, ids):
        prefix = self.proj(self.vit(img, return_tokens=True))
        x = torch.cat([prefix, self.dec.emb(ids) + self.dec.pos[:, : ids.shape[1]]], 1)
        for b in self.dec.blocks:
            x = b(x, causal=True)
        return self.head(self.dec.norm(x))[:, prefix.shape[1]:]

    @torch.no_grad()
    def caption(self, img, bos=1, eos=2, max_tokens=16):
        ids = torch.full((img.shape[0], 1), bos, dtype=torch.long, device=img.device)
        for _ in range(max_tokens):
            nxt = self.forward(img, ids)[:, -1].argmax(-1, keepdim=True)
            ids = torch.cat([ids, nxt], 1)
            if bool((nxt == eos).all()):
                break
        return ids


class VisualQA(nn.Module):
    def __init__(self, vit: VisionTransformer, text: TextEncoder, num_answers, hidden=None):
        super().__init__()
        hidden = hidden or vit.cfg.hidden_dim
        self.vit, self.text = vit, text
        self.pv, self.pt = TFLinear(vit.cfg.hidden_dim, hidden), TFLinear(text.emb.embedding_dim, hidden)
        self.fuse = CrossAttentionFusion(hidden, 4)
        self.head = TFLinear(hidden, num_answers)

    def forward(self, img, question_ids):
        v = self.pv(self.vit(img, return_tokens=True))
        q = self.pt(self.text(question_ids))
        return self.head(self.fuse(q, v).mean(1))

    @torch.no_grad()
    def answer(self, img, question_ids, answers: Optional[Sequence[str]] = None):
        """The most likely answer per example: its index, or its text when ``answers`` names the classes."""
        best = self.forward(img, question_ids).argmax(-1).tolist()
        return [answers[b] for b in best] if answers else best


class TextToImage(nn.Module):
    """Autoregressive image-code decoder conditioned on text: predicts a grid of discrete codes that a codebook decoder
    turns into pixels (``codes_to_image`` with a learned patch codebook)."""

    def __init__(self, text: TextEncoder, num_codes=512, grid=8, dim=None, layers=2, heads=4, patch=8, channels=3):
        super().__init__()
        dim = dim or text.emb.embedding_dim
        self.text, self.grid, self.patch, self.channels = text, grid, patch, channels
        self.code_emb = nn.Embedding(num_codes + 1, dim)
        self.pos = nn.Parameter(torch.randn(1, grid * grid + 1, dim) * 0.02)
        self.blocks = nn.ModuleList(EncoderBlock(dim, heads, 4 * dim) for _ in range(layers))
        self.xattn = CrossAttentionBlock(CrossAttentionLayerConfig(dim, heads, dim // heads))
        self.head = TFLinear(dim, num_codes, False)
        self.codebook = nn.Parameter(torch.randn(num_codes, channels * patch * patch) * 0.1)
        self.start = num_codes

    def logits(self, text_ids, codes):
        ctx = self.text(text_ids)
        x = self.code_emb(codes) + self.pos[:, : codes.shape[1]]
        for b in self.blocks:
            x = b(x, causal=True)
        return self.head(self.xattn(x, ctx))

    @torch.no_grad()
    def generate(self, text_ids):
        B = text_ids.shape[0]
        codes = torch.full((B, 1), self.start, dtype=torch.long, device=text_ids.device)
        for _ in range(self.grid * self.grid):
            codes = torch.cat([codes, self.logits(text_ids, codes)[:, -1].argmax(-1, keepdim=True)], 1)
        return self.codes_to_image(codes[:, 1:])

    def codes_to_image(self, codes):
        B, g, p, C = codes.shape[0], self.grid, self.patch, self.channels
        px = self.codebook[codes].view(B, g, g, C, p, p).permute(0, 3, 1, 4, 2, 5)
        return px.reshape(B, C, g * p, g * p)


class JointMultimodalModel(MultimodalCrossAttention):
    pass


# ================================================================================================ containers
class Image:
    """CHW float image with the usual helpers."""

    def __init__(self, data: torch.Tensor):
        self.data = data.float()

    @classmethod
    def zeros(cls, c, h, w):
        return cls(torch.zeros(c, h, w))

    def resize(self, h, w):
        return Image(TF.interpolate(self.data[None], size=(h, w), mode="bilinear", align_corners=False)[0])

    def normalize(self, mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225)):
        m, s = torch.tensor(mean)[:, None, None], torch.tensor(std)[:, None, None]
        return Image((self.data - m[: self.data.shape[0]]) / s[: self.data.shape[0]])

    def center_crop(self, size):
        _, h, w = self.data.shape
        t, l = (h - size) // 2, (w - size) // 2
        return Image(self.data[:, t:t + size, l:l + size])

    def to_grayscale(self):
        w = torch.tensor([0.299, 0.587, 0.114])[:, None, None]
        return Image((self.data[:3] * w).sum(0, keepdim=True))

    # ---- accessors and file verbs of the reference (include/quant/image.h)
    def channels(self) -> int: return self.data.shape[0]
    def height(self) -> int: return self.data.shape[1]
    def width(self) -> int: return self.data.shape[2]
    def numel(self) -> int: return self.data.numel()
    def to_tensor(self) -> torch.Tensor: return self.data

    def save(self, path): return self.save_ppm(path)

    @classmethod
    def load(cls, path): return cls.load_ppm(path)

    def save_ppm(self, path):
        d = (self.data.clamp(0, 1) * 255).to(torch.uint8)
        if d.shape[0] == 1:
            d = d.expand(3, -1, -1)
        with open(path, "wb") as f:
            f.write(f"P6\n{d.shape[2]} {d.shape[1]}\n255\n".encode() + d.permute(1, 2, 0).contiguous().numpy().tobytes())

    @classmethod
    def load_ppm(cls, path):
        raw = open(path, "rb").read()
        parts = raw.split(b"\n", 3)
        w, h = map(int, parts[1].split())
        px = torch.frombuffer(bytearray(parts[3][: w * h * 3]), dtype=torch.uint8).view(h, w, 3)
        return cls(px.permute(2, 0, 1).float() / 255.0)


class Video:
    def __init__(self, frames: torch.Tensor, fps: float = 30.0):
        self.frames, self.fps = frames.float(), fps            # [T, C, H, W]

    def sample_uniform(self, n):
        idx = torch.linspace(0, self.frames.shape[0] - 1, n).round().long()
        return Video(self.frames[idx], self.fps * n / max(1, self.frames.shape[0]))

    def duration(self):
        return self.frames.shape[0] / self.fps

    # ---- accessors and file verbs of the reference (include/quant/video.h)
    def num_frames(self) -> int: return self.frames.shape[0]
    def height(self) -> int: return self.frames.shape[2]
    def width(self) -> int: return self.frames.shape[3]
    def frame(self, i: int) -> Image: return Image(self.frames[i])

    @classmethod
    def load(cls, directory: str, fps: float = 30.0) -> "Video":
        """Frames from a directory of PPM files (sorted by name)."""
        import os
        names = sorted(n for n in os.listdir(directory) if n.lower().endswith(".ppm"))
        return cls(torch.stack([Image.load_ppm(os.path.join(directory, n)).data for n in names]), fps)

    def save(self, directory: str):
        import os
        os.makedirs(directory, exist_ok=True)
        for i in range(self.num_frames()):
            self.frame(i).save_ppm(os.path.join(directory, f"frame_{i:06d}.ppm"))


VisionEncoder = VisionTransformer
AudioEncoder = AudioTransformer


class TextDecoder(TextEncoder):
    def __init__(self, vocab, dim, layers, heads, max_len=2048):
        super().__init__(vocab, dim, layers, heads, max_len, causal=True)
        self.head = TFLinear(dim, vocab, False)

    def forward(self, ids):
        return self.head(super().forward(ids))

    @torch.no_grad()
    def decode(self, ids, max_tokens: int = 16, eos: int = -1):
        """Greedy continuation of a prompt [1, S] -> the new ids."""
        ids = list(ids[0].tolist() if torch.is_tensor(ids) else ids)
        out = []
        for _ in range(max_tokens):
            nxt = int(self(torch.tensor([ids + out]))[0, -1].argmax())
            out.append(nxt)
            if nxt == eos:
                break
        return out


class SentenceEmbedder:
    def __init__(self, text: TextEncoder, tokenizer, normalize=True):
        self.text, self.tok, self.normalize = text, tokenizer, normalize

    @torch.no_grad()
    def embed(self, sentences: Sequence[str]):
        out = []
        for s in sentences:
            ids = torch.tensor([self.tok.encode(s)[: self.text.pos.shape[1]] or [0]])
            e = self.text(ids, return_tokens=False)[0].float()
            out.append(TF.normalize(e, dim=0) if self.normalize else e)
        return torch.stack(out)

    def similarity(self, a: str, b: str) -> float:
        e = self.embed([a, b])
        return float(e[0] @ e[1])

    forward = embed

    def hidden_size(self) -> int: return self.text.hidden_size()
    def output_size(self) -> int: return self.text.hidden_size()
