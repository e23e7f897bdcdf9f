"""Parameter-efficient and selective fine-tuning on top of the fused training step.

* ``RankAdapterEngine``   - LoRA / DoRA adapters.  The adapted matrix is materialised as
  W_eff = W0 + B A (DoRA: m * (W0 + B A) / ||W0 + B A||_row) before the fused forward+backward, whose
  weight-gradient GEMM already produces G = dL/dW_eff in fp32; the adapter gradients follow from the chain
  rule through the tiny graph (A, B, m) -> W_eff.  No extra activations are kept and any projection can carry
  an adapter (default: FFN down projection, as the reference).  ``save`` / ``load`` use the ``.nrad`` store
  (quantised factors, fp32 magnitudes); ``merge_into_base`` bakes the adapters in.
* ``SelectiveFineTuner``  - Fisher-diagonal accumulation, saliency block selection (RMS gradient x
  (1 + bias * log1p(mean Fisher)) above mean + sigma * std, with a floor), masked updates and an optional
  straight-through round trip of the selected blocks through a wire format.
* ``KnowledgeExpansionEngine`` - gated side slots h + w_out * tanh(gate) * act(w_in h) on the final hidden state,
  consulted only when the base model's confidence is low.
* ``FineTuner``           - plain full fine-tuning with a straight-through quantised update.

Reference counterparts: include/quant/fine_tuning.h:43-242, src/trainer/fine_tuning.cpp (select_blocks :299-349,
.nrad :816-890), src/trainer/finetune.cpp."""
from __future__ import annotations

import os

import math
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..quant import codec
from ..quant.qat import ste_roundtrip_


# ================================================================================================ LoRA / DoRA
@dataclass
class RankAdapterConfig:
    rank: int = 16
    alpha: float = 1.0
    learning_rate: float = 3e-4
    weight_decay: float = 0.0
    warmup_steps: int = 10
    factor_format: str = "q8"
    output_path: str = "adapters.nrad"
    use_dora: bool = False
    targets: Sequence[str] = ("down",)      # any of: qkv, o, gate_up, down


class LayerAdapter:
    def __init__(self, layer_index, name, param, rank, alpha, dora):
        self.layer_index, self.name, self.param = layer_index, name, param
        out_dim, in_dim = param.shape
        self.in_dim, self.out_dim, self.rank = in_dim, out_dim, rank
        dev = param.device
        self.W0 = param.data.float().clone()
        g = torch.Generator(device="cpu").manual_seed(1234 + layer_index)
        self.A = (torch.randn(rank, in_dim, generator=g) * (alpha / rank) / math.sqrt(in_dim)).to(dev).requires_grad_()
        self.B = torch.zeros(out_dim, rank, device=dev, requires_grad=True)
        self.magnitude = self.W0.norm(dim=1).clone().requires_grad_() if dora else None

    def params(self):
        return [self.A, self.B] + ([self.magnitude] if self.magnitude is not None else [])

    def effective(self):
        W = self.W0 + self.B @ self.A
        if self.magnitude is not None:
            W = W * (self.magnitude / W.norm(dim=1).clamp(min=1e-12))[:, None]
        return W


class RankAdapterEngine:
    def __init__(self, model, cfg: Optional[RankAdapterConfig] = None, **kw):
        self.model = model
        self.cfg = cfg or RankAdapterConfig(**{({"lr": "learning_rate"}.get(k, k)): v for k, v in kw.items()})
        self.adapters: List[LayerAdapter] = []
        self.step_count = 0
        self.last_loss = 0.0
        model.flatten()
        self.init_adapters()

    def configure(self, cfg: RankAdapterConfig):
        self.cfg = cfg
        self.init_adapters()

    def init_adapters(self):
        c = self.cfg
        self.adapters = []
        for i, l in enumerate(self.model.layers):
            for tname in c.targets:
                p = {"qkv": l.qkv, "o": l.o, "gate_up": l.gate_up, "down": l.down}[tname]
                nm = {"down": "ffn.down_proj", "o": "attention.o_proj", "qkv": "attention.qkv_proj", "gate_up": "ffn.gate_up_proj"}[tname]
                self.adapters.append(LayerAdapter(i, f"layers.{i}.{nm}", p, c.rank, c.alpha, c.use_dora))
        ps = [p for a in self.adapters for p in a.params()]
        self.opt = torch.optim.AdamW(ps, lr=c.learning_rate, weight_decay=c.weight_decay, betas=(0.9, 0.999))

    def freeze_base(self, freeze=True):
        self.base_frozen = freeze        # the base is never stepped by this engine; kept for API parity

    def dora_enabled(self):
        return self.cfg.use_dora

    def adapter_param_count(self):
        return sum(p.numel() for a in self.adapters for p in a.params())

    def dora_param_count(self):
        return sum(a.magnitude.numel() for a in self.adapters if a.magnitude is not None)

    def _materialise(self):
        eff = []
        for a in self.adapters:
            W = a.effective()
            with torch.no_grad():
                a.param.data.copy_(W.to(a.param.dtype))
            eff.append(W)
        return eff

    @torch.no_grad()
    def forward_with_adapters(self, ids):
        self._materialise()
        return self.model.forward(ids)

    def train_step(self, ids, labels) -> float:
        c = self.cfg
        eff = self._materialise()
        self.model.flat.zero_grad()
        loss = self.model.forward_backward(ids, labels)
        lr = c.learning_rate * min(1.0, (self.step_count + 1) / max(1, c.warmup_steps))
        for g in self.opt.param_groups:
            g["lr"] = lr
        self.opt.zero_grad(set_to_none=True)
        torch.autograd.backward(eff, [a.param.main_grad for a in self.adapters])
        self.opt.step()
        self.step_count += 1
        self.last_loss = float(loss)
        return self.last_loss

    def clear_grads(self):
        self.opt.zero_grad(set_to_none=True)
        self.model.flat.zero_grad()

    def step(self) -> int:
        """Training steps taken so far."""
        return self.step_count

    @torch.no_grad()
    def magnitude_step(self, dL_dW, lr: float) -> int:
        """Plain gradient step on the DoRA magnitudes alone, from given gradients of the MERGED weights (one tensor per
        adapter, shaped like the adapted matrix [out, in]; None or a wrong shape skips that adapter).  With the direction
        V = W0 + B A held fixed, W' = m * V / |V| row by row, so dL/dm[o] = sum_k dL/dW'[o, k] V[o, k] / |V[o, :]|.
        Returns how many adapters were stepped.  Reference counterpart: RankAdapterEngine::magnitude_step
        (include/quant/fine_tuning.h:189-197)."""
        n = 0
        for a, g in zip(self.adapters, dL_dW):
            if a.magnitude is None or g is None or tuple(g.shape) != (a.out_dim, a.in_dim):
                continue
            V = a.W0 + a.B @ a.A
            a.magnitude.sub_(lr * (g.float().to(V.device) * V).sum(1) / V.norm(dim=1).clamp(min=1e-12))
            n += 1
        return n

    @torch.no_grad()
    def merge_into_base(self):
        self._materialise()
        for a in self.adapters:
            a.W0 = a.param.data.float().clone()
            a.B.zero_()
            if a.magnitude is not None:
                a.magnitude.copy_(a.W0.norm(dim=1))

    # ---- .nrad: "NRAD" | u32 version (1 LoRA, 2 +DoRA magnitudes) | u32 count | per adapter {i64 layer, u64 rank,
    #      u64 out, u64 in, qtensor A, qtensor B, [fp32 magnitude x out]};  qtensor = u8 fmt | u64 numel | u32 nblocks |
    #      per 256-weight block {u32 bytes, payload}
    @staticmethod
    def _write_q(f, t, fmt):
        a = t.detach().float().cpu().contiguous().numpy().reshape(-1)
        f.write(struct.pack("<BQI", fmt, a.size, (a.size + 255) // 256))
        for o in range(0, a.size, 256):
            pay = codec.quantize_block(fmt, a[o:o + 256])
            f.write(struct.pack("<I", len(pay)))
            f.write(pay)

    @staticmethod
    def _read_q(f):
        fmt, n, nb = struct.unpack("<BQI", f.read(13))
        if n > (1 << 32) or nb != (n + 255) // 256:
            raise ValueError("corrupt .nrad tensor header")
        out = np.empty(n, dtype=np.float32)
        for b in range(nb):
            (ln,) = struct.unpack("<I", f.read(4))
            cnt = min(256, n - b * 256)
            out[b * 256: b * 256 + cnt] = codec.dequantize_block(fmt, f.read(ln), cnt)
        return torch.from_numpy(out)

    def save(self, path=None):
        path = path or self.cfg.output_path
        fmt = codec.parse_format(self.cfg.factor_format)
        fmt = fmt if fmt >= 0 else codec.parse_format("q8")
        with open(path, "wb") as f:
            f.write(b"NRAD" + struct.pack("<II", 2 if self.cfg.use_dora else 1, len(self.adapters)))
            for a in self.adapters:
                f.write(struct.pack("<qQQQ", a.layer_index, a.rank, a.out_dim, a.in_dim))
                self._write_q(f, a.A, fmt)
                self._write_q(f, a.B, fmt)
                if self.cfg.use_dora:
                    f.write(a.magnitude.detach().float().cpu().numpy().tobytes())
        return path

    save_adapters = save

    def load(self, path) -> bool:
        try:
            with open(path, "rb") as f:
                if f.read(4) != b"NRAD":
                    return False
                version, count = struct.unpack("<II", f.read(8))
                if version not in (1, 2) or count != len(self.adapters):
                    return False
                for a in self.adapters:
                    li, rk, od, idim = struct.unpack("<qQQQ", f.read(32))
                    if (rk, od, idim) != (a.rank, a.out_dim, a.in_dim):
                        return False
                    A, B = self._read_q(f), self._read_q(f)
                    with torch.no_grad():
                        a.A.copy_(A.view(a.rank, a.in_dim))
                        a.B.copy_(B.view(a.out_dim, a.rank))
                        if version >= 2:
                            m = torch.from_numpy(np.frombuffer(f.read(4 * od), dtype=np.float32).copy())
                            if a.magnitude is not None:
                                a.magnitude.copy_(m)
            return True
        except (OSError, struct.error, ValueError):
            return False


# ================================================================================================ selective tuning
@dataclass
class SelectiveTunerConfig:
    block_size: int = 256
    saliency_sigma: float = 1.0
    fisher_bias: float = 0.5
    learning_rate: float = 1e-4
    warmup_steps: int = 10
    min_select_fraction: float = 0.01
    target_format: str = "q16"
    ste_roundtrip: bool = True
    output_path: str = "finetuned_selective.quant"


@dataclass
class SelectiveStats:
    selected_fraction: float = 0.0
    selected_blocks: int = 0
    total_blocks: int = 0
    last_loss: float = 0.0
    steps: int = 0


class SelectiveFineTuner:
    def __init__(self, model, cfg: Optional[SelectiveTunerConfig] = None):
        self.model, self.cfg = model, cfg or SelectiveTunerConfig()
        self.flat = model.flatten()
        self.fisher = torch.zeros_like(self.flat.grads)
        self.fisher_batches = 0
        self.stats = SelectiveStats()
        self.m = torch.zeros_like(self.flat.grads)
        self.v = torch.zeros_like(self.flat.grads)
        self.master = self.flat.params.float().clone()

    def configure(self, cfg):
        self.cfg = cfg

    @staticmethod
    def select_blocks(grad: torch.Tensor, fisher: torch.Tensor, block_size=256, sigma=1.0, fisher_bias=0.5, min_frac=0.01):
        """(bool mask per block, threshold)."""
        n = grad.numel()
        nb = (n + block_size - 1) // block_size
        pad = nb * block_size - n
        g = torch.nn.functional.pad(grad.float().reshape(-1), (0, pad)).view(nb, block_size)
        f = torch.nn.functional.pad(fisher.float().reshape(-1).clamp(min=0), (0, pad)).view(nb, block_size)
        cnt = torch.full((nb,), float(block_size), device=g.device)
        cnt[-1] = block_size - pad
        sal = torch.sqrt((g * g).sum(1) / cnt) * (1.0 + fisher_bias * torch.log1p(f.sum(1) / cnt))
        thr = float(sal.mean() + sigma * sal.var(unbiased=False).sqrt())
        mask = sal > thr
        floor = min(nb, int(min_frac * nb))
        if int(mask.sum()) < floor:
            mask = torch.zeros(nb, dtype=torch.bool, device=g.device)
            mask[sal.topk(floor).indices] = True
        return mask, thr

    def accumulate_fisher(self, ids, labels):
        self.flat.zero_grad()
        self.model.forward_backward(ids, labels)
        self.fisher.add_(self.flat.grads ** 2)
        self.fisher_batches += 1
        self.flat.zero_grad()

    def accumulate_fisher_loader(self, dl, max_batches):
        for _ in range(max_batches):
            self.accumulate_fisher(*dl.next_batch())

    def fine_tune(self, ids, labels, steps=1):
        c = self.cfg
        bs = c.block_size
        for _ in range(steps):
            self.flat.zero_grad()
            loss = self.model.forward_backward(ids, labels)
            g = self.flat.grads
            fisher = self.fisher / max(1, self.fisher_batches)
            mask, _ = self.select_blocks(g, fisher, bs, c.saliency_sigma, c.fisher_bias, c.min_select_fraction)
            wmask = mask.repeat_interleave(bs)[: g.numel()]
            st = self.stats
            st.steps += 1
            lr = c.learning_rate * min(1.0, st.steps / max(1, c.warmup_steps))
            g = g * wmask
            self.m.mul_(0.9).add_(g, alpha=0.1)
            self.v.mul_(0.999).addcmul_(g, g, value=0.001)
            upd = (self.m / (1 - 0.9 ** st.steps)) / ((self.v / (1 - 0.999 ** st.steps)).sqrt() + 1e-8)
            self.master.add_(upd * wmask, alpha=-lr)
            if c.ste_roundtrip:
                # forward weights = wire-format round trip of the selected blocks; the master copy stays exact
                w = self.master.clone()
                sel = mask.nonzero().reshape(-1).tolist()
                if sel:
                    host = w.cpu()
                    fmt = codec.parse_format(c.target_format)
                    a = host.numpy()
                    for b in sel:
                        seg = a[b * bs:(b + 1) * bs]
                        a[b * bs:(b + 1) * bs] = codec.dequantize_block(fmt, codec.quantize_block(fmt, seg), seg.size)
                    w = host.to(self.master.device)
                self.flat.params.copy_(w.to(self.flat.params.dtype))
            else:
                self.flat.params.copy_(self.master.to(self.flat.params.dtype))
            st.selected_blocks, st.total_blocks = int(mask.sum()), mask.numel()
            st.selected_fraction = st.selected_blocks / max(1, st.total_blocks)
            st.last_loss = float(loss)
        self.flat.zero_grad()
        return self.stats.last_loss

    def fine_tune_loader(self, dl, max_batches):
        for _ in range(max_batches):
            self.fine_tune(*dl.next_batch())

    def fisher_diag(self) -> List[torch.Tensor]:
        """The accumulated Fisher diagonal (mean squared gradient over the anchor batches), one tensor per model parameter
        in the flat buffer's order and shape."""
        f = self.fisher / max(1, self.fisher_batches)
        return [f[off:off + p.numel()].view(p.shape) for p, off in zip(self.flat.params_list, self.flat.offsets)]

    def freeze_all(self, freeze):
        self.frozen = freeze

    def save(self, path=None):
        codec.save_model(self.model, path or self.cfg.output_path, self.cfg.target_format)


# ================================================================================================ knowledge slots
@dataclass
class KnowledgeExpansionConfig:
    slot_width: int = 256
    learning_rate: float = 3e-4
    warmup_steps: int = 10
    confidence_threshold: float = 0.35
    slot_gate_threshold: float = 0.5
    output_path: str = "knowledge_slots.kexp"


class KnowledgeSlot:
    def __init__(self, name, hidden, width, device):
        self.name, self.hidden_size, self.width = name, hidden, width
        self.w_in = (torch.randn(width, hidden, device=device) / math.sqrt(hidden)).requires_grad_()
        self.w_out = torch.zeros(hidden, width, device=device, requires_grad=True)
        self.gate = torch.ones(1, device=device)
        self.usage, self.avg_confidence = 0.0, 0.0

    def __call__(self, h):
        return (torch.nn.functional.silu(h @ self.w_in.t()) @ self.w_out.t()) * torch.tanh(self.gate)


class KnowledgeExpansionEngine:
    def __init__(self, model, cfg: Optional[KnowledgeExpansionConfig] = None):
        self.model, self.cfg = model, cfg or KnowledgeExpansionConfig()
        self.slots: List[KnowledgeSlot] = []
        self.opt = None
        self.step_count, self.last_loss = 0, 0.0

    def configure(self, cfg):
        self.cfg = cfg

    def freeze_base(self, freeze=True):
        self.base_frozen = freeze

    def add_slot(self, name, width=0) -> int:
        dev = self.model.tok_embeddings.device
        self.slots.append(KnowledgeSlot(name, self.model.cfg.hidden_size, width or self.cfg.slot_width, dev))
        self.opt = torch.optim.AdamW([p for s in self.slots for p in (s.w_in, s.w_out)], lr=self.cfg.learning_rate, weight_decay=0.0)
        return len(self.slots) - 1

    def slot_count(self):
        return len(self.slots)

    def slot_param_count(self):
        return sum(s.w_in.numel() + s.w_out.numel() for s in self.slots)

    def _hidden(self, ids):
        with torch.no_grad():
            return self.model.hidden_states(ids).float()

    def _logits(self, h):
        return h @ self.model.lm_head.data.float().t()

    def forward_with_slots(self, ids):
        h = self._hidden(ids)
        for s in self.slots:
            h = h + s(h)
        return self._logits(h).view(*ids.shape, -1)

    @torch.no_grad()
    def forward_guarded(self, ids):
        """(logits, confidence [T], slot_used [T]): slots are consulted only where the base top-1 probability is low."""
        h = self._hidden(ids)
        base = self._logits(h)
        conf = torch.softmax(base, -1).amax(-1)
        use = conf < self.cfg.confidence_threshold
        hs = h
        for s in self.slots:
            hs = hs + s(hs)
            s.usage = 0.9 * s.usage + 0.1 * float(use.float().mean())
            s.avg_confidence = 0.9 * s.avg_confidence + 0.1 * float(conf.mean())
        out = torch.where(use[:, None], self._logits(hs), base)
        return out.view(*ids.shape, -1), conf.view(ids.shape), use.view(ids.shape)

    def train_step(self, ids, labels):
        logits = self.forward_with_slots(ids)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1), ignore_index=-100)
        lr = self.cfg.learning_rate * min(1.0, (self.step_count + 1) / max(1, self.cfg.warmup_steps))
        for g in self.opt.param_groups:
            g["lr"] = lr
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        self.opt.step()
        self.step_count += 1
        self.last_loss = float(loss)
        return self.last_loss

    def clear_grads(self):
        if self.opt:
            self.opt.zero_grad(set_to_none=True)

    def step(self) -> int:
        return self.step_count

    def save(self, path=None):
        w = codec.QuantWriter(path or self.cfg.output_path, struct.pack("<II", len(self.slots), self.model.cfg.hidden_size), flags=2)
        for i, s in enumerate(self.slots):
            w.add_tensor(f"slots.{i}.{s.name}.w_in", s.w_in, codec.Q_32)
            w.add_tensor(f"slots.{i}.{s.name}.w_out", s.w_out, codec.Q_32)
        w.close(write_idx=False)

    def load(self, path) -> bool:
        try:
            r = codec.QuantReader(path)
        except ValueError:
            return False
        by = {}
        for n in r.tensor_names():
            _, i, rest = n.split(".", 2)
            name, kind = rest.rsplit(".", 1)
            by.setdefault((int(i), name), {})[kind] = r.read_tensor(n)
        self.slots = []
        H = self.model.cfg.hidden_size
        for (i, name), d in sorted(by.items()):
            self.add_slot(name, d["w_in"].numel() // H)
            with torch.no_grad():
                self.slots[-1].w_in.copy_(d["w_in"].view(-1, H))
                self.slots[-1].w_out.copy_(d["w_out"].view(H, -1))
        return True


# ================================================================================================ plain fine-tuning
class FineTuner:
    """Full fine-tuning whose forward weights are the wire-format round trip of the fp32 master weights after
    every ``requant_interval`` steps (straight-through update)."""

    def __init__(self, model, lr=1e-5, fmt="q16", requant_interval=1):
        from .fused_optim import FlatAdamW
        self.model, self.fmt, self.interval = model, fmt, requant_interval
        self.flat = model.flatten()
        self.opt = FlatAdamW(self.flat, lr=lr, weight_decay=0.0)
        self.lr, self.steps = lr, 0

    def train_step(self, ids, labels):
        loss = self.model.forward_backward(ids, labels)
        self.opt.step(self.lr)
        self.steps += 1
        if self.fmt and self.steps % self.interval == 0:
            for p in self.model.parameters():
                if p.dim() >= 2 and p.numel() >= 1024:
                    ste_roundtrip_(p.data, self.fmt)
        return float(loss)

    # ---- the reference's surface (include/quant/finetune.h: FineTuneConfig / FineTuner) -----------------------------------
    def configure(self, learning_rate: Optional[float] = None, num_epochs: int = 1, batch_size: int = 4, seq_length: int = 512,
                  log_interval: int = 10, save_interval: int = 100, grad_threshold: float = 1e-6, max_grad_norm: float = 1.0,
                  output_path: str = "finetuned.quant", tokenizer=None, log=None):
        if learning_rate is not None:
            self.lr = learning_rate
        self.opt.max_grad_norm = max_grad_norm
        self.cfg = dict(num_epochs=num_epochs, batch_size=batch_size, seq_length=seq_length, log_interval=log_interval,
                        save_interval=save_interval, grad_threshold=grad_threshold, output_path=output_path)
        self.tok, self.log = tokenizer, log
        return self

    def fine_tune(self, data):
        """``data``: a text file (tokenised with the configured tokenizer) or a loader with ``next_batch()`` / ``len``.
        Runs the configured epochs, saves at the save interval and at the end; returns the last loss."""
        from .trainer import DataLoader
        c = getattr(self, "cfg", None) or self.configure().cfg
        dl = DataLoader(self.tok, data, c["batch_size"], c["seq_length"]) if isinstance(data, (str, os.PathLike)) else data
        dev = self.model.tok_embeddings.device
        loss = 0.0
        for _ in range(c["num_epochs"]):
            dl.reset()
            for _ in range(len(dl)):
                ids, labels = dl.next_batch()
                loss = self.train_step(ids.to(dev), labels.to(dev))
                if self.log and c["log_interval"] and self.steps % c["log_interval"] == 0:
                    self.log(self.steps, loss)
                if c["save_interval"] and self.steps % c["save_interval"] == 0:
                    self.save(c["output_path"])
        self.save(c["output_path"])
        return loss

    @staticmethod
    def find_trainable_blocks(gradients: torch.Tensor, threshold: float = 1e-6, block: int = 256) -> List[int]:
        """Indices of the ``block``-weight blocks whose mean |gradient| exceeds the threshold: the blocks worth updating."""
        g = gradients.detach().float().reshape(-1)
        pad = (-g.numel()) % block
        if pad:
            g = torch.cat([g, torch.zeros(pad, device=g.device)])
        return (g.view(-1, block).abs().mean(1) > threshold).nonzero().reshape(-1).tolist()

    def apply_quant_update(self, fp32_grad: torch.Tensor, quant_weight: torch.Tensor, fmt=None, lr: Optional[float] = None):
        """Straight-through step on a weight that is stored in a block format: w <- roundtrip_fmt(w - lr * grad), in place."""
        quant_weight.add_(fp32_grad.to(quant_weight.dtype), alpha=-(self.lr if lr is None else lr))
        return ste_roundtrip_(quant_weight, fmt or self.fmt or "q16")

    def save(self, path: str):
        from ..quant import codec
        codec.save_model(self.model, path)
        return path
