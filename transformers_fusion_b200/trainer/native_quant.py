"""Training directly in a quantised weight representation.

``NativeQWeightStore`` holds every weight as (block format, index, block scale): the most sensitive blocks in an 8-bit
format (256-entry codebook), the bulk in a ternary format {-1, 0, +1} x scale, the rest in a 4-bit format (16-entry
codebook).  ``apply_quant_update`` is a two-time-scale SGD: the continuous block scales follow their gradient with
``lr_scale``; the indices follow a *virtual* fp32 weight that accumulates ``lr_weight * grad`` and flips an index only
when the accumulated move leaves the dead zone around the current centroid (half the distance to the neighbouring
centroid, times ``dead_zone_scale``).  ``NativeQUANTTrainer`` runs fp32 warm-up steps, allocates formats by a
moving-average gradient-norm sensitivity, and then trains with dequantise -> fused forward/backward -> quantised update.
All tensor work stays on the model's device.

Reference counterparts: include/quant/native_weight.h:13-170, native_trainer.h:13-135, src/trainer/native_weight.cpp,
native_trainer.cpp."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch

Q8, Q1, Q4 = 0, 1, 2
FORMAT_NAMES = {Q8: "native_quant8", Q1: "native_quant1", Q4: "native_quant4"}


def _codebook(n):
    """Symmetric normal-quantile codebook with n entries scaled to [-1, 1]."""
    p = (torch.arange(n, dtype=torch.float64) + 0.5) / n
    c = torch.erfinv(2 * p - 1) * (2 ** 0.5)
    return (c / c.abs().max()).float()


@dataclass
class NativeTrainConfig:
    block_size: int = 128
    warmup_steps: int = 100
    frac_quant8: float = 0.01
    frac_quant: float = 0.95
    lr_scale: float = 1e-4
    lr_weight: float = 1e-4
    lr_decay: float = 0.0
    weight_decay: float = 1e-2
    dead_zone_scale: float = 1.0
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-8
    batch_size: int = 8
    seq_length: int = 512
    max_steps: int = 10000
    log_interval: int = 10
    eval_interval: int = 100
    save_interval: int = 1000
    output_dir: str = "./checkpoints"
    sens_window: int = 10
    warmup_lr: float = 1e-3


@dataclass
class NativeTrainMetrics:
    loss: float = 0.0
    scale_lr: float = 0.0
    weight_lr: float = 0.0
    grad_norm: float = 0.0
    frozen_fraction: float = 0.0
    quant8_count: int = 0
    quant1_count: int = 0
    quant_count: int = 0
    avg_scale: float = 1.0


class NativeQWeightStore:
    def __init__(self, num_weights: int, block_size: int = 128, device="cpu"):
        self.n, self.bs = num_weights, block_size
        self.nb = (num_weights + block_size - 1) // block_size
        self.device = torch.device(device)
        self.formats = torch.full((self.nb,), Q1, dtype=torch.uint8, device=self.device)
        self.indices = torch.zeros(self.nb * block_size, dtype=torch.uint8, device=self.device)
        self.scales = torch.ones(self.nb, dtype=torch.float32, device=self.device)
        self.virtual = torch.zeros(self.nb * block_size, dtype=torch.float32, device=self.device)   # accumulated sub-threshold moves
        self.frozen = torch.zeros(self.nb * block_size, dtype=torch.bool, device=self.device)
        self.cb8 = _codebook(256).to(self.device)
        self.cb4 = _codebook(16).to(self.device)
        self.cb1 = torch.tensor([-1.0, 0.0, 1.0], device=self.device)
        self.dead_zone_scale = 1.0

    # ---- helpers
    def _cb(self, fmt):
        return {Q8: self.cb8, Q1: self.cb1, Q4: self.cb4}[fmt]

    def _pad(self, x):
        out = torch.zeros(self.nb * self.bs, dtype=torch.float32, device=self.device)
        out[: self.n] = x.reshape(-1).float().to(self.device)
        return out.view(self.nb, self.bs)

    def size(self):
        return self.n

    def num_blocks(self):
        return self.nb

    def counts(self):
        return {f: int((self.formats == f).sum()) for f in (Q8, Q1, Q4)}

    # ---- allocation / conversion
    def allocate(self, sensitivity: Optional[torch.Tensor], frac_quant8=0.01, frac_quant1=0.95):
        """Per-block formats: the top ``frac_quant8`` blocks by sensitivity -> 8-bit, the next ``frac_quant1`` -> ternary,
        the remainder -> 4-bit."""
        if sensitivity is None:
            score = torch.zeros(self.nb, device=self.device)
        else:
            score = self._pad(sensitivity).abs().mean(1)
        order = torch.argsort(score, descending=True, stable=True)
        n8 = int(round(frac_quant8 * self.nb))
        n1 = min(self.nb - n8, int(round(frac_quant1 * self.nb)))
        self.formats[order[:n8]] = Q8
        self.formats[order[n8:n8 + n1]] = Q1
        self.formats[order[n8 + n1:]] = Q4

    def initialize(self, fp32_weights, sensitivity=None, frac_quant8=0.01, frac_quant1=0.95):
        self.allocate(sensitivity, frac_quant8, frac_quant1)
        self.convert_from_fp32(fp32_weights)

    def convert_from_fp32(self, src):
        w = self._pad(src)
        idx = torch.zeros_like(w, dtype=torch.uint8)
        for fmt in (Q8, Q1, Q4):
            rows = (self.formats == fmt).nonzero().reshape(-1)
            if rows.numel() == 0:
                continue
            cb = self._cb(fmt)
            blk = w[rows]
            if fmt == Q1:
                s = blk.abs().mean(1).clamp(min=1e-12) * 1.5      # ternary threshold at s/2 ~ 0.75 mean|w|
            else:
                s = blk.abs().amax(1).clamp(min=1e-12)
            self.scales[rows] = s
            x = blk / s[:, None]
            if fmt == Q1:
                idx[rows] = (torch.where(x > 0.5, 2, torch.where(x < -0.5, 0, 1))).to(torch.uint8)
            else:
                idx[rows] = torch.bucketize(x, (cb[1:] + cb[:-1]) / 2).to(torch.uint8)
        self.indices = idx.view(-1)
        self.virtual.zero_()

    def reallocate_by_sensitivity(self, sensitivity, frac_quant8=0.01, frac_quant1=0.95):
        w = self.dequantize()
        self.allocate(sensitivity, frac_quant8, frac_quant1)
        self.convert_from_fp32(w)

    def dequantize(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        idx = self.indices.view(self.nb, self.bs).long()
        w = torch.empty((self.nb, self.bs), dtype=torch.float32, device=self.device)
        for fmt in (Q8, Q1, Q4):
            rows = (self.formats == fmt).nonzero().reshape(-1)
            if rows.numel():
                w[rows] = self._cb(fmt)[idx[rows]] * self.scales[rows, None]
        flat = w.view(-1)[: self.n]
        if out is not None:
            out.copy_(flat.view(out.shape).to(out.dtype))
            return out
        return flat

    # ---- the quantised update
    def apply_quant_update(self, grad, lr_scale, lr_weight, weight_decay=0.0):
        """Two-time-scale SGD step.  Returns the fraction of weights whose index stayed inside its dead zone."""
        g = self._pad(grad)
        idx = self.indices.view(self.nb, self.bs).long()
        virt = self.virtual.view(self.nb, self.bs)
        moved = torch.zeros_like(idx, dtype=torch.bool)
        for fmt in (Q8, Q1, Q4):
            rows = (self.formats == fmt).nonzero().reshape(-1)
            if rows.numel() == 0:
                continue
            cb = self._cb(fmt)
            c = cb[idx[rows]]
            s = self.scales[rows]
            # scale: d loss / d s = sum_i g_i * c_i  (w_i = c_i * s), decoupled weight decay
            gs = (g[rows] * c).sum(1)
            # a step may change a scale by at most 10 %: one large gradient must not flip its sign or collapse it
            s_new = s * (1 - lr_scale * weight_decay) - lr_scale * gs
            self.scales[rows] = torch.minimum(torch.maximum(s_new, 0.9 * s), 1.1 * s).clamp(min=1e-12)
            # virtual weight (in centroid units): accumulate the step, flip the index when it leaves the dead zone
            v = virt[rows] - lr_weight * g[rows] / s[:, None]
            i = idx[rows]
            up = cb[(i + 1).clamp(max=cb.numel() - 1)] - c
            dn = c - cb[(i - 1).clamp(min=0)]
            go_up = (v > 0.5 * up * self.dead_zone_scale) & (i < cb.numel() - 1)
            go_dn = (v < -0.5 * dn * self.dead_zone_scale) & (i > 0)
            i2 = i + go_up.long() - go_dn.long()
            v = torch.where(go_up, v - up, torch.where(go_dn, v + dn, v))
            idx[rows] = i2
            virt[rows] = v
            moved[rows] = go_up | go_dn
        self.indices = idx.to(torch.uint8).view(-1)
        self.frozen = (~moved).view(-1)
        return float((~moved).float().mean())

    def get_weight(self, i):
        b = i // self.bs
        return float(self._cb(int(self.formats[b]))[int(self.indices[i])] * self.scales[b])

    # ---- element / buffer access (reference: NativeQWeightStore, include/quant/native_weight.h:127-143)
    def block_size(self) -> int: return self.bs
    def get_index(self, i: int) -> int: return int(self.indices[i])
    def get_scale(self, i: int) -> float: return float(self.scales[i // self.bs])
    def get_format(self, i: int) -> int: return int(self.formats[i // self.bs])
    def indices_data(self) -> torch.Tensor: return self.indices          # uint8 [num_blocks * block_size], writable
    def block_scales_data(self) -> torch.Tensor: return self.scales      # fp32 [num_blocks], writable
    def formats_data(self) -> torch.Tensor: return self.formats          # uint8 [num_blocks]

    @staticmethod
    def global_codebook() -> torch.Tensor:
        """The shared 256-entry codebook of the 8-bit blocks (every store uses the same table)."""
        return _codebook(256)

    @staticmethod
    def global_quant4_codebook() -> torch.Tensor:
        return _codebook(16)

    def bits_per_weight(self):
        c = self.counts()
        return (8 * c[Q8] + 2 * c[Q1] + 4 * c[Q4]) / max(1, self.nb) + 32.0 / self.bs

    def state(self):
        return {"formats": self.formats.cpu(), "indices": self.indices.cpu(), "scales": self.scales.cpu(), "n": self.n, "bs": self.bs}

    def load_state(self, st):
        self.formats, self.indices, self.scales = (st[k].to(self.device) for k in ("formats", "indices", "scales"))
        self.virtual.zero_()


class NativeQUANTTrainer:
    def __init__(self, model, cfg: Optional[NativeTrainConfig] = None):
        self.model, self.cfg = model, cfg or NativeTrainConfig()
        self.flat = model.flatten()
        dev = self.flat.params.device
        self.store = NativeQWeightStore(self.flat.numel, self.cfg.block_size, dev)
        self.store.dead_zone_scale = self.cfg.dead_zone_scale
        self.master = self.flat.params.float().clone()          # fp32 copy used only during warm-up
        self.sens = torch.zeros(self.flat.numel, device=dev)
        self.step_count = 0
        self.native = False
        self.best_eval = float("inf")

    def weight_store(self):
        return self.store

    def config(self) -> NativeTrainConfig:
        return self.cfg

    def warmup_phase(self, batches) -> float:
        """The floating-point warm-up as one call: a warm-up step on every (ids, labels) batch until ``warmup_steps`` steps
        have been taken or the batches run out, then the transition to the quantised store.  Returns the last loss."""
        loss = 0.0
        for ids, labels in batches:
            if self.native or self.step_count >= self.cfg.warmup_steps:
                break
            self.step_count += 1
            loss = self.warmup_step(ids, labels)
        if not self.native:
            self.transition()
        return loss

    def _update_sensitivity(self):
        a = 1.0 / self.cfg.sens_window
        self.sens.mul_(1 - a).add_(self.flat.grads.abs(), alpha=a)

    def _push(self):
        self.store.dequantize(self.flat.params)

    def warmup_step(self, ids, labels):
        self.flat.zero_grad()
        loss = self.model.forward_backward(ids, labels)
        self._update_sensitivity()
        self.master.add_(self.flat.grads, alpha=-self.cfg.warmup_lr)
        self.flat.params.copy_(self.master.to(self.flat.params.dtype))
        return float(loss)

    def transition(self):
        """fp32 -> native quantised representation with sensitivity-driven format allocation."""
        c = self.cfg
        self.store.initialize(self.master, self.sens, c.frac_quant8, c.frac_quant)
        self._push()
        self.native = True

    def train_step(self, ids, labels) -> NativeTrainMetrics:
        c = self.cfg
        self.step_count += 1
        m = NativeTrainMetrics()
        if not self.native:
            m.loss = self.warmup_step(ids, labels)
            if self.step_count >= c.warmup_steps:
                self.transition()
        else:
            self.flat.zero_grad()
            m.loss = float(self.model.forward_backward(ids, labels))
            self._update_sensitivity()
            decay = 1.0 / (1.0 + c.lr_decay * (self.step_count - c.warmup_steps))
            m.scale_lr, m.weight_lr = c.lr_scale * decay, c.lr_weight * decay
            m.grad_norm = float(self.flat.grads.norm())
            m.frozen_fraction = self.store.apply_quant_update(self.flat.grads, m.scale_lr, m.weight_lr, c.weight_decay)
            self._push()
        cnt = self.store.counts()
        m.quant8_count, m.quant1_count, m.quant_count = cnt[Q8], cnt[Q1], cnt[Q4]
        m.avg_scale = float(self.store.scales.mean())
        return m

    def train(self, batches, eval_batches=()):
        out = []
        for ids, labels in batches:
            out.append(self.train_step(ids, labels))
            if eval_batches and self.step_count % self.cfg.eval_interval == 0:
                self.best_eval = min(self.best_eval, self.evaluate(eval_batches))
            if self.step_count >= self.cfg.max_steps:
                break
        return out

    @torch.no_grad()
    def evaluate(self, batches):
        tot, n = 0.0, 0
        for ids, labels in batches:
            logits = self.model.forward(ids).float()
            tot += float(torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1)))
            n += 1
        return tot / max(1, n)

    def save_checkpoint(self, path):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        torch.save({"store": self.store.state(), "step": self.step_count, "native": self.native, "sens": self.sens.cpu(),
                    "master": self.master.cpu()}, path)

    def load_checkpoint(self, path):
        st = torch.load(path, map_location="cpu", weights_only=False)
        self.store.load_state(st["store"])
        self.step_count, self.native = st["step"], st["native"]
        self.sens, self.master = st["sens"].to(self.sens.device), st["master"].to(self.master.device)
        if self.native:
            self._push()
        else:
            self.flat.params.copy_(self.master.to(self.flat.params.dtype))


# ----------------------------------------------------------------------------------------------- MoE in native low-bit form
@dataclass
class NativeMoEConfig:
    hidden_size: int = 512
    num_heads: int = 8
    ffn_hidden: int = 1024
    num_layers: int = 4
    num_experts: int = 8
    top_k: int = 2
    load_balance_coef: float = 0.01
    z_loss_coef: float = 0.001
    block_size: int = 128
    frac_quant8: float = 0.01
    frac_quant: float = 0.95
    vocab_size: int = 256
    max_seq_len: int = 128


@dataclass
class NativeMoEMetrics:
    loss: float = 0.0
    lb_loss: float = 0.0
    z_loss: float = 0.0
    grad_norm: float = 0.0
    frozen_pct: float = 0.0
    quant8: int = 0
    quant: int = 0
    quant1: int = 0
    total_params: int = 0
    active_params: int = 0


class NativeQUANTMoEModel:
    """MoE language model whose large tensors (embedding, LM head, every expert's gate/up and down matrices) live in
    NativeQWeightStore form and are updated there; attention, norms and routers stay in floating point with plain SGD.
    Before each step the stores are expanded into the model's parameters, after backward they take the gradients.

    Reference counterpart: NativeQUANTMoEModel (include/quant/native_quant_moe.h:11-76, src/model/native_quant_moe.cpp)."""

    def __init__(self, cfg: Optional[NativeMoEConfig] = None, device="cpu", seed: int = 0):
        from ..models.config import MoEConfig
        from ..models.moe import MoEModel
        self.cfg = cfg = cfg or NativeMoEConfig()
        mc = MoEConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_layers=cfg.num_layers, num_heads=cfg.num_heads,
                       ffn_hidden_size=cfg.ffn_hidden, max_seq_len=cfg.max_seq_len, num_experts=cfg.num_experts, top_k=cfg.top_k,
                       load_balance_weight=cfg.load_balance_coef, router_z_weight=cfg.z_loss_coef, init_std=0.05)
        dev = torch.device(device)
        self.model = MoEModel(mc, device=dev, dtype=torch.float32 if dev.type == "cpu" else torch.bfloat16, seed=seed)
        self.model.flatten()
        self.stores: List[tuple] = []           # (parameter, store)
        self.total_params_ = sum(p.numel() for p in self.model.parameters())

    def _stored_tensors(self):
        m = self.model
        out = [m.tok_embeddings]
        if m.lm_head is not m.tok_embeddings:
            out.append(m.lm_head)
        for blk in m.layers:
            out += [blk.gate_up, blk.down]
        return out

    def init_from_fp32(self):
        c = self.cfg
        self.stores = []
        for p in self._stored_tensors():
            st = NativeQWeightStore(p.numel(), c.block_size, p.device)
            st.initialize(p.data.float().reshape(-1), None, c.frac_quant8, c.frac_quant)
            self.stores.append((p, st))
        self.push_weights()

    def push_weights(self):
        for p, st in self.stores:
            p.data.copy_(st.dequantize().view(p.shape).to(p.dtype))

    def total_params(self) -> int: return self.total_params_

    def forward(self, ids):
        return self.model(ids)

    def step(self, ids, labels, lr_s: float, lr_w: float) -> NativeMoEMetrics:
        if not self.stores:
            self.init_from_fp32()
        m = self.model
        m.flat.zero_grad()
        loss = float(m.forward_backward(ids, labels))
        met = NativeMoEMetrics(loss=loss, total_params=self.total_params_)
        met.lb_loss = float(m.last_aux.detach()) if m.last_aux is not None else 0.0
        met.grad_norm = float(m.flat.grads.norm())
        stored = {id(p) for p, _ in self.stores}
        frozen = []
        for p, st in self.stores:
            frozen.append(st.apply_quant_update(p.main_grad.reshape(-1).float(), lr_s, lr_w))
            cnt = st.counts()
            met.quant8 += cnt[Q8]
            met.quant1 += cnt[Q1]
            met.quant += cnt[Q4]
        with torch.no_grad():
            for p in m.parameters():
                if id(p) not in stored and getattr(p, "main_grad", None) is not None:
                    p.data.add_(p.main_grad.to(p.dtype), alpha=-lr_w)
        self.push_weights()
        met.frozen_pct = 100.0 * sum(frozen) / max(1, len(frozen))
        per_expert = (m.layers[0].gate_up.numel() + m.layers[0].down.numel()) // self.cfg.num_experts
        met.active_params = self.total_params_ - self.cfg.num_layers * (self.cfg.num_experts - self.cfg.top_k) * per_expert
        return met

    # ---- the step in its three parts (reference: forward / backward / apply_update, include/quant/native_quant_moe.h:44-46)
    def backward(self, ids, labels) -> float:
        """Forward and backward through the fused training path: gradients land in the model's flat gradient buffer (the
        stores are created from the current weights on first use).  Returns the loss."""
        if not self.stores:
            self.init_from_fp32()
        self.model.flat.zero_grad()
        return float(self.model.forward_backward(ids, labels))

    def apply_update(self, lr_scale: float, lr_weight: float) -> float:
        """Take the gradients left by ``backward``: quantised update of every stored tensor, plain SGD on the rest, then the
        stores are expanded into the model again.  Returns the mean fraction of weights whose index did not move."""
        m = self.model
        stored = {id(p) for p, _ in self.stores}
        frozen = [st.apply_quant_update(p.main_grad.reshape(-1).float(), lr_scale, lr_weight) for p, st in self.stores]
        with torch.no_grad():
            for p in m.parameters():
                if id(p) not in stored and getattr(p, "main_grad", None) is not None:
                    p.data.add_(p.main_grad.to(p.dtype), alpha=-lr_weight)
        self.push_weights()
        return sum(frozen) / max(1, len(frozen))

    def print_memory_report(self) -> str:
        r = self.memory_report()
        text = (f"native-quant MoE memory: {r['stored_params']:,} stored weights at {r['stored_bits_per_weight']:.2f} bits, "
                f"{r['float_params']:,} floating-point weights; {r['bytes'] / 1e6:.2f} MB vs {r['fp32_bytes'] / 1e6:.2f} MB in fp32 "
                f"({r['fp32_bytes'] / max(1.0, r['bytes']):.1f}x smaller)")
        print(text)
        return text

    def memory_report(self) -> dict:
        bits = sum(st.bits_per_weight() * st.size() for _, st in self.stores)
        n = sum(st.size() for _, st in self.stores)
        rest = self.total_params_ - n
        return {"stored_params": n, "stored_bits_per_weight": bits / max(1, n), "float_params": rest,
                "bytes": bits / 8 + rest * 4, "fp32_bytes": self.total_params_ * 4}
