"""Dense training engine facade: one object that owns the trainer, schedule and statistics, plus the stand-alone helpers
(losses with explicit gradients, optimiser suite with parameter groups, token loaders, augmentation, curriculum,
bare parameter checkpoints, policy-gradient utilities, evaluation harness).

Reference counterparts: engines/trainer/dense/trainer.h:18-85, optim.h:13-58, loss.h:10-40, dataloader.h:12-88,
unified.h:13-61, eval.h:12-47."""
from __future__ import annotations

import math
import struct
import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn.functional as TF

from ..trainer import training_utils as TU
from ..trainer.optimizers import build_optimizer
from ..trainer.schedulers import schedule_lr
from ..trainer.trainer import DataLoader, TrainConfig, Trainer, UnifiedTrainArgs, UnifiedTrainer, unified_trainer_parse_kind
from ..utils import metrics as MX


# ----------------------------------------------------------------------------------------------- schedule / statistics
@dataclass
class DenseStats:
    steps: int = 0
    tokens: int = 0
    tok_per_sec: float = 0.0
    last_loss: float = 0.0
    last_grad_norm: float = 0.0
    last_lr: float = 0.0
    best_val_loss: float = 1e30
    eval_batches: int = 0


@dataclass
class LRSchedule:
    kind: str = "WARMUP_COSINE"
    base_lr: float = 3e-4
    warmup_steps: int = 100
    total_steps: int = 10000
    min_lr_ratio: float = 0.1

    def lr_at(self, step: int) -> float:
        return schedule_lr(self.kind, self.base_lr, step, self.total_steps, self.warmup_steps, self.min_lr_ratio)


@dataclass
class EvalOut:
    loss: float = 0.0
    perplexity: float = 0.0
    batches: int = 0
    tokens: int = 0


def eval_loop(trainer: Trainer, dl, max_batches: int = 20) -> EvalOut:
    """Mean next-token loss of up to ``max_batches`` batches, without touching gradients."""
    out, tot = EvalOut(), 0.0
    dl.reset()
    with torch.no_grad():
        for _ in range(min(max_batches, len(dl))):
            ids, labels = dl.next_batch()
            logits = trainer.model(ids).float()
            tot += float(TF.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1)))
            out.batches += 1
            out.tokens += ids.numel()
    if out.batches:
        out.loss = tot / out.batches
        out.perplexity = math.exp(min(out.loss, 20.0))
    return out


def global_grad_norm(params: Sequence[torch.Tensor]) -> float:
    sq = 0.0
    for p in params:
        g = getattr(p, "main_grad", None)
        g = g if g is not None else p.grad
        if g is not None:
            sq += float(g.float().pow(2).sum())
    return math.sqrt(sq)


def add_grad_noise(params: Sequence[torch.Tensor], eta: float, gamma: float, step: int, generator=None) -> None:
    """Annealed Gaussian gradient noise with variance eta / (1 + step)^gamma."""
    std = math.sqrt(eta / (1.0 + step) ** gamma)
    for p in params:
        g = getattr(p, "main_grad", None)
        g = g if g is not None else p.grad
        if g is not None:
            g.add_(torch.randn(g.shape, generator=generator, device="cpu").to(g.device, g.dtype) * std)


class DenseTrainer:
    """Trainer plus running statistics; every call forwards to the underlying Trainer and records what it did."""

    def __init__(self, model, tokenizer=None):
        self.model, self.tok = model, tokenizer
        self.trainer = Trainer(model, tokenizer)
        self.cfg = TrainConfig()
        self._stats = DenseStats()
        self._t0 = time.perf_counter()
        self._continual = None

    def compile(self, optimizer=None, cfg: Optional[TrainConfig] = None):
        self.cfg = cfg or self.cfg
        self.trainer.compile(optimizer, self.cfg)
        self._t0 = time.perf_counter()
        return self

    def _record(self, loss, ids):
        s, m = self._stats, self.trainer.metrics()
        s.steps += 1
        s.tokens += ids.numel()
        s.last_loss, s.last_grad_norm, s.last_lr = float(loss), m.grad_norm, m.learning_rate
        s.tok_per_sec = s.tokens / max(1e-9, time.perf_counter() - self._t0)

    def train_step(self, ids, labels) -> float:
        loss = self.trainer.train_step(ids, labels)
        if self._continual is not None:
            self._continual.after_step(self.model)
        self._record(loss, ids)
        return loss

    def micro_step(self, ids, labels, loss_scale: float = 1.0) -> float:
        return self.trainer.micro_step(ids, labels, loss_scale)

    def fit(self, dl, cfg: Optional[TrainConfig] = None, val_dl=None):
        r = self.trainer.fit(dl, cfg, val_dl)
        m = self.trainer.metrics()
        self._stats.steps, self._stats.last_loss = m.step, m.loss
        if val_dl is not None:
            self._stats.best_val_loss = min(self._stats.best_val_loss, m.val_loss)
        return r

    def eval_loss(self, val_dl, max_batches: int = 20) -> float:
        v = self.trainer.eval_loss(val_dl, max_batches)
        self._stats.eval_batches += min(max_batches, len(val_dl))
        self._stats.best_val_loss = min(self._stats.best_val_loss, v)
        return v

    def clip_gradients(self, max_norm: float) -> float: return self.trainer.clip_gradients(max_norm)
    def save_checkpoint(self, path): self.trainer.save_checkpoint(path)
    def load_checkpoint(self, path): self.trainer.load_checkpoint(path)
    def set_log_callback(self, cb): self.trainer.set_log_callback(cb)
    def set_step_callback(self, cb): self.trainer.set_step_callback(cb)
    def metrics(self): return self.trainer.metrics()
    def stats(self) -> DenseStats: return self._stats

    def enable_qat(self, bits: int = 8, symmetric: bool = True):
        self.cfg.qat_bits, self.cfg.qat_symmetric = bits, symmetric
        self.trainer.cfg = self.cfg

    def disable_qat(self):
        self.cfg.qat_bits = 0

    def enable_continual(self, cfg=None):
        from ..trainer.continual import ContinualLearner
        self._continual = ContinualLearner(self.model, cfg) if cfg is not None else ContinualLearner(self.model)

    def disable_continual(self):
        self._continual = None

    def ema_init(self, decay: float = 0.999): self.trainer.ema_init(decay)
    def ema_step(self): self.trainer.ema_step()

    def inject_gradient_noise(self, step: int):
        self.trainer.inject_gradient_noise(step, self.cfg.grad_noise_eta, self.cfg.grad_noise_gamma)


# ----------------------------------------------------------------------------------------------- optimiser suite
@dataclass
class OptimStats:
    steps: int = 0
    last_lr: float = 0.0
    last_update_norm: float = 0.0


class _Flat:
    """The flat parameter / gradient view the optimisers work on, built over loose tensors."""

    def __init__(self, ps):
        self.params_list = list(ps)
        self.offsets, n = [], 0
        for p in self.params_list:
            self.offsets.append(n)
            n += p.numel()
        self.numel = n
        dev = self.params_list[0].device if self.params_list else "cpu"
        self.params = torch.cat([p.detach().float().reshape(-1) for p in self.params_list]) if n else torch.zeros(0, device=dev)
        self.grads = torch.zeros_like(self.params)


class OptimSuite:
    """One optimiser chosen by name over several parameter groups with their own lr / weight-decay multipliers.
    Each group is flattened into one fp32 master vector (the layout the flat optimisers work on) and written back."""

    KINDS = ("adamw", "adam", "adafactor", "sgd", "lion")

    def __init__(self, kind: str = "adamw", lr: float = 3e-4, wd: float = 1e-2):
        kind = kind.lower()
        if kind not in self.KINDS:
            raise ValueError(f"unknown optimiser '{kind}'")
        self.kind, self.lr, self.wd = kind, lr, wd
        self.groups: List[dict] = []
        self._sched = None
        self._stats = OptimStats()

    def add_params(self, ps: Sequence[torch.Tensor]):
        self.add_group(ps, 1.0, 1.0)

    def add_group(self, ps: Sequence[torch.Tensor], lr_scale: float, wd_scale: float):
        ps = list(ps)
        flat = _Flat(ps)
        opt = build_optimizer(self.kind, flat, lr=self.lr * lr_scale, weight_decay=self.wd * wd_scale, max_grad_norm=0.0)
        self.groups.append(dict(params=ps, flat=flat, opt=opt, lr_scale=lr_scale, wd_scale=wd_scale))

    def _gather_grads(self, g):
        fl = g["flat"]
        for p, off in zip(fl.params_list, fl.offsets):
            gr = getattr(p, "main_grad", None)
            gr = gr if gr is not None else p.grad
            fl.grads[off:off + p.numel()] = 0 if gr is None else gr.detach().float().reshape(-1)

    def step(self):
        upd = 0.0
        for g in self.groups:
            fl = g["flat"]
            self._gather_grads(g)
            before = fl.params.clone()
            g["opt"].step(self.lr * g["lr_scale"])
            upd += float((fl.params - before).pow(2).sum())
            for p, off in zip(fl.params_list, fl.offsets):
                p.data.copy_(fl.params[off:off + p.numel()].view(p.shape).to(p.dtype))
        self._stats.steps += 1
        self._stats.last_lr, self._stats.last_update_norm = self.lr, math.sqrt(upd)

    def zero_grad(self):
        for g in self.groups:
            g["flat"].grads.zero_()
            for p in g["params"]:
                p.grad = None
                if getattr(p, "main_grad", None) is not None:
                    p.main_grad.zero_()

    def set_lr(self, lr: float): self.lr = lr
    def get_lr(self) -> float: return self.lr

    def set_schedule(self, kind: str, warmup: int, total: int):
        self._sched = LRSchedule(kind, self.lr, warmup, total, 0.0)

    def scheduler_step(self, step: int):
        if self._sched is not None:
            self.lr = self._sched.lr_at(step)

    def clip(self, max_norm: float) -> float:
        ps = [p for g in self.groups for p in g["params"]]
        norm = global_grad_norm(ps)
        if max_norm > 0 and norm > max_norm:
            for p in ps:
                gr = getattr(p, "main_grad", None)
                gr = gr if gr is not None else p.grad
                if gr is not None:
                    gr.mul_(max_norm / (norm + 1e-6))
        return norm

    def stats(self) -> OptimStats: return self._stats

    @staticmethod
    def param_norm(ps) -> float:
        return math.sqrt(sum(float(p.detach().float().pow(2).sum()) for p in ps))

    @staticmethod
    def snapshot(ps) -> List[torch.Tensor]:
        return [p.detach().clone() for p in ps]

    @staticmethod
    def update_norm(before, after) -> float:
        return math.sqrt(sum(float((a.detach().float() - b.float()).pow(2).sum()) for b, a in zip(before, after)))


# ----------------------------------------------------------------------------------------------- losses with gradients
@dataclass
class LossOut:
    loss: float = 0.0
    acc: float = 0.0


def _rows(logits, labels):
    return logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1)


def _acc(lg, lab, keep):
    return float((lg.argmax(-1)[keep] == lab[keep]).float().mean()) if keep.any() else 0.0


def ce_loss(logits, labels, ignore_index: int = -100):
    """Mean cross entropy over the kept rows; returns (LossOut, dlogits) with dlogits = (softmax - onehot) / n_kept."""
    return label_smooth_ce(logits, labels, 0.0, ignore_index)


def label_smooth_ce(logits, labels, smoothing: float = 0.1, ignore_index: int = -100):
    lg, lab = _rows(logits, labels)
    keep = lab != ignore_index
    n = max(1, int(keep.sum()))
    lp = torch.log_softmax(lg, -1)
    tgt = torch.full_like(lp, smoothing / lg.shape[-1])
    tgt.scatter_add_(1, lab.clamp(min=0)[:, None], torch.full((lg.shape[0], 1), 1.0 - smoothing, device=lg.device))
    loss = -(tgt * lp).sum(-1)
    d = (lp.exp() - tgt) * keep[:, None] / n
    return LossOut(float((loss * keep).sum() / n), _acc(lg, lab, keep)), d.view(logits.shape)


def focal_loss(logits, labels, gamma: float = 2.0, alpha: float = 0.25, ignore_index: int = -100):
    """alpha * (1 - p_t)^gamma * (-log p_t), averaged over kept rows; the gradient comes from autograd on the fp32 copy."""
    lg, lab = _rows(logits, labels)
    lg = lg.detach().requires_grad_(True)
    keep = lab != ignore_index
    n = max(1, int(keep.sum()))
    lpt = torch.log_softmax(lg, -1).gather(1, lab.clamp(min=0)[:, None])[:, 0]
    loss = (-(alpha * (1 - lpt.exp()) ** gamma) * lpt * keep).sum() / n
    (d,) = torch.autograd.grad(loss, lg)
    return LossOut(float(loss.detach()), _acc(lg.detach(), lab, keep)), d.view(logits.shape)


@dataclass
class RDropOut:
    ce: float = 0.0
    kl: float = 0.0
    total: float = 0.0


def rdrop_loss(logits1, logits2, labels, alpha: float = 1.0, ignore_index: int = -100) -> RDropOut:
    ce = 0.5 * (TU.cross_entropy_loss(logits1, labels, ignore_index) + TU.cross_entropy_loss(logits2, labels, ignore_index))
    p, q = torch.log_softmax(logits1.float(), -1), torch.log_softmax(logits2.float(), -1)
    kl = 0.5 * ((p.exp() * (p - q)).sum(-1) + (q.exp() * (q - p)).sum(-1)).mean()
    return RDropOut(float(ce), float(kl), float(ce + alpha * kl))


def infonce_loss(emb, pos, temperature: float = 0.07):
    """Row i of ``emb`` should match row i of ``pos``; returns (loss, demb, dpos)."""
    a, b = emb.detach().float().requires_grad_(True), pos.detach().float().requires_grad_(True)
    loss = TU.infonce_loss(a, b, temperature)
    da, db = torch.autograd.grad(loss, (a, b))
    return float(loss.detach()), da, db


def mse_loss_fn(pred, target):
    d = pred.float() - target.float()
    return LossOut(float(d.pow(2).mean()), 0.0), 2.0 * d / d.numel()


def seq_z_loss(logits) -> float:
    return float((torch.logsumexp(logits.float(), -1) ** 2).mean())


# ----------------------------------------------------------------------------------------------- data
class DenseDataLoader(DataLoader):
    """Whole-file token loader with epoch shuffling of the sequence order."""

    def __init__(self, tokenizer, data_path: str, batch_size: int, seq_length: int, tokens=None):
        super().__init__(tokenizer, data_path, batch_size, seq_length, tokens=tokens)
        self._order = None

    def num_batches(self) -> int: return len(self)
    def batch_size(self) -> int: return self.B
    def seq_length(self) -> int: return self.S

    def shuffle(self, epoch: int = 0):
        n_seq = (self.tokens.numel() - 1) // self.S
        g = torch.Generator().manual_seed(0x5EED + epoch)
        self._order = torch.randperm(n_seq, generator=g)
        self.offset = 0

    def next_batch(self):
        if self._order is None:
            return super().next_batch()
        B, S = self.B, self.S
        if (self.offset + 1) * B > self._order.numel():
            self.offset = 0
        rows = self._order[self.offset * B:(self.offset + 1) * B]
        self.offset += 1
        idx = rows[:, None] * S + torch.arange(S + 1)[None, :]
        chunk = self.tokens[idx]
        return chunk[:, :-1].contiguous(), chunk[:, 1:].contiguous()


class StreamDataLoader:
    """Reads the text in chunks of ``chunk_bytes`` and tokenises as it goes: memory stays bounded by one chunk."""

    def __init__(self, tokenizer, data_path: str, batch_size: int, seq_length: int, chunk_bytes: int = 1 << 20):
        self.tok, self.path, self.B, self.S, self.chunk = tokenizer, data_path, batch_size, seq_length, chunk_bytes
        self._f = open(data_path, "rb")
        self._buf: List[int] = []
        self._batches, self._eof = 0, False

    def batches_served(self) -> int: return self._batches

    def reset(self):
        self._f.seek(0)
        self._buf, self._eof = [], False

    def _refill(self):
        raw = self._f.read(self.chunk)
        if not raw:
            self._eof = True
            return
        self._buf.extend(self.tok.encode(raw.decode("utf-8", errors="ignore")))

    def next_batch(self):
        need = self.B * self.S + 1
        while len(self._buf) < need and not self._eof:
            self._refill()
        if len(self._buf) < need:
            return None
        t = torch.tensor(self._buf[:need], dtype=torch.long)
        del self._buf[:need - 1]
        self._batches += 1
        return t[:-1].view(self.B, self.S), t[1:].view(self.B, self.S)

    def close(self):
        self._f.close()


@dataclass
class AugmentPolicy:
    token_dropout: float = 0.0
    span_mask_prob: float = 0.0
    span_len: int = 8
    logit_noise_std: float = 0.0
    pad_id: int = 0
    seed: int = 1234

    def __post_init__(self):
        self._g = torch.Generator().manual_seed(self.seed)

    def apply_ids(self, ids: torch.Tensor) -> torch.Tensor:
        """In place: independent token dropout to ``pad_id`` and whole-span masking starting with span_mask_prob / span_len."""
        if self.token_dropout > 0:
            ids[torch.rand(ids.shape, generator=self._g) < self.token_dropout] = self.pad_id
        if self.span_mask_prob > 0:
            start = torch.rand(ids.shape, generator=self._g) < self.span_mask_prob / max(1, self.span_len)
            m = start.clone()
            for k in range(1, self.span_len):
                m[..., k:] |= start[..., :-k]
            ids[m] = self.pad_id
        return ids

    def apply_logits(self, logits: torch.Tensor) -> torch.Tensor:
        if self.logit_noise_std > 0:
            logits.add_(torch.randn(logits.shape, generator=self._g).to(logits.device, logits.dtype) * self.logit_noise_std)
        return logits


@dataclass
class Curriculum:
    min_len: int = 64
    max_len: int = 512
    total_epochs: int = 3
    current_epoch: int = 0

    def effective_len(self) -> int:
        f = min(1.0, self.current_epoch / max(1, self.total_epochs - 1))
        return int(self.min_len + f * (self.max_len - self.min_len))

    def difficulty_mix(self) -> float:
        return min(1.0, (self.current_epoch + 1) / max(1, self.total_epochs))


class DenseCheckpoint:
    """Bare parameter dump: magic 'TFDC', u32 version, i64 step, u32 count, then per tensor u64 numel + fp32 data."""

    MAGIC = b"TFDC"

    @staticmethod
    def save(path: str, params: Sequence[torch.Tensor], step: int) -> None:
        with open(path, "wb") as f:
            f.write(DenseCheckpoint.MAGIC + struct.pack("<IqI", 1, step, len(params)))
            for p in params:
                a = p.detach().float().cpu().contiguous()
                f.write(struct.pack("<Q", a.numel()))
                f.write(a.numpy().tobytes())

    @staticmethod
    def load(path: str, params: Sequence[torch.Tensor]) -> int:
        with open(path, "rb") as f:
            if f.read(4) != DenseCheckpoint.MAGIC:
                raise ValueError("not a dense checkpoint")
            _ver, step, n = struct.unpack("<IqI", f.read(16))
            if n != len(params):
                raise ValueError(f"checkpoint holds {n} tensors, the model has {len(params)}")
            for p in params:
                (numel,) = struct.unpack("<Q", f.read(8))
                if numel != p.numel():
                    raise ValueError("tensor size mismatch")
                buf = bytearray(f.read(numel * 4))
                p.data.copy_(torch.frombuffer(buf, dtype=torch.float32).view(p.shape).to(p.dtype))
        return step


# ----------------------------------------------------------------------------------------------- unified entry, RL helpers
@dataclass
class UnifiedStats:
    steps: int = 0
    tokens: int = 0
    tok_per_sec: float = 0.0
    last_loss: float = 0.0


class UnifiedEntry:
    """Error-returning wrapper of UnifiedTrainer for callers that do not want exceptions: every call gives (ok, message)."""

    def __init__(self, model, tokenizer=None):
        self.inner = UnifiedTrainer(model, tokenizer)
        self._stats = UnifiedStats()
        self._t0 = time.perf_counter()

    def configure(self, args: UnifiedTrainArgs):
        try:
            self.inner.configure(args)
            return True, ""
        except (ValueError, OSError) as e:
            return False, str(e)

    def run(self):
        try:
            self.inner.run()
            m = self.inner.metrics()
            self._stats.steps, self._stats.last_loss = m.step, m.loss
            return True, ""
        except (ValueError, OSError, RuntimeError) as e:
            return False, str(e)

    def train_step_once(self, ids, labels):
        try:
            loss = self.inner.train_step_once(ids, labels)
        except (ValueError, RuntimeError) as e:
            return False, 0.0, str(e)
        s = self._stats
        s.steps += 1
        s.tokens += ids.numel()
        s.last_loss = float(loss)
        s.tok_per_sec = s.tokens / max(1e-9, time.perf_counter() - self._t0)
        return True, float(loss), ""

    def save_checkpoint(self, path): self.inner.save_checkpoint(path)
    def load_checkpoint(self, path): self.inner.load_checkpoint(path)
    def metrics(self): return self.inner.metrics()
    def stats(self) -> UnifiedStats: return self._stats

    @staticmethod
    def kind_name(k: str) -> str: return unified_trainer_parse_kind(k) or "unknown"

    @staticmethod
    def parse_kind(s: str): return unified_trainer_parse_kind(s)


@dataclass
class RewardStats:
    mean: float = 0.0
    std: float = 1.0


def normalize_rewards(rewards: torch.Tensor) -> RewardStats:
    r = rewards.float()
    return RewardStats(float(r.mean()), max(float(r.std(unbiased=False)), 1e-6))


def policy_grad_loss(logits, labels, advantages, ignore_index: int = -100):
    """REINFORCE surrogate -(A * log pi(label)) averaged over kept rows; advantages per row.  Returns (loss, dlogits)."""
    lg, lab = _rows(logits, labels)
    adv = advantages.float().reshape(-1)
    keep = lab != ignore_index
    n = max(1, int(keep.sum()))
    lp = torch.log_softmax(lg, -1)
    lpt = lp.gather(1, lab.clamp(min=0)[:, None])[:, 0]
    loss = -(adv * lpt * keep).sum() / n
    onehot = torch.zeros_like(lp).scatter_(1, lab.clamp(min=0)[:, None], 1.0)
    d = (adv * keep / n)[:, None] * (lp.exp() - onehot)
    return float(loss), d.view(logits.shape)


@dataclass
class GroupOut:
    loss: float = 0.0
    mean_reward: float = 0.0


def grpo_step(logits, labels, rewards, group: int, clip_eps: float = 0.2, kl_coef: float = 0.01, old_logp=None, ref_logp=None):
    """Group-relative policy optimisation on sequence-level log-probabilities.  ``logits`` [N, S, V], ``labels`` [N, S],
    ``rewards`` [N] with N a multiple of ``group``; advantages are rewards standardised inside each group.  Without
    ``old_logp`` the ratio is 1 (first step of an on-policy update); ``ref_logp`` adds the k3 KL estimate."""
    N = rewards.numel()
    if N % group:
        raise ValueError("rewards do not divide into groups")
    r = rewards.float().view(-1, group)
    adv = ((r - r.mean(1, keepdim=True)) / (r.std(1, unbiased=False, keepdim=True) + 1e-6)).view(-1)
    lp = torch.log_softmax(logits.float(), -1).gather(-1, labels.clamp(min=0)[..., None])[..., 0]
    keep = (labels != -100).float()
    seq = (lp * keep).sum(-1) / keep.sum(-1).clamp(min=1)
    old = seq.detach() if old_logp is None else old_logp.float()
    ratio = (seq - old).exp()
    surr = torch.minimum(ratio * adv, ratio.clamp(1 - clip_eps, 1 + clip_eps) * adv)
    loss = -surr.mean()
    if ref_logp is not None:
        d = ref_logp.float() - seq
        loss = loss + kl_coef * (d.exp() - d - 1).mean()
    return GroupOut(float(loss), float(rewards.float().mean()))


# ----------------------------------------------------------------------------------------------- evaluation harness
class NgramScore:
    @staticmethod
    def precision(cand: Sequence[int], ref: Sequence[int], n: int) -> float:
        from collections import Counter
        c = Counter(tuple(cand[i:i + n]) for i in range(len(cand) - n + 1))
        r = Counter(tuple(ref[i:i + n]) for i in range(len(ref) - n + 1))
        tot = sum(c.values())
        return sum(min(v, r[k]) for k, v in c.items()) / tot if tot else 0.0

    @staticmethod
    def lcs_len(a: Sequence[int], b: Sequence[int]) -> int:
        prev = [0] * (len(b) + 1)
        for x in a:
            cur = [0]
            for j, y in enumerate(b):
                cur.append(prev[j] + 1 if x == y else max(prev[j + 1], cur[j]))
            prev = cur
        return prev[-1]


@dataclass
class HarnessOut:
    perplexity: object = None
    accuracy: object = None
    bleu: float = 0.0
    rouge_l: float = 0.0
    tokens: int = 0
    tok_per_sec: float = 0.0


class EvalHarness:
    def __init__(self, model, tokenizer=None):
        self.model, self.tok = model, tokenizer
        self.evaluator = MX.ModelEvaluator(model)

    def run_tokens(self, tokens: Sequence[int], name: str = "eval", context: int = 512) -> HarnessOut:
        t0 = time.perf_counter()
        out = HarnessOut(self.evaluator.evaluate_perplexity(list(tokens), name + "/ppl", context),
                         self.evaluator.evaluate_accuracy(list(tokens), name + "/acc", context), tokens=len(tokens))
        out.tok_per_sec = 2 * len(tokens) / max(1e-9, time.perf_counter() - t0)
        return out

    def run_loader(self, dl, max_batches: int = 20) -> HarnessOut:
        toks: List[int] = []
        dl.reset()
        for _ in range(min(max_batches, len(dl))):
            ids, _ = dl.next_batch()
            toks.extend(ids.reshape(-1).tolist())
        return self.run_tokens(toks, "loader", dl.S)

    def _seq_logp(self, ctx: Sequence[int], cont: Sequence[int]) -> float:
        dev = next(self.model.parameters()).device
        ids = torch.tensor([list(ctx) + list(cont)], device=dev)
        with torch.no_grad():
            lp = torch.log_softmax(self.model(ids).float(), -1)[0]
        pos = torch.arange(len(ctx) - 1, len(ctx) + len(cont) - 1, device=dev)
        return float(lp[pos, ids[0, len(ctx):]].mean())

    def hellaswag(self, contexts, good, bad):
        """Fraction of items whose true ending has the higher mean token log-probability."""
        hits = sum(self._seq_logp(c, g) > self._seq_logp(c, b) for c, g, b in zip(contexts, good, bad))
        n = len(contexts)
        return MX.EvalResult(name="hellaswag", accuracy=hits / max(1, n), correct=hits, total=n)

    def bleu(self, cand, ref, max_n: int = 4) -> float: return MX.bleu(cand, [ref], max_n)
    def rouge_l(self, cand, ref) -> float: return MX.rouge_l(cand, ref)["f1"]
