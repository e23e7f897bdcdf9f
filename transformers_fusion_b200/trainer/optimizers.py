"""The optimizer family over flat fp32 master weights.

Fifteen update rules with the reference's names (include/quant/optimizer.h, src/trainer/optimizer.cpp):
SGD, Adam, AdamW, Adamax, NAdam, RAdam, Lion, Adafactor, RMSProp, Ranger, Adabound, Lamb, LARS,
NovoGrad (+ Adagrad).  AdamW / Lion / SGD on CUDA go through the fused kernels (``FlatAdamW`` is the
production path); the others are expressed with torch ops on the same flat buffers so every one of
them works with ZeRO sharding, bf16 compute copies and gradient clipping.

Every optimizer: ``step(lr=None)`` -> clip (global L2) -> update fp32 master -> refresh the model's
compute-dtype parameters -> zero the gradients.  Adafactor is the reference CLI's default
(tools/train.cpp ``--optimizer adafactor|adamw``) with a factored second moment for matrices.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


class FlatOptimizer:
    name = "base"
    per_tensor = False

    def __init__(self, flat, lr=1e-3, weight_decay=0.0, max_grad_norm=0.0, shard=None, **hyper):
        self.flat, self.lr, self.wd, self.max_grad_norm = flat, lr, weight_decay, max_grad_norm
        self.lo, self.hi = shard if shard is not None else (0, flat.numel)
        self.h = hyper
        self.step_count = 0
        self.master = flat.params[self.lo:self.hi].float().clone()
        self.state = {}
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=flat.params.device)
        self.norm_reduce = None

    # ---- helpers
    def _buf(self, key, like=None, fill=0.0):
        if key not in self.state:
            ref = self.master if like is None else like
            self.state[key] = torch.full_like(ref, fill)
        return self.state[key]

    def _tensors(self):
        """(name, master view, grad view) for every parameter that lies inside this shard."""
        out = []
        for i, (p, off) in enumerate(zip(self.flat.params_list, self.flat.offsets)):
            a, b = max(off, self.lo), min(off + p.numel(), self.hi)
            if a >= b:
                continue
            whole = a == off and b == off + p.numel()
            shape = p.shape if whole else (b - a,)
            out.append((i, self.master[a - self.lo:b - self.lo].view(shape), self.flat.grads[a:b].view(shape)))
        return out

    def clip(self):
        g = self.flat.grads[self.lo:self.hi]
        ss = (g * g).sum().reshape(1)
        if self.norm_reduce is not None:
            self.norm_reduce(ss)
        self.grad_norm = ss.sqrt()
        if self.max_grad_norm > 0:
            g.mul_(torch.clamp(self.max_grad_norm / (self.grad_norm + 1e-6), max=1.0))

    def step(self, lr: Optional[float] = None):
        self.step_count += 1
        lr = self.lr if lr is None else lr
        self.clip()
        if self.per_tensor:
            for i, p, g in self._tensors():
                self.update(p, g, lr, i)
        else:
            self.update(self.master, self.flat.grads[self.lo:self.hi], lr, -1)
        self.flat.params[self.lo:self.hi].copy_(self.master.to(self.flat.params.dtype))
        self.flat.grads[self.lo:self.hi].zero_()

    def update(self, p, g, lr, idx):
        raise NotImplementedError

    def zero_grad(self):
        self.flat.grads.zero_()

    def reset(self):
        """Forget the optimizer state (moments, step count, a built-in schedule's position); the weights stay as they are."""
        self.state.clear()
        self.step_count = 0
        self.master.copy_(self.flat.params[self.lo:self.hi].float())
        if hasattr(self, "current_lr"):
            self.current_lr = None

    def get_lr(self) -> float: return self.lr
    def set_lr(self, lr: float): self.lr = float(lr)

    def state_dict(self):
        return {"step": self.step_count, "lr": self.lr, "master": self.master, "state": self.state}

    def load_state_dict(self, sd):
        self.step_count, self.lr = int(sd["step"]), float(sd["lr"])
        self.master.copy_(sd["master"])
        self.state = sd["state"]
        self.flat.params[self.lo:self.hi].copy_(self.master.to(self.flat.params.dtype))


class SGD(FlatOptimizer):
    name = "sgd"

    def update(self, p, g, lr, idx):
        mu = self.h.get("momentum", 0.9)
        g = g + self.wd * p
        if mu > 0:
            m = self._buf("m")
            m.mul_(mu).add_(g)
            g = g + mu * m if self.h.get("nesterov", False) else m
        p.add_(g, alpha=-lr)


class Adam(FlatOptimizer):
    name = "adam"
    decoupled = False

    def update(self, p, g, lr, idx):
        b1, b2 = self.h.get("betas", (0.9, 0.999))
        eps = self.h.get("eps", 1e-8)
        if not self.decoupled and self.wd:
            g = g + self.wd * p
        m, v = self._buf("m"), self._buf("v")
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = m / (1 - b1 ** self.step_count)
        vh = v / (1 - b2 ** self.step_count)
        upd = mh / (vh.sqrt() + eps)
        if self.decoupled and self.wd:
            upd = upd + self.wd * p
        p.add_(upd, alpha=-lr)


class AdamW(Adam):
    """Decoupled weight decay.  It can carry its own learning-rate schedule (reference: AdamW::set_schedule /
    scheduler_step, include/quant/optimizer.h:60-63, src/trainer/optimizer.cpp:54-90): after ``scheduler_step(s)`` the next
    ``step()`` without an explicit rate uses the scheduled one."""
    name = "adamw"
    decoupled = True
    SCHEDULES = ("constant", "cosine", "linear", "warmup_cosine", "cosine_restart")
    current_lr = None

    def set_schedule(self, schedule: str, warmup_steps: int = 0, total_steps: int = 0, restart_period: int = 0):
        schedule = schedule.lower()
        if schedule not in self.SCHEDULES:
            raise ValueError(f"unknown schedule {schedule!r}; one of {self.SCHEDULES}")
        self._sched = (schedule, int(warmup_steps), int(total_steps), int(restart_period))

    def adjusted_lr(self, step: int) -> float:
        kind, warm, total, period = getattr(self, "_sched", ("constant", 0, 0, 0))
        if total <= 0 or kind == "constant":
            return self.lr
        ratio = min(1.0, step / total)
        if kind == "cosine":
            return self.lr * 0.5 * (1.0 + math.cos(math.pi * ratio))
        if kind == "linear":
            return self.lr * (1.0 - ratio)
        if kind == "warmup_cosine":
            if step < warm:
                return self.lr * step / warm
            r = min(1.0, (step - warm) / max(1, total - warm))
            return self.lr * 0.5 * (1.0 + math.cos(math.pi * r))
        p = period if period > 0 else max(1, total // 4)            # cosine with restarts; every cycle starts at half the last peak
        return self.lr * 0.5 ** (step // p) * 0.5 * (1.0 + math.cos(math.pi * (step % p) / p))

    def scheduler_step(self, step: int) -> float:
        self.current_lr = self.adjusted_lr(step)
        return self.current_lr

    def step(self, lr: Optional[float] = None):
        super().step(self.current_lr if lr is None and self.current_lr is not None else lr)


class Adamax(FlatOptimizer):
    name = "adamax"

    def update(self, p, g, lr, idx):
        b1, b2 = self.h.get("betas", (0.9, 0.999))
        m, u = self._buf("m"), self._buf("u")
        g = g + self.wd * p
        m.mul_(b1).add_(g, alpha=1 - b1)
        torch.maximum(u * b2, g.abs(), out=u)
        p.add_(m / (u + self.h.get("eps", 1e-8)), alpha=-lr / (1 - b1 ** self.step_count))


class NAdam(FlatOptimizer):
    name = "nadam"

    def update(self, p, g, lr, idx):
        b1, b2 = self.h.get("betas", (0.9, 0.999))
        eps, t = self.h.get("eps", 1e-8), self.step_count
        g = g + self.wd * p
        m, v = self._buf("m"), self._buf("v")
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = b1 * m / (1 - b1 ** (t + 1)) + (1 - b1) * g / (1 - b1 ** t)
        p.add_(mh / ((v / (1 - b2 ** t)).sqrt() + eps), alpha=-lr)


class RAdam(FlatOptimizer):
    name = "radam"

    def _radam(self, p, g, lr):
        b1, b2 = self.h.get("betas", (0.9, 0.999))
        eps, t = self.h.get("eps", 1e-8), self.step_count
        m, v = self._buf("m", p), self._buf("v", p)
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = m / (1 - b1 ** t)
        rho_inf = 2 / (1 - b2) - 1
        rho = rho_inf - 2 * t * b2 ** t / (1 - b2 ** t)
        if rho > 5:
            r = math.sqrt((rho - 4) * (rho - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho))
            p.add_(mh * r / ((v / (1 - b2 ** t)).sqrt() + eps), alpha=-lr)
        else:
            p.add_(mh, alpha=-lr)

    def update(self, p, g, lr, idx):
        if self.wd:
            p.mul_(1 - lr * self.wd)
        self._radam(p, g, lr)


class Ranger(RAdam):
    """RAdam + lookahead (slow weights pulled toward fast weights every k steps)."""
    name = "ranger"

    def update(self, p, g, lr, idx):
        super().update(p, g, lr, idx)
        k, alpha = self.h.get("k", 6), self.h.get("alpha", 0.5)
        slow = self.state.setdefault("slow", p.clone())
        if self.step_count % k == 0:
            slow.add_(p - slow, alpha=alpha)
            p.copy_(slow)


class Lion(FlatOptimizer):
    name = "lion"

    def update(self, p, g, lr, idx):
        b1, b2 = self.h.get("betas", (0.9, 0.99))
        m = self._buf("m")
        u = (b1 * m + (1 - b1) * g).sign()
        p.add_(u + self.wd * p, alpha=-lr)
        m.mul_(b2).add_(g, alpha=1 - b2)


class RMSProp(FlatOptimizer):
    name = "rmsprop"

    def update(self, p, g, lr, idx):
        a, eps = self.h.get("alpha", 0.99), self.h.get("eps", 1e-8)
        g = g + self.wd * p
        v = self._buf("v")
        v.mul_(a).addcmul_(g, g, value=1 - a)
        p.addcdiv_(g, v.sqrt() + eps, value=-lr)


class Adagrad(FlatOptimizer):
    name = "adagrad"

    def update(self, p, g, lr, idx):
        g = g + self.wd * p
        v = self._buf("v")
        v.addcmul_(g, g)
        p.addcdiv_(g, v.sqrt() + self.h.get("eps", 1e-10), value=-lr)


class Adabound(FlatOptimizer):
    name = "adabound"

    def update(self, p, g, lr, idx):
        b1, b2 = self.h.get("betas", (0.9, 0.999))
        final_lr, gamma, eps, t = self.h.get("final_lr", 0.1), self.h.get("gamma", 1e-3), self.h.get("eps", 1e-8), self.step_count
        g = g + self.wd * p
        m, v = self._buf("m"), self._buf("v")
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        step = lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        lo, hi = final_lr * (1 - 1 / (gamma * t + 1)), final_lr * (1 + 1 / (gamma * t))
        p.sub_((step / (v.sqrt() + eps)).clamp_(lo, hi) * m)


class Lamb(FlatOptimizer):
    name = "lamb"
    per_tensor = True

    def update(self, p, g, lr, idx):
        b1, b2 = self.h.get("betas", (0.9, 0.999))
        eps, t = self.h.get("eps", 1e-6), self.step_count
        m, v = self._buf(f"m{idx}", p), self._buf(f"v{idx}", p)
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        r = (m / (1 - b1 ** t)) / ((v / (1 - b2 ** t)).sqrt() + eps) + self.wd * p
        wn, rn = p.norm(), r.norm()
        trust = torch.where((wn > 0) & (rn > 0), wn / rn, torch.ones_like(wn))
        p.add_(r * trust, alpha=-lr)


class LARS(FlatOptimizer):
    name = "lars"
    per_tensor = True

    def update(self, p, g, lr, idx):
        mu, eta = self.h.get("momentum", 0.9), self.h.get("trust_coefficient", 1e-3)
        wn, gn = p.norm(), g.norm()
        local = torch.where((wn > 0) & (gn > 0), eta * wn / (gn + self.wd * wn + 1e-12), torch.ones_like(wn))
        m = self._buf(f"m{idx}", p)
        m.mul_(mu).add_((g + self.wd * p) * local)
        p.add_(m, alpha=-lr)


class NovoGrad(FlatOptimizer):
    name = "novograd"
    per_tensor = True

    def update(self, p, g, lr, idx):
        b1, b2 = self.h.get("betas", (0.95, 0.98))
        eps = self.h.get("eps", 1e-8)
        gn2 = (g * g).sum()
        v = self.state.get(f"v{idx}")
        v = gn2.clone() if v is None else v * b2 + (1 - b2) * gn2
        self.state[f"v{idx}"] = v
        m = self._buf(f"m{idx}", p)
        m.mul_(b1).add_(g / (v.sqrt() + eps) + self.wd * p)
        p.add_(m, alpha=-lr)


class Adafactor(FlatOptimizer):
    """Factored second moments for matrices (row / column statistics), full for vectors; relative-step
    free variant with update clipping (reference Adafactor::step, src/trainer/optimizer.cpp:338).

    On CUDA the whole step is the multi-tensor kernel set of csrc/kernels/adafactor.cu (five launches for all tensors);
    the per-tensor PyTorch statement below is the CPU path and the oracle of its test."""
    name = "adafactor"
    per_tensor = True

    def _fused_tables(self):
        """Device table of (offset, r offset, c offset, d0, d1, first row, decay scale) per tensor plus the flat r / c /
        scratch buffers; None when this optimizer's shard cuts through a tensor (sharded runs keep the PyTorch path)."""
        if getattr(self, "_af", None) is not None:
            return self._af
        import ctypes as C
        import numpy as np
        rows, r_off, c_off, recs, max_d1 = 0, 0, 0, [], 1
        for i, (p, off) in enumerate(zip(self.flat.params_list, self.flat.offsets)):
            if off < self.lo or off + p.numel() > self.hi:
                return None
            d0, d1 = (p.numel() // p.shape[-1], p.shape[-1]) if p.dim() >= 2 else (1, p.numel())
            recs.append((off - self.lo, r_off, c_off, d0, d1, rows, 1.0))
            rows, r_off, c_off, max_d1 = rows + d0, r_off + d0, c_off + d1, max(max_d1, d1)
        dt = np.dtype([("off", "<i8"), ("r_off", "<i8"), ("c_off", "<i8"), ("d0", "<i4"), ("d1", "<i4"), ("row0", "<i4"), ("wd", "<f4")])
        tab = np.array(recs, dtype=dt)
        dev = self.master.device
        f32 = dict(dtype=torch.float32, device=dev)
        self._af = {"table": torch.from_numpy(tab.view(np.uint8).copy()).to(dev), "nt": len(recs), "rows": rows, "max_d1": max_d1,
                    "r": torch.zeros(r_off, **f32), "c": torch.zeros(c_off, **f32), "csum": torch.zeros(c_off, **f32),
                    "rmean": torch.zeros(len(recs), **f32), "usq": torch.zeros(len(recs), **f32),
                    "m": torch.zeros_like(self.master) if self.h.get("beta1", 0.0) > 0 else None}
        from ..ops import _lib
        fn = _lib.lib().tfb_adafactor
        c_p, c_i, c_f = C.c_void_p, C.c_int, C.c_float
        fn.argtypes = [c_p, c_i, c_i, c_i] + [c_p] * 10 + [c_f] * 6 + [c_p]
        fn.restype = c_i
        return self._af

    def step(self, lr=None):
        af = self._fused_tables() if self.master.is_cuda and self.lo == 0 and self.hi == self.flat.numel else None
        if af is None:
            return super().step(lr)
        from ..ops import _lib
        self.step_count += 1
        lr = self.lr if lr is None else lr
        self.clip()
        b2 = min(0.999, 1.0 - self.step_count ** -0.8)
        g = self.flat.grads[self.lo:self.hi]
        lp = self.flat.params[self.lo:self.hi]
        _lib.check(_lib.lib().tfb_adafactor(af["table"].data_ptr(), af["nt"], af["rows"], af["max_d1"], g.data_ptr(),
                                            self.master.data_ptr(), lp.data_ptr() if lp.dtype == torch.bfloat16 else None,
                                            _lib.ptr(af["m"]), af["r"].data_ptr(), af["c"].data_ptr(), af["csum"].data_ptr(),
                                            af["rmean"].data_ptr(), af["usq"].data_ptr(), None, b2, self.h.get("eps", 1e-30),
                                            self.h.get("clip_threshold", 1.0), lr, self.wd, self.h.get("beta1", 0.0),
                                            _lib.stream()), "adafactor", 5)
        if lp.dtype != torch.bfloat16:
            lp.copy_(self.master.to(lp.dtype))

    def update(self, p, g, lr, idx):
        b2 = min(0.999, 1.0 - self.step_count ** -0.8)
        eps1, clip_thr = self.h.get("eps", 1e-30), self.h.get("clip_threshold", 1.0)
        g2 = g * g + eps1
        if p.dim() >= 2:
            r = self.state.get(f"r{idx}")
            c = self.state.get(f"c{idx}")
            if r is None:
                r, c = torch.zeros(p.shape[:-1], device=p.device), torch.zeros(p.shape[:-2] + p.shape[-1:], device=p.device)
            r = r * b2 + (1 - b2) * g2.mean(-1)
            c = c * b2 + (1 - b2) * g2.mean(-2)
            self.state[f"r{idx}"], self.state[f"c{idx}"] = r, c
            v = (r / r.mean(-1, keepdim=True)).unsqueeze(-1) * c.unsqueeze(-2)
        else:
            v = self.state.get(f"v{idx}")
            v = g2.clone() if v is None else v * b2 + (1 - b2) * g2
            self.state[f"v{idx}"] = v
        u = g / v.sqrt()
        u = u / torch.clamp(u.pow(2).mean().sqrt() / clip_thr, min=1.0)
        b1 = self.h.get("beta1", 0.0)
        if b1 > 0:
            m = self._buf(f"m{idx}", p)
            m.mul_(b1).add_(u, alpha=1 - b1)
            u = m
        if self.wd:
            p.mul_(1 - lr * self.wd)
        p.add_(u, alpha=-lr)


OPTIMIZERS = {c.name: c for c in (SGD, Adam, AdamW, Adamax, NAdam, RAdam, Ranger, Lion, RMSProp, Adagrad, Adabound, Lamb,
                                  LARS, NovoGrad, Adafactor)}


def build_optimizer(name: str, flat, **kw) -> FlatOptimizer:
    name = name.lower()
    if name not in OPTIMIZERS:
        raise ValueError(f"unknown optimizer '{name}' (known: {', '.join(sorted(OPTIMIZERS))})")
    return OPTIMIZERS[name](flat, **kw)
