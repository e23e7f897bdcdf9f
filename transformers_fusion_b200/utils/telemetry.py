"""Run-time telemetry: an estimated cache-level hit logger, a categorised memory tracker with footprint verification, the
ASCII expert-utilisation histogram, the age-tiered KV-cache precision policy and the training-step printer.
Reference counterparts: include/quant/telemetry.h:57-256, src/core/telemetry.cpp."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

import torch


class CacheHitLogger:
    """Classifies accesses by working-set size against cache capacities (an estimate, not a hardware counter)."""

    def __init__(self, l1_bytes=256 << 10, l2_bytes=126 << 20):
        self.l1, self.l2 = l1_bytes, l2_bytes
        self.hits = {"L1": 0, "L2": 0, "HBM": 0}
        self.bytes = {"L1": 0, "L2": 0, "HBM": 0}

    def log_access(self, working_set_bytes, nbytes=None):
        lvl = "L1" if working_set_bytes <= self.l1 else ("L2" if working_set_bytes <= self.l2 else "HBM")
        self.hits[lvl] += 1
        self.bytes[lvl] += nbytes if nbytes is not None else working_set_bytes
        return lvl

    def report(self):
        tot = max(1, sum(self.hits.values()))
        return {k: v / tot for k, v in self.hits.items()}


class MemoryTracker:
    CATEGORIES = ("weights", "gradients", "optimizer", "activations", "kv_cache", "offload")

    def __init__(self):
        self.bytes: Dict[str, int] = {c: 0 for c in self.CATEGORIES}
        self.peak = 0

    def add(self, category, nbytes):
        self.bytes[category] += int(nbytes)
        self.peak = max(self.peak, self.total())

    def sub(self, category, nbytes):
        self.bytes[category] = max(0, self.bytes[category] - int(nbytes))

    def total(self):
        return sum(v for k, v in self.bytes.items() if k != "offload")

    def verify_footprint(self, measured_bytes, tolerance=0.15) -> bool:
        """True when the accounted device bytes explain the measured ones within ``tolerance``."""
        t = self.total()
        return abs(measured_bytes - t) <= tolerance * max(measured_bytes, t, 1)

    def track_model(self, model, optimizer_bytes_per_param=12):
        n = sum(p.numel() for p in model.parameters())
        es = next(model.parameters()).element_size()
        self.add("weights", n * es)
        self.add("gradients", n * 4)
        self.add("optimizer", n * optimizer_bytes_per_param)

    def report(self):
        return {**self.bytes, "total": self.total(), "peak": self.peak}


class RoutingHistogram:
    def __init__(self, num_experts):
        self.counts = [0] * num_experts

    def record(self, expert_indices):
        for e in torch.as_tensor(expert_indices).reshape(-1).tolist():
            self.counts[e] += 1

    def is_balanced(self, tolerance=0.5):
        tot = sum(self.counts)
        if tot == 0:
            return True
        mean = tot / len(self.counts)
        return all(abs(c - mean) <= tolerance * mean for c in self.counts)

    def render(self, width=40):
        mx = max(self.counts + [1])
        return "\n".join(f"expert {i:3d} | {'#' * int(round(width * c / mx)):<{width}} | {c}" for i, c in enumerate(self.counts))


class KVCacheQuantizer:
    """Precision by token age: the most recent ``recent`` tokens stay in full precision, the next ``middle`` in 4 bits,
    everything older in ternary."""

    def __init__(self, recent=4096, middle=32768):
        self.recent, self.middle = recent, middle

    def tier(self, age: int) -> str:
        return "fp" if age < self.recent else ("q4" if age < self.recent + self.middle else "ternary")

    def plan(self, seq_len: int):
        """{tier: (start, end)} token ranges of a sequence (positions; the newest token has position seq_len - 1)."""
        a = max(0, seq_len - self.recent)
        b = max(0, a - self.middle)
        return {"ternary": (0, b), "q4": (b, a), "fp": (a, seq_len)}

    def bytes_per_token(self, seq_len, head_bytes_fp=2.0):
        p = self.plan(seq_len)
        w = {"fp": head_bytes_fp, "q4": 0.5 + 2.0 / 32, "ternary": 0.25 + 2.0 / 128}
        return sum((hi - lo) * w[t] for t, (lo, hi) in p.items()) / max(1, seq_len)

    @staticmethod
    def quantize(x: torch.Tensor, tier: str):
        """Round-trip ``x`` through the tier's format (rows of the last dimension; 32-element groups)."""
        if tier == "fp":
            return x
        f = x.float()
        g = f.reshape(-1, 32) if f.shape[-1] % 32 == 0 else f.reshape(-1, f.shape[-1])
        if tier == "q4":
            s = g.abs().amax(1, keepdim=True).clamp(min=1e-30) / 7.0
            q = torch.clamp(torch.round(g / s), -8, 7) * s
        else:
            s = g.abs().mean(1, keepdim=True).clamp(min=1e-30)
            q = torch.where(g > 0.5 * s, s, torch.where(g < -0.5 * s, -s, torch.zeros_like(g)))
        return q.reshape(x.shape).to(x.dtype)


class TelemetryPrinter:
    @staticmethod
    def print_training_step(step, loss, lr, tokens_per_sec, grad_norm=None, mem: MemoryTracker = None, file=None):
        import math
        line = f"Step {step} | loss: {loss:.6g} | ppl: {math.exp(min(loss, 30.0)):.6g} | lr: {lr:.6g} | tok/s: {tokens_per_sec:.6g}"
        if grad_norm is not None:
            line += f" | gnorm: {grad_norm:.4g}"
        if mem is not None:
            line += f" | mem: {mem.total() / 2 ** 30:.2f} GiB"
        print(line, file=file, flush=True)
        return line
