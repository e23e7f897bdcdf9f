"""Run-time telemetry: an estimated cache-level hit logger, a categorised memory tracker with footprint verification, the
ASCII expert-utilisation histogram, the age-tiered KV-cache precision policy and the training-step printer.
Reference counterparts: include/quant/telemetry.h:57-256, src/core/telemetry.cpp."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

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

    # ---- address-stream form of the reference (include/quant/telemetry.h: CacheHitLogger) -------------------------
    _instance = None

    @classmethod
    def instance(cls) -> "CacheHitLogger":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def record_access(self, addr: int, size_bytes: int):
        """One access at ``addr``: the distance from the previous access decides the level it is charged to (within a
        128-byte line: L1; within the L2 capacity: L2; else HBM) and whether the stream counts as sequential."""
        last = getattr(self, "_last_addr", None)
        dist = abs(addr - last) if last is not None else self.l2 + 1
        self._last_addr = addr + size_bytes
        self.sequential = getattr(self, "sequential", 0) + (last is not None and addr == last)
        self.random = getattr(self, "random", 0) + (last is None or addr != last)
        lvl = "L1" if dist <= 128 else ("L2" if dist <= self.l2 else "HBM")
        self.hits[lvl] += 1
        self.bytes[lvl] += size_bytes
        return lvl

    def record_sequential(self, base: int, count: int, stride: int):
        for i in range(count):
            self.record_access(base + i * stride, stride)

    def stats(self) -> dict:
        tot = sum(self.hits.values())
        return {"total_accesses": tot, "l1_hits": self.hits["L1"], "l2_hits": self.hits["L2"], "ram_fetches": self.hits["HBM"],
                "sequential_reads": int(getattr(self, "sequential", 0)), "random_reads": int(getattr(self, "random", 0)),
                "l1_hit_rate": self.hits["L1"] / max(1, tot), "l2_hit_rate": self.hits["L2"] / max(1, tot),
                "ram_rate": self.hits["HBM"] / max(1, tot)}

    def print_report(self, file=None) -> str:
        st = self.stats()
        text = (f"cache (estimated): {st['total_accesses']} accesses | L1 {100 * st['l1_hit_rate']:.1f}% | L2 {100 * st['l2_hit_rate']:.1f}% | "
                f"HBM {100 * st['ram_rate']:.1f}% | sequential {st['sequential_reads']} / random {st['random_reads']}")
        print(text, file=file)
        return text

    def reset(self):
        self.hits = {k: 0 for k in self.hits}
        self.bytes = {k: 0 for k in self.bytes}
        self.sequential = self.random = 0
        self._last_addr = None


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

    # ---- named tracking of the reference (include/quant/telemetry.h: MemoryTracker) -----------------------------------
    _instance = None

    @classmethod
    def instance(cls) -> "MemoryTracker":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def _named(self, category: str, name: str, nbytes: int):
        """Entries are keyed by name: tracking a name again replaces its earlier figure."""
        items = self.__dict__.setdefault("items", {})
        old = items.get((category, name), 0)
        items[(category, name)] = int(nbytes)
        self.bytes[category] += int(nbytes) - old
        self.peak = max(self.peak, self.total())

    def track_weights(self, name: str, nbytes: int): self._named("weights", name, nbytes)
    def track_gradients(self, name: str, nbytes: int): self._named("gradients", name, nbytes)
    def track_optimizer(self, name: str, m_bytes: int, v_bytes: int): self._named("optimizer", name, int(m_bytes) + int(v_bytes))
    def track_activations(self, name: str, nbytes: int): self._named("activations", name, nbytes)
    def track_kv_cache(self, nbytes: int): self._named("kv_cache", "kv", nbytes)
    def track_offload(self, name: str, nbytes: int): self._named("offload", name, nbytes)

    def update(self):
        """Refresh the peak (and, on a GPU, remember what the allocator reports for ``verify_footprint``)."""
        self.peak = max(self.peak, self.total())
        if torch.cuda.is_available():
            self.measured = torch.cuda.memory_allocated()
        return self.total()

    def breakdown(self) -> dict:
        b = self.bytes
        dev = self.total()
        return {"weights_bytes": b["weights"], "gradients_bytes": b["gradients"], "optimizer_bytes": b["optimizer"],
                "activations_bytes": b["activations"], "kv_cache_bytes": b["kv_cache"], "cpu_offloaded_bytes": b["offload"],
                "total_device_bytes": dev, "total_bytes": dev + b["offload"]}

    def bpw(self, model_params: int) -> float:
        """Achieved bits per weight of the stored weights."""
        return 8.0 * self.bytes["weights"] / max(1, model_params)

    def verify_bpw(self, model_params: int, target_bpw: float, tolerance: float = 0.1) -> bool:
        return abs(self.bpw(model_params) - target_bpw) <= tolerance * target_bpw

    def print_report(self, model_params: int = 0, target_bpw: float = 0.0, file=None) -> str:
        bd = self.breakdown()
        lines = ["memory:"] + [f"  {k:<22}{v / 2**20:12.2f} MiB" for k, v in bd.items()]
        if model_params:
            lines.append(f"  bits per weight       {self.bpw(model_params):12.3f}" + (f" (target {target_bpw:g})" if target_bpw else ""))
        text = "\n".join(lines)
        print(text, file=file)
        return text

    def reset(self):
        self.bytes = {c: 0 for c in self.CATEGORIES}
        self.items, self.peak = {}, 0


class RoutingHistogram:
    def __init__(self, num_experts):
        self.counts = [0] * num_experts

    def record(self, expert_indices, num_tokens=None, top_k=None):
        for e in torch.as_tensor(expert_indices).reshape(-1).tolist():
            self.counts[e] += 1

    def record_with_modalities(self, expert_indices, modality_names, num_tokens=None, top_k=None):
        """``modality_names[t]``: the modality of token t; per expert the modality it served most is reported."""
        idx = torch.as_tensor(expert_indices)
        idx = idx.reshape(len(modality_names), -1) if idx.dim() == 1 else idx
        per = self.__dict__.setdefault("modalities", [dict() for _ in self.counts])
        for t, name in enumerate(modality_names):
            for e in idx[t].tolist():
                self.counts[e] += 1
                per[e][name] = per[e].get(name, 0) + 1

    def entries(self) -> List[dict]:
        tot = max(1, sum(self.counts))
        per = getattr(self, "modalities", None)
        return [{"expert_id": i, "tokens_routed": c, "utilization": c / tot,
                 "modality_name": (max(per[i], key=per[i].get) if per and per[i] else "")} for i, c in enumerate(self.counts)]

    def print(self, file=None) -> str:
        text = self.render()
        print(text, file=file)
        return text

    def print_with_loss(self, load_balance_loss: float, file=None) -> str:
        text = self.render() + f"\nload-balance loss: {load_balance_loss:.6f} | balanced: {self.is_balanced()}"
        print(text, file=file)
        return text

    def reset(self):
        self.counts = [0] * len(self.counts)
        self.modalities = [dict() for _ in self.counts]

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

    # ---- in-place ageing of a cache (reference: KVCacheQuantizer, include/quant/telemetry.h) ----------------------
    def config(self) -> dict:
        return {"full_precision_window": self.recent, "quant4_window": self.middle, "enabled": True}

    def quantize_old_states(self, k_cache: torch.Tensor, v_cache: torch.Tensor, current_seq_len: int) -> int:
        """Round the positions of [seq, ...] caches that have left the full-precision window to their tier's values, in
        place; returns the bytes a packed store of those positions saves against ``k_cache``'s dtype."""
        plan = self.plan(current_seq_len)
        saved = 0
        per_tok = k_cache[0].numel() * k_cache.element_size() if k_cache.shape[0] else 0
        done = self.__dict__.setdefault("_aged", {"q4": 0, "ternary": 0})
        for tier, cost in (("ternary", (0.25 + 2.0 / 128) / 2.0), ("q4", (0.5 + 2.0 / 32) / 2.0)):
            lo, hi = plan[tier]
            if hi > lo:
                for c in (k_cache, v_cache):
                    c[lo:hi] = self.quantize(c[lo:hi], tier)
                saved += int(2 * (hi - lo) * per_tok * (1.0 - cost * 2.0 / k_cache.element_size()))
            done[tier] = hi - lo
        self._bytes_saved = saved
        self._bytes_full = 2 * current_seq_len * per_tok
        return saved

    def restore_for_attention(self, quantized: torch.Tensor, start: int, end: int, out: Optional[torch.Tensor] = None):
        """The cache rows [start, end) in compute precision (aged rows already hold their rounded values)."""
        rows = quantized[start:end].float()
        if out is not None:
            out.copy_(rows)
            return out
        return rows

    def bytes_saved(self) -> int: return int(getattr(self, "_bytes_saved", 0))

    def compression_ratio(self) -> float:
        full = getattr(self, "_bytes_full", 0)
        return full / max(1, full - self.bytes_saved()) if full else 1.0

    def estimated_quality_loss(self) -> float:
        """Rough relative error of the attention output: the aged fraction of the cache times its tier's rounding error
        (4-bit groups about 4 %, ternary about 30 % of a value's magnitude), discounted because old tokens get little
        attention mass."""
        aged = getattr(self, "_aged", {"q4": 0, "ternary": 0})
        tot = max(1, getattr(self, "_bytes_full", 0) and (aged["q4"] + aged["ternary"] + self.recent))
        return 0.1 * (0.04 * aged["q4"] + 0.3 * aged["ternary"]) / tot

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
    """Report printers over the process-wide trackers (reference: TelemetryPrinter, include/quant/telemetry.h)."""
    routing: "RoutingHistogram" = None         # set by the trainer that wants its routing printed
    kv: "KVCacheQuantizer" = None

    @staticmethod
    def print_all_header(file=None):
        print("=" * 30 + " telemetry " + "=" * 30, file=file)

    @staticmethod
    def print_all_footer(file=None):
        print("=" * 71, file=file)

    @staticmethod
    def print_cache_report(file=None):
        return CacheHitLogger.instance().print_report(file)

    @staticmethod
    def print_memory_report(model_params: int = 0, target_bpw: float = 0.0, file=None):
        return MemoryTracker.instance().print_report(model_params, target_bpw, file)

    @classmethod
    def print_routing_report(cls, load_balance_loss: float = 0.0, file=None):
        if cls.routing is None:
            print("routing: no histogram registered", file=file)
            return ""
        return cls.routing.print_with_loss(load_balance_loss, file)

    @classmethod
    def print_kv_quant_report(cls, file=None):
        if cls.kv is None:
            print("kv cache: no quantizer registered", file=file)
            return ""
        text = (f"kv cache: saved {cls.kv.bytes_saved() / 2**20:.2f} MiB | ratio {cls.kv.compression_ratio():.2f}x | "
                f"estimated quality loss {100 * cls.kv.estimated_quality_loss():.3f}%")
        print(text, file=file)
        return text

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
