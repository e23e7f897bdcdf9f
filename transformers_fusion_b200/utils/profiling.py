"""Timing and memory instrumentation: NVTX ranges (no-ops without CUDA), device-side timers built on CUDA events with
the max over ranks, a memory tracker, and the micro-benchmark hook.

Reference counterparts: KernelPerf / profile_gemv_* (include/quant/kernel_production.h), MemoryTracker
(include/quant/telemetry.h:103-149), benchmark_operation (src/backend/backend.cpp:2997-3099), pipeline ns counters."""
from __future__ import annotations

import contextlib
import statistics
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """``with timer("phase"):`` accumulates device time per phase (CUDA events on the current stream; host clock on CPU)."""

    def __init__(self):
        self.ms: Dict[str, List[float]] = {}
        self._pending = []

    @contextlib.contextmanager
    def __call__(self, name):
        if torch.cuda.is_available():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            with nvtx_range(name):
                yield
            e1.record()
            self._pending.append((name, e0, e1))
        else:
            t0 = time.perf_counter()
            yield
            self.ms.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)

    def collect(self):
        if self._pending:
            torch.cuda.synchronize()
            for name, e0, e1 in self._pending:
                self.ms.setdefault(name, []).append(e0.elapsed_time(e1))
            self._pending = []
        return self.ms

    def summary(self, reduce_max_over_ranks=False):
        out = {}
        for k, v in self.collect().items():
            tot = sum(v)
            if reduce_max_over_ranks and torch.distributed.is_available() and torch.distributed.is_initialized():
                t = torch.tensor([tot], device="cuda" if torch.cuda.is_available() else "cpu")
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
                tot = float(t)
            out[k] = {"total_ms": tot, "calls": len(v), "mean_ms": tot / max(1, len(v))}
        return out


@dataclass
class KernelPerf:
    name: str = ""
    ms: float = 0.0
    bytes: int = 0
    flops: float = 0.0

    @property
    def gbs(self):
        return self.bytes / max(self.ms, 1e-9) / 1e6

    @property
    def gflops(self):
        return self.flops / max(self.ms, 1e-9) / 1e6


def benchmark_operation(fn: Callable, iters=20, warmup=3, nbytes=0, flops=0.0, name="op") -> KernelPerf:
    """Best-of-``iters`` time of ``fn`` (device-timed on CUDA, an L2-sized write between iterations)."""
    if torch.cuda.is_available():
        from ..cli.bench import time_kernel
        ms = min(time_kernel(fn, iters, warmup))
    else:
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e3)
        ms = min(ts)
    return KernelPerf(name, ms, nbytes, flops)


class MemoryTracker:
    """Named allocations with current / peak totals (host-side accounting; ``device_stats`` adds the allocator's view)."""

    def __init__(self):
        self.live: Dict[str, int] = {}
        self.current = self.peak = 0

    def alloc(self, name, nbytes):
        self.live[name] = self.live.get(name, 0) + int(nbytes)
        self.current += int(nbytes)
        self.peak = max(self.peak, self.current)

    def free(self, name):
        self.current -= self.live.pop(name, 0)

    def track_tensor(self, name, t):
        self.alloc(name, t.numel() * t.element_size())

    def report(self):
        return {"current": self.current, "peak": self.peak, "live": dict(sorted(self.live.items(), key=lambda kv: -kv[1]))}

    @staticmethod
    def device_stats(device=None):
        if not torch.cuda.is_available():
            return {}
        return {"allocated": torch.cuda.memory_allocated(device), "reserved": torch.cuda.memory_reserved(device),
                "peak_allocated": torch.cuda.max_memory_allocated(device)}
