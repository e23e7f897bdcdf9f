"""Inferno: a bit-width-aware throughput figure, an operation counter and a priority task queue.

``inferno_metric(flops, bpw)`` = FLOPS x (32 / bpw) / 2 / 1e21: arithmetic on b-bit weights is credited as 32 / b times the
same arithmetic on 32-bit weights.  ``InfernoCounter`` accumulates operations between ``start`` / ``stop`` on a monotonic
nanosecond clock (the reference reads the time-stamp counter) and reports the metric.  ``TaskQueue`` runs callables by
priority on worker threads.  Reference counterparts: include/quant/inferno.h:23-140, inferno/*."""
from __future__ import annotations

import heapq
import itertools
import threading
import time
from dataclasses import dataclass


def inferno_metric(flops_per_sec: float, bits_per_weight: float) -> float:
    return flops_per_sec * (32.0 / max(bits_per_weight, 1e-9)) / 2.0 / 1e21


@dataclass
class InfernoFormat:
    name: str
    bits_per_weight: float

    def multiplier(self):
        return 32.0 / self.bits_per_weight


class InfernoCounter:
    def __init__(self, bits_per_weight=32.0):
        self.bpw, self.ops, self.ns, self._t0 = bits_per_weight, 0, 0, None

    def start(self):
        self._t0 = time.perf_counter_ns()

    def add_ops(self, n):
        self.ops += int(n)

    def add_gemm(self, M, N, K):
        self.ops += 2 * M * N * K

    def stop(self):
        if self._t0 is not None:
            self.ns += time.perf_counter_ns() - self._t0
            self._t0 = None

    def flops(self):
        return self.ops / max(self.ns, 1) * 1e9

    def inferno(self):
        return inferno_metric(self.flops(), self.bpw)

    def reset(self):
        self.ops = self.ns = 0
        self.info_ops = self.elements = 0.0

    # ---- per-format recording (reference: InfernoCounter, include/quant/inferno.h:123-205): every recorded element is one
    # multiply-add on a weight of the named format; a b-bit weight carries the information weight 32 / b
    FORMATS = (("Q_1", 1.0), ("Q_2", 2.0), ("Q_3", 3.0), ("Q_4", 4.0), ("Q_6", 6.0), ("Q_8", 8.0), ("Q_12", 12.0), ("Q_16", 16.0),
               ("Q_24", 24.0), ("Q_32", 32.0), ("Q_G_1", 1.0), ("Q_G_2", 2.625), ("Q_G_3", 3.5), ("Q_G_4", 4.5), ("Q_G_6", 6.5625),
               ("Q_G_8", 8.5), ("Q_G_12", 12.5), ("Q_G_16", 16.5), ("Q_G_24", 24.5))
    MIXES = (("Q_MX_3_5", 3.5), ("Q_MX_4_5", 4.5), ("Q_MX_6_5", 6.5), ("Q_MX_8_5", 8.5), ("Q_MX_12_5", 12.5), ("Q_MX_16_5", 16.5),
             ("Q_MX_24_5", 24.5), ("Q_G_MX_3_5", 3.78125), ("Q_G_MX_4_5", 4.5), ("Q_G_MX_6_5", 6.5), ("Q_G_MX_8_5", 8.5),
             ("Q_G_MX_12_5", 12.5), ("Q_G_MX_16_5", 16.5), ("Q_G_MX_24_5", 24.5))

    def record_iw(self, info_weight: float, count: int):
        self.info_ops = getattr(self, "info_ops", 0.0) + count * info_weight
        self.elements = getattr(self, "elements", 0.0) + count
        self.ops += 2 * int(count)

    def record(self, fmt, count: int):
        """``fmt``: index into ``FORMATS`` or a format name."""
        table = self.FORMATS
        i = fmt if isinstance(fmt, int) else next((k for k, (n, _) in enumerate(table) if n == fmt), -1)
        if 0 <= i < len(table):
            self.record_iw(32.0 / table[i][1], count)

    def record_mix(self, mix, count: int):
        table = self.MIXES
        i = mix if isinstance(mix, int) else next((k for k, (n, _) in enumerate(table) if n == mix), -1)
        if 0 <= i < len(table):
            self.record_iw(32.0 / table[i][1], count)

    def elapsed_sec(self) -> float: return self.ns / 1e9
    def gflops(self) -> float: return self.flops() / 1e9
    def effective_gflops(self) -> float: return self.gflops()

    def mean_info_weight(self) -> float:
        el = getattr(self, "elements", 0.0)
        return getattr(self, "info_ops", 0.0) / el if el else 32.0 / max(self.bpw, 1e-9)

    def raw_ops_per_sec(self) -> float: return self.flops() * self.mean_info_weight() / 2.0
    def pinferno(self) -> float: return self.raw_ops_per_sec() / 1e15
    def ninferno(self) -> float: return self.raw_ops_per_sec() / 1e12
    def uinferno(self) -> float: return self.raw_ops_per_sec() / 1e9
    def minferno(self) -> float: return self.raw_ops_per_sec() / 1e6

    def best_unit(self) -> str:
        v = self.raw_ops_per_sec() / 1e21
        for name in ("Inferno", "mInferno", "uInferno", "nInferno", "pInferno"):
            if v >= 1.0:
                return name
            v *= 1e3
        return "fInferno"

    def best_value(self) -> float:
        v = self.raw_ops_per_sec() / 1e21
        for _ in range(4):
            if v >= 1.0:
                return v
            v *= 1e3
        return v


class TaskQueue:
    """Highest priority first, FIFO within a priority; ``submit`` returns an event-like handle with ``result()``."""

    class _Handle:
        def __init__(self):
            self.ev, self.value, self.error = threading.Event(), None, None

        def result(self, timeout=None):
            if not self.ev.wait(timeout):
                raise TimeoutError
            if self.error:
                raise self.error
            return self.value

    def __init__(self, workers=2):
        self.heap, self.cv, self.seq = [], threading.Condition(), itertools.count()
        self.stopped = False
        self.order = []
        self.threads = [threading.Thread(target=self._loop, daemon=True) for _ in range(workers)]
        for t in self.threads:
            t.start()

    def submit(self, fn, *args, priority=0):
        h = self._Handle()
        with self.cv:
            heapq.heappush(self.heap, (-priority, next(self.seq), fn, args, h))
            self.cv.notify()
        return h

    def _loop(self):
        while True:
            with self.cv:
                while not self.heap and not self.stopped:
                    self.cv.wait(0.1)
                if self.stopped and not self.heap:
                    return
                pr, _, fn, args, h = heapq.heappop(self.heap)
                self.order.append(-pr)
            try:
                h.value = fn(*args)
            except Exception as e:
                h.error = e
            h.ev.set()

    def stop(self):
        with self.cv:
            self.stopped = True
            self.cv.notify_all()
        for t in self.threads:
            t.join(timeout=2)
