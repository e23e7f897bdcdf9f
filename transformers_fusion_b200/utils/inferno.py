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
