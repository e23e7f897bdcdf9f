"""Self-evaluation suite: accuracy, calibration, self-consistency, robustness to prompt perturbations, speed, memory,
pass@k and version comparison.  Reference counterpart: include/quant/self_eval.h:16-144, src/agi/self_eval.cpp."""
from __future__ import annotations

import math
import random
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Sequence


def pass_at_k(n: int, c: int, k: int) -> float:
    """Unbiased estimator 1 - C(n - c, k) / C(n, k): probability that at least one of k samples out of n (c correct) passes."""
    if n - c < k:
        return 1.0
    return 1.0 - math.prod((n - c - i) / (n - i) for i in range(k))


@dataclass
class EvaluationReport:
    accuracy: float = 0.0
    ece: float = 0.0
    consistency: float = 0.0
    robustness: float = 0.0
    tokens_per_sec: float = 0.0
    peak_memory_bytes: int = 0
    pass_at_k: Dict[int, float] = field(default_factory=dict)

    def overall(self):
        return 0.4 * self.accuracy + 0.2 * (1 - self.ece) + 0.2 * self.consistency + 0.2 * self.robustness


class SelfEvalSuite:
    def __init__(self, generate: Callable[[str], str], confidence: Callable[[str, str], float] = None, seed=0):
        self.generate, self.confidence = generate, confidence or (lambda p, o: 0.5)
        self.rng = random.Random(seed)

    @staticmethod
    def _match(out, exp):
        return exp.strip().lower() in out.strip().lower()

    def accuracy(self, cases: Sequence[tuple]):
        outs = [(p, self.generate(p), e) for p, e in cases]
        ok = [self._match(o, e) for _, o, e in outs]
        return sum(ok) / max(1, len(ok)), outs, ok

    def calibration(self, cases, n_bins=10):
        _, outs, ok = self.accuracy(cases)
        conf = [min(1.0, max(0.0, self.confidence(p, o))) for p, o, _ in outs]
        ece, n = 0.0, len(conf)
        for b in range(n_bins):
            idx = [i for i, c in enumerate(conf) if b / n_bins <= c < (b + 1) / n_bins or (b == n_bins - 1 and c == 1.0)]
            if idx:
                ece += len(idx) / n * abs(sum(ok[i] for i in idx) / len(idx) - sum(conf[i] for i in idx) / len(idx))
        return ece

    def consistency(self, prompts, samples=3):
        agree = []
        for p in prompts:
            outs = [self.generate(p) for _ in range(samples)]
            agree.append(sum(o == outs[0] for o in outs) / samples)
        return sum(agree) / max(1, len(agree))

    def perturb(self, prompt):
        words = prompt.split()
        if len(words) > 2:
            i = self.rng.randrange(len(words) - 1)
            words[i], words[i + 1] = words[i + 1], words[i]
        return "  ".join(words).upper() if self.rng.random() < 0.5 else " ".join(words) + " "

    def robustness(self, cases, variants=3):
        """Fraction of originally correct cases that stay correct under prompt perturbations."""
        kept = tot = 0
        for p, e in cases:
            if not self._match(self.generate(p), e):
                continue
            for _ in range(variants):
                tot += 1
                kept += self._match(self.generate(self.perturb(p)), e)
        return kept / tot if tot else 0.0

    def speed(self, prompts, count_tokens=lambda s: len(s.split())):
        t0 = time.perf_counter()
        n = sum(count_tokens(self.generate(p)) for p in prompts)
        return n / max(time.perf_counter() - t0, 1e-9)

    @staticmethod
    def memory():
        import torch
        if torch.cuda.is_available():
            return int(torch.cuda.max_memory_allocated())
        import resource
        return int(resource.getrusage(resource.RUSAGE_SELF).ru_maxrss) * 1024

    def pass_at(self, cases, n=5, ks=(1, 5)):
        res = {k: [] for k in ks}
        for p, e in cases:
            c = sum(self._match(self.generate(p), e) for _ in range(n))
            for k in ks:
                res[k].append(pass_at_k(n, c, min(k, n)))
        return {k: sum(v) / max(1, len(v)) for k, v in res.items()}

    def evaluate(self, cases, pass_n=3) -> EvaluationReport:
        r = EvaluationReport()
        r.accuracy = self.accuracy(cases)[0]
        r.ece = self.calibration(cases)
        r.consistency = self.consistency([p for p, _ in cases])
        r.robustness = self.robustness(cases)
        r.tokens_per_sec = self.speed([p for p, _ in cases])
        r.peak_memory_bytes = self.memory()
        r.pass_at_k = self.pass_at(cases, pass_n, (1, pass_n))
        return r

    @staticmethod
    def compare_versions(old: EvaluationReport, new: EvaluationReport, tolerance=0.01):
        deltas = {k: getattr(new, k) - getattr(old, k) for k in ("accuracy", "consistency", "robustness", "tokens_per_sec")}
        deltas["ece"] = old.ece - new.ece
        regressions = [k for k, d in deltas.items() if d < -tolerance * max(1.0, abs(getattr(old, k)))]
        return {"deltas": deltas, "regressions": regressions, "improved": new.overall() > old.overall() and not regressions}
