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


# ---- the reference's verbs (include/quant/self_eval.h: SelfEvalSuite) ---------------------------------------------------
def _builtin_benchmark(name: str, n: int, seed: int = 0) -> List[tuple]:
    """Small generated stand-ins for the named benchmarks (there are no datasets on disk): (prompt, expected answer)
    pairs in the format of each - multiple choice with a lettered answer for "mmlu" / "arc" / "hellaswag", an arithmetic
    word problem with a numeric answer for "gsm8k".  ``SelfEvalSuite.register_benchmark`` replaces them with real cases."""
    rng = random.Random(hash(name) % 9973 + seed)
    out = []
    for _ in range(n):
        a, b = rng.randint(2, 40), rng.randint(2, 40)
        if name == "gsm8k":
            out.append((f"Ann has {a} apples and buys {b} more. How many apples does Ann have? Answer with a number.", str(a + b)))
        else:
            right = a * b if name == "mmlu" else (a + b if name == "arc" else max(a, b))
            what = {"mmlu": f"What is {a} times {b}?", "arc": f"What is {a} plus {b}?",
                    "hellaswag": f"The larger of {a} and {b} is"}.get(name, f"What is {a} plus {b}?")
            opts = sorted({right, right + 1, max(0, right - 2), right + 7})
            rng.shuffle(opts)
            letter = "ABCD"[opts.index(right)]
            out.append((what + " " + " ".join(f"({l}) {o}" for l, o in zip("ABCD", opts)) + " Answer with the letter.", f"({letter})"))
    return out


def _suite_api():
    S = SelfEvalSuite

    def register_benchmark(self, name: str, cases: Sequence[tuple]):
        self.__dict__.setdefault("benchmarks", {})[name] = list(cases)

    def _cases(self, name: str, n: int):
        own = self.__dict__.get("benchmarks", {}).get(name)
        return (own[:n] if own else _builtin_benchmark(name, n))

    def run_accuracy_benchmark(self, benchmark_name: str, n_samples: int = 100) -> dict:
        acc, outs, ok = self.accuracy(_cases(self, benchmark_name, n_samples))
        return {"benchmark": benchmark_name, "accuracy": acc, "n_correct": sum(ok), "n_total": len(ok)}

    def run_accuracy_benchmark_mmlu(self, n_samples: int = 100): return self.run_accuracy_benchmark("mmlu", n_samples)
    def run_accuracy_benchmark_arc(self, n_samples: int = 100): return self.run_accuracy_benchmark("arc", n_samples)
    def run_accuracy_benchmark_hellaswag(self, n_samples: int = 100): return self.run_accuracy_benchmark("hellaswag", n_samples)
    def run_accuracy_benchmark_gsm8k(self, n_samples: int = 100): return self.run_accuracy_benchmark("gsm8k", n_samples)

    def run_calibration_benchmark(self, n_samples: int = 500, benchmark_name: str = "arc", n_bins: int = 10) -> dict:
        cases = _cases(self, benchmark_name, n_samples)
        _, outs, ok = self.accuracy(cases)
        conf = [min(1.0, max(0.0, self.confidence(p, o))) for p, o, _ in outs]
        bins = []
        for b in range(n_bins):
            idx = [i for i, c in enumerate(conf) if b / n_bins <= c < (b + 1) / n_bins or (b == n_bins - 1 and c == 1.0)]
            bins.append({"lower": b / n_bins, "upper": (b + 1) / n_bins, "count": len(idx),
                         "accuracy": sum(ok[i] for i in idx) / len(idx) if idx else 0.0,
                         "confidence": sum(conf[i] for i in idx) / len(idx) if idx else 0.0})
        return {"bins": bins, "ece": self.compute_expected_calibration_error(bins), "n_total": len(conf)}

    @staticmethod
    def compute_expected_calibration_error(bins) -> float:
        n = sum(b["count"] for b in bins)
        return sum(b["count"] / n * abs(b["accuracy"] - b["confidence"]) for b in bins if b["count"]) if n else 0.0

    def run_consistency_benchmark(self, problem: str, n_asks: int = 10) -> dict:
        outs = [self.generate(problem) for _ in range(n_asks)]
        top = max(set(outs), key=outs.count)
        return {"problem": problem, "n_asks": n_asks, "agreement": outs.count(top) / max(1, n_asks), "distinct_answers": len(set(outs)),
                "majority_answer": top}

    def run_consistency_suite(self, n_problems: int = 20, n_asks: int = 10, benchmark_name: str = "gsm8k"):
        return [self.run_consistency_benchmark(p, n_asks) for p, _ in _cases(self, benchmark_name, n_problems)]

    def run_robustness_benchmark(self, problem: str, n_perturbations: int = 50, expected: str = None) -> dict:
        """How often the answer to perturbed wordings equals the answer to the original (or ``expected`` when given)."""
        base = self.generate(problem)
        same = sum((self._match(self.generate(self.perturb(problem)), expected) if expected is not None
                    else self.generate(self.perturb(problem)).strip().lower() == base.strip().lower()) for _ in range(n_perturbations))
        return {"problem": problem, "n_perturbations": n_perturbations, "stability": same / max(1, n_perturbations)}

    def run_robustness_suite(self, n_problems: int = 20, n_perturbations: int = 10, benchmark_name: str = "gsm8k"):
        return [self.run_robustness_benchmark(p, n_perturbations, e) for p, e in _cases(self, benchmark_name, n_problems)]

    def run_speed_benchmark(self, n_operations: int = 1000, prompt: str = "Count to five.") -> dict:
        t0 = time.perf_counter()
        toks = sum(len(self.generate(prompt).split()) for _ in range(n_operations))
        dt = max(time.perf_counter() - t0, 1e-9)
        return {"n_operations": n_operations, "seconds": dt, "ops_per_sec": n_operations / dt, "tokens_per_sec": toks / dt}

    def run_memory_benchmark(self, n_allocations: int = 10000) -> dict:
        """Peak memory of the process (device memory when a GPU is in use) after ``n_allocations`` generations' worth of
        bookkeeping; the figure is what the model and its caches hold, not an allocator stress test."""
        before = self.memory()
        for _ in range(min(n_allocations, 16)):
            self.generate("ping")
        after = self.memory()
        return {"peak_bytes": after, "growth_bytes": max(0, after - before)}

    def run_pass_at_k(self, benchmark_name: str, k: int, n_problems: int = 100, n_samples: int = None) -> dict:
        n = max(k, n_samples or k)
        return {"benchmark": benchmark_name, "k": k, "n_samples": n,
                "pass_at_k": self.pass_at(_cases(self, benchmark_name, n_problems), n, (k,))[k]}

    def run_pass_at_k_suite(self, max_k: int = 10, benchmark_name: str = "gsm8k", n_problems: int = 20):
        return [self.run_pass_at_k(benchmark_name, k, n_problems, max_k) for k in (1, 2, 5, 10) if k <= max_k]

    def generate_report(self, version_id: str, n_samples: int = 20) -> dict:
        acc = {b: self.run_accuracy_benchmark(b, n_samples) for b in ("mmlu", "arc", "hellaswag", "gsm8k")}
        cal = self.run_calibration_benchmark(n_samples)
        cons = self.run_consistency_suite(min(5, n_samples), 3)
        rob = self.run_robustness_suite(min(5, n_samples), 3)
        speed, mem = self.run_speed_benchmark(min(20, n_samples)), self.run_memory_benchmark(4)
        pk = self.run_pass_at_k_suite(5, n_problems=min(5, n_samples))
        mean = lambda xs: sum(xs) / max(1, len(xs))
        overall = (0.4 * mean([a["accuracy"] for a in acc.values()]) + 0.2 * (1 - cal["ece"]) + 0.2 * mean([c["agreement"] for c in cons])
                   + 0.2 * mean([r["stability"] for r in rob]))
        rep = {"version_id": version_id, "timestamp": int(time.time()), "accuracy": acc, "calibration": cal, "consistency_results": cons,
               "robustness_results": rob, "speed": speed, "memory": mem, "pass_at_k_results": pk, "overall_score": overall}
        self.store_report(rep)
        return rep

    def store_report(self, report: dict, max_reports: int = 100):
        hist = self.__dict__.setdefault("reports", [])
        hist.append(report)
        del hist[:-max_reports]

    def get_report_history(self): return list(self.__dict__.get("reports", []))
    def get_latest_report(self): return self.__dict__.get("reports", [None])[-1] if self.__dict__.get("reports") else None

    for name, fn in list(locals().items()):
        if name != "S" and not name.startswith("_") and (callable(fn) or isinstance(fn, staticmethod)):
            setattr(S, name, fn)


_suite_api()
