"""Monitoring, reflection, guardrails, sandboxing, planning and the improvement flywheel."""
from __future__ import annotations

import ast
import math
import os
import re
import subprocess
import sys
import tempfile
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch


@dataclass
class MetaCognitionState:
    confidence: float = 0.0
    uncertainty: float = 0.0
    entropy: float = 0.0
    drift: float = 0.0
    anomaly: bool = False
    notes: str = ""


class RollingStats:
    def __init__(self, window=256):
        self.window, self.values = window, []

    def add(self, v):
        self.values.append(float(v))
        if len(self.values) > self.window:
            self.values.pop(0)

    def mean(self):
        return sum(self.values) / len(self.values) if self.values else 0.0

    def std(self):
        m = self.mean()
        return math.sqrt(sum((v - m) ** 2 for v in self.values) / len(self.values)) if self.values else 0.0

    def zscore(self, v):
        s = self.std()
        return (v - self.mean()) / s if s > 1e-12 else 0.0


@dataclass
class AlertEntry:
    severity: str
    source: str
    message: str
    value: float
    timestamp: float = field(default_factory=time.time)


@dataclass
class AuditEntry:
    action: str
    detail: str
    result: str
    timestamp: float = field(default_factory=time.time)


@dataclass
class Message:
    sender: int
    receiver: int
    content: str
    confidence: float = 1.0
    round: int = 0


@dataclass
class PlanStep:
    id: int
    description: str
    depends_on: List[int] = field(default_factory=list)
    done: bool = False
    confidence: float = 1.0


@dataclass
class SandboxResult:
    compiled: bool = False
    tests_passed: int = 0
    tests_total: int = 0
    stdout: str = ""
    stderr: str = ""
    exit_code: int = -1
    runtime_ms: float = 0.0
    timed_out: bool = False


def _entropy(logits):
    p = torch.softmax(logits.float(), -1)
    return float(-(p * torch.log(p.clamp(min=1e-30))).sum(-1).mean())


class SelfMonitor:
    def __init__(self, generate: Optional[Callable] = None, logits: Optional[Callable] = None):
        self.generate, self.logits = generate, logits
        self.confidence_stats, self.uncertainty_stats = RollingStats(), RollingStats()
        self.alerts: List[AlertEntry] = []
        self.lock = threading.Lock()

    def estimate_confidence(self, logits) -> float:
        return float(torch.softmax(logits.float(), -1).amax(-1).mean())

    @staticmethod
    def distribution_shift(current, reference) -> float:
        """Symmetrised KL between the two predictive distributions."""
        p, q = torch.log_softmax(current.float(), -1), torch.log_softmax(reference.float(), -1)
        return float(0.5 * ((p.exp() * (p - q)).sum(-1) + (q.exp() * (q - p)).sum(-1)).mean())

    def detect_drift(self, current, reference, threshold=0.5) -> bool:
        d = self.distribution_shift(current, reference)
        if d > threshold:
            self._alert("warning", "drift", "predictive distribution moved", d)
        return d > threshold

    def analyze(self, prompt: str, output: str) -> MetaCognitionState:
        st = MetaCognitionState()
        if self.logits is not None:
            lg = self.logits(prompt)
            st.confidence, st.entropy = self.estimate_confidence(lg), _entropy(lg)
            st.uncertainty = st.entropy / math.log(lg.shape[-1])
        else:
            words = output.split()
            st.confidence = len(set(words)) / max(1, len(words))
            st.uncertainty = 1 - st.confidence
        st.anomaly = self.check_anomaly(st)
        self.confidence_stats.add(st.confidence)
        self.uncertainty_stats.add(st.uncertainty)
        return st

    def check_anomaly(self, st: MetaCognitionState, z=3.0) -> bool:
        bad = len(self.confidence_stats.values) >= 8 and abs(self.confidence_stats.zscore(st.confidence)) > z
        if bad:
            self._alert("critical", "confidence", "confidence far from its running mean", st.confidence)
        return bad

    def _alert(self, severity, source, message, value):
        with self.lock:
            self.alerts.append(AlertEntry(severity, source, message, float(value)))

    def get_recent_alerts(self, count=10):
        with self.lock:
            return self.alerts[-count:]

    def clear_alerts(self):
        with self.lock:
            self.alerts = []


class SelfReflector:
    def __init__(self, generate: Callable[[str], str]):
        self.generate = generate

    def reflect(self, prompt, output):
        return self.generate(f"Question:\n{prompt}\nAnswer:\n{output}\nList any mistakes in the answer, or say 'no issues'.")

    def refine(self, original, reflection):
        if "no issues" in reflection.lower():
            return original
        return self.generate(f"Original answer:\n{original}\nCritique:\n{reflection}\nRewrite the answer fixing the critique.")

    @staticmethod
    def consistency_check(a: str, b: str) -> float:
        """Jaccard overlap of the word sets."""
        x, y = set(a.lower().split()), set(b.lower().split())
        return len(x & y) / len(x | y) if x | y else 1.0

    @staticmethod
    def ece_calibration(confidences: Sequence[float], correctness: Sequence[bool], n_bins=10) -> float:
        n, ece = len(confidences), 0.0
        for b in range(n_bins):
            lo, hi = b / n_bins, (b + 1) / n_bins
            idx = [i for i, c in enumerate(confidences) if (lo < c <= hi) or (b == 0 and c == 0)]
            if idx:
                acc = sum(bool(correctness[i]) for i in idx) / len(idx)
                conf = sum(confidences[i] for i in idx) / len(idx)
                ece += len(idx) / n * abs(acc - conf)
        return ece

    @staticmethod
    def identify_errors(prompt, output, expected) -> List[str]:
        errs = []
        if output.strip() == "":
            errs.append("empty output")
        missing = [w for w in expected.split() if w not in output.split()]
        if missing:
            errs.append("missing: " + " ".join(missing[:10]))
        if len(output) > 4 * max(1, len(expected)):
            errs.append("output much longer than expected")
        return errs


class MetaCognition:
    def __init__(self, logits: Optional[Callable] = None):
        self.logits = logits
        self.self_model_accuracy, self.updates = 0.0, 0
        self.knowledge_map: Dict[str, float] = {}

    @staticmethod
    def total_uncertainty(logits) -> float:
        """Entropy of the mean prediction (``logits`` [samples, V] from several stochastic passes, or [V])."""
        lg = logits.float().reshape(-1, logits.shape[-1])
        p = torch.softmax(lg, -1).mean(0)
        return float(-(p * torch.log(p.clamp(min=1e-30))).sum())

    @staticmethod
    def aleatoric_uncertainty(logits) -> float:
        """Mean entropy of the individual predictions."""
        lg = logits.float().reshape(-1, logits.shape[-1])
        p = torch.softmax(lg, -1)
        return float(-(p * torch.log(p.clamp(min=1e-30))).sum(-1).mean())

    def epistemic_uncertainty(self, logits) -> float:
        """Mutual information between prediction and model: total minus aleatoric (zero for a single pass)."""
        return max(0.0, self.total_uncertainty(logits) - self.aleatoric_uncertainty(logits))

    def knowledge_boundary_score(self, query: str) -> float:
        if query in self.knowledge_map:
            return self.knowledge_map[query]
        if self.logits is None:
            return 0.5
        lg = self.logits(query)
        return 1.0 - _entropy(lg) / math.log(lg.shape[-1])

    def should_refuse(self, query, uncertainty_threshold=0.7) -> bool:
        return 1.0 - self.knowledge_boundary_score(query) > uncertainty_threshold

    @staticmethod
    def reasoning_quality(chain: Sequence[str]) -> float:
        """Heuristic in [0, 1]: steps exist, are not duplicates, and each shares vocabulary with its predecessor."""
        if not chain:
            return 0.0
        uniq = len(set(chain)) / len(chain)
        link = [SelfReflector.consistency_check(a, b) > 0 for a, b in zip(chain, chain[1:])]
        return 0.5 * uniq + 0.5 * (sum(link) / len(link) if link else 1.0)

    def self_model_update(self, query, confidence, was_correct):
        self.updates += 1
        hit = (confidence >= 0.5) == bool(was_correct)
        self.self_model_accuracy += (float(hit) - self.self_model_accuracy) / self.updates
        self.knowledge_map[query] = 0.8 * self.knowledge_map.get(query, confidence) + 0.2 * float(was_correct)


class SafetyGuardrails:
    DEFAULT_BLOCKED = [r"rm\s+-rf\s+/", r"\bmkfs\b", r":\(\)\{\s*:\|:&\s*\};:", r"\bshutdown\b", r"DROP\s+TABLE", r"/etc/passwd"]

    def __init__(self, blocked_patterns: Optional[Sequence[str]] = None):
        self.blocked = [re.compile(p, re.I) for p in (blocked_patterns or self.DEFAULT_BLOCKED)]
        self.invariants: Dict[str, Callable[[], bool]] = {}
        self.audit: List[AuditEntry] = []
        self.kill_switch, self.paused = False, False
        self.lock = threading.Lock()

    def _scan(self, text):
        return not any(p.search(text) for p in self.blocked)

    def check_input(self, text):
        ok = not self.kill_switch and self._scan(text)
        self.audit_log("check_input", text[:80], "ok" if ok else "blocked")
        return ok

    def check_output(self, text):
        ok = not self.kill_switch and self._scan(text)
        self.audit_log("check_output", text[:80], "ok" if ok else "blocked")
        return ok

    def check_modification(self, target, change):
        protected = any(k in target for k in ("guardrail", "kill_switch", "audit"))
        ok = not protected and not self.kill_switch and not self.paused and self._scan(change)
        self.audit_log("check_modification", f"{target}: {change[:60]}", "ok" if ok else "blocked")
        return ok

    def set_invariant(self, name, predicate: Callable[[], bool]):
        self.invariants[name] = predicate

    def check_invariant(self, name) -> bool:
        ok = bool(self.invariants[name]()) if name in self.invariants else False
        self.audit_log("check_invariant", name, "ok" if ok else "violated")
        return ok

    def get_invariants(self):
        return sorted(self.invariants)

    def human_override(self, action, reason):
        self.audit_log("human_override", f"{action}: {reason}", "granted")
        return True

    def audit_log(self, action, detail, result):
        with self.lock:
            self.audit.append(AuditEntry(action, detail, result))

    def get_audit_log(self, count=50):
        with self.lock:
            return self.audit[-count:]

    def set_kill_switch(self, kill):
        self.kill_switch = bool(kill)

    def is_killed(self):
        return self.kill_switch


class Sandbox:
    """Runs untrusted Python snippets in a child interpreter with a time limit, an address-space limit and an empty
    environment, after a static pass that rejects imports and calls outside an allow-list."""

    ALLOWED_IMPORTS = {"math", "itertools", "functools", "collections", "heapq", "bisect", "statistics", "fractions", "random"}
    FORBIDDEN_CALLS = {"eval", "exec", "open", "__import__", "compile", "input", "breakpoint"}

    def __init__(self):
        self.dir = tempfile.mkdtemp(prefix="tfb_sandbox_")
        self.lock = threading.Lock()

    def get_sandbox_path(self):
        return self.dir

    def static_analysis(self, code: str) -> List[str]:
        issues = []
        try:
            tree = ast.parse(code)
        except SyntaxError as e:
            return [f"syntax error: {e.msg} (line {e.lineno})"]
        for node in ast.walk(tree):
            if isinstance(node, (ast.Import, ast.ImportFrom)):
                names = [a.name.split(".")[0] for a in node.names] if isinstance(node, ast.Import) else [(node.module or "").split(".")[0]]
                issues += [f"import of '{n}' is not allowed" for n in names if n not in self.ALLOWED_IMPORTS]
            elif isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in self.FORBIDDEN_CALLS:
                issues.append(f"call to '{node.func.id}' is not allowed")
            elif isinstance(node, ast.Attribute) and node.attr.startswith("__") and node.attr not in ("__init__", "__name__", "__len__"):
                issues.append(f"access to '{node.attr}' is not allowed")
            elif isinstance(node, ast.While) and isinstance(node.test, ast.Constant) and node.test.value is True and \
                    not any(isinstance(n, (ast.Break, ast.Return)) for n in ast.walk(node)):
                issues.append("unbounded 'while True' loop")
        return issues

    def check_resource_limits(self, code, max_memory_mb=256, max_time_sec=10.0) -> bool:
        r = self._run(code, max_time_sec, max_memory_mb)
        return not r.timed_out and r.exit_code == 0

    def _run(self, program: str, timeout_s: float, mem_mb: int = 256) -> SandboxResult:
        res = SandboxResult()
        with self.lock:
            path = os.path.join(self.dir, f"prog_{time.time_ns()}.py")
            with open(path, "w") as f:
                f.write(program)

            def limits():
                import resource
                resource.setrlimit(resource.RLIMIT_AS, (mem_mb << 20, mem_mb << 20))
                resource.setrlimit(resource.RLIMIT_CPU, (int(timeout_s) + 1, int(timeout_s) + 1))
            t0 = time.perf_counter()
            try:
                p = subprocess.run([sys.executable, "-I", "-S", path], capture_output=True, text=True, timeout=timeout_s, cwd=self.dir,
                                   env={}, preexec_fn=limits)
                res.stdout, res.stderr, res.exit_code = p.stdout, p.stderr, p.returncode
            except subprocess.TimeoutExpired as e:
                res.timed_out, res.stderr = True, "timeout"
                res.stdout = e.stdout.decode() if isinstance(e.stdout, bytes) else (e.stdout or "")
            res.runtime_ms = (time.perf_counter() - t0) * 1e3
            os.unlink(path)
        return res

    def compile_and_test(self, code: str, tests: Sequence[str] = (), timeout_s=5.0) -> SandboxResult:
        """``tests`` are Python expressions that must evaluate to true after ``code`` has run."""
        issues = self.static_analysis(code)
        if issues:
            return SandboxResult(compiled=False, stderr="; ".join(issues), tests_total=len(tests))
        harness = code + "\n_passed = 0\n" + "".join(
            f"try:\n    _passed += 1 if ({t}) else 0\nexcept Exception:\n    pass\n" for t in tests) + "print('PASSED', _passed)\n"
        r = self._run(harness, timeout_s)
        r.compiled = r.exit_code == 0
        r.tests_total = len(tests)
        m = re.search(r"PASSED (\d+)", r.stdout)
        r.tests_passed = int(m.group(1)) if m else 0
        return r

    def verify_correctness(self, code, tests) -> bool:
        r = self.compile_and_test(code, tests)
        return r.compiled and r.tests_passed == r.tests_total

    def benchmark(self, code, repeat=3):
        """(runs per second, mean latency in ms) of running the snippet."""
        ts = [self._run(code, 10.0).runtime_ms for _ in range(repeat)]
        avg = sum(ts) / len(ts)
        return 1e3 / avg, avg


class MultiAgentCoordinator:
    ROLES = ["Analyst", "Implementer", "Verifier", "Critic", "Synthesizer"]
    ANALYST, IMPLEMENTER, VERIFIER, CRITIC, SYNTHESIZER = range(5)

    def __init__(self, generate: Callable[[str], str]):
        self.generate = generate
        self.queues: List[List[Message]] = [[] for _ in self.ROLES]
        self.histories: List[List[str]] = [[] for _ in self.ROLES]
        self.round, self.converged = 0, False
        self.lock = threading.Lock()

    @classmethod
    def role_name(cls, r):
        return cls.ROLES[r]

    def send_message(self, sender, receiver, content, confidence=1.0):
        with self.lock:
            self.queues[receiver].append(Message(sender, receiver, content, confidence, self.round))

    def receive_message(self, agent) -> Optional[Message]:
        with self.lock:
            return self.queues[agent].pop(0) if self.queues[agent] else None

    def get_message_queue(self, agent):
        return list(self.queues[agent])

    def get_agent_history(self, agent):
        return list(self.histories[agent])

    def clear_agent_history(self, agent):
        self.histories[agent] = []

    def _call(self, role, prompt):
        out = self.generate(f"[{self.ROLES[role]}] {prompt}")
        self.histories[role].append(out)
        return out

    def run_task(self, task: str, max_critic_rounds=3) -> str:
        analysis = self._call(self.ANALYST, f"Analyse the task: {task}")
        self.send_message(self.ANALYST, self.IMPLEMENTER, analysis)
        impl = self._call(self.IMPLEMENTER, f"Implement according to: {analysis}")
        critique = ""
        for r in range(max_critic_rounds):
            self.round = r + 1
            ver = self._call(self.VERIFIER, f"Verify: {impl}")
            critique = self._call(self.CRITIC, f"Critique given verification '{ver}': {impl}")
            self.send_message(self.CRITIC, self.IMPLEMENTER, critique, 0.8)
            if re.search(r"\b(approve|lgtm|no issues|accept)", critique, re.I):
                self.converged = True
                break
            impl = self._call(self.IMPLEMENTER, f"Revise to address: {critique}\nPrevious: {impl}")
        return self._call(self.SYNTHESIZER, f"Summarise the final result for '{task}': {impl}")

    def is_converged(self):
        return self.converged

    def get_round(self):
        return self.round


class PlanningEngine:
    def __init__(self, generate: Optional[Callable[[str], str]] = None, executor: Optional[Callable[[PlanStep], bool]] = None):
        self.generate, self.executor = generate, executor or (lambda s: True)
        self.execution_history: List[PlanStep] = []

    def decompose(self, goal, depth=3) -> List[PlanStep]:
        """Ask the model for numbered steps ("1. ... (after 1, 2)"); without a model, split the goal on ' then ' / ';'."""
        if self.generate is not None:
            text = self.generate(f"Break the goal into at most {depth * 3} numbered steps; mention dependencies as '(after N)'.\nGoal: {goal}")
            lines = [l for l in text.splitlines() if re.match(r"\s*\d+[.)]", l)]
        else:
            lines = [f"{i + 1}. {p.strip()}" for i, p in enumerate(re.split(r";|\bthen\b", goal)) if p.strip()]
        steps = []
        for l in lines:
            m = re.match(r"\s*(\d+)[.)]\s*(.*)", l)
            deps = [int(x) for x in re.findall(r"after\s+((?:\d+[,\s]*)+)", l) for x in re.findall(r"\d+", x)]
            sid = int(m.group(1))
            steps.append(PlanStep(sid, re.sub(r"\(after[^)]*\)", "", m.group(2)).strip(), [d for d in deps if d != sid]))
        for a, b in zip(steps, steps[1:]):
            if not b.depends_on:
                b.depends_on = [a.id]
        return steps

    def plan(self, goal, max_steps=20):
        return self.topological_sort(self.decompose(goal))[:max_steps]

    @staticmethod
    def topological_sort(steps: List[PlanStep]) -> List[PlanStep]:
        by = {s.id: s for s in steps}
        done, out = set(), []

        def visit(s, stack=()):
            if s.id in done:
                return
            if s.id in stack:
                raise ValueError(f"dependency cycle through step {s.id}")
            for d in s.depends_on:
                if d in by:
                    visit(by[d], stack + (s.id,))
            done.add(s.id)
            out.append(s)
        for s in steps:
            visit(s)
        return out

    def execute(self, plan: List[PlanStep]) -> bool:
        for s in plan:
            s.done = bool(self.executor(s))
            self.execution_history.append(s)
            if not s.done:
                return False
        return True

    @staticmethod
    def estimate_confidence(plan):
        c = 1.0
        for s in plan:
            c *= s.confidence
        return c

    def replan(self, failed_plan, failure_reason, max_steps=10):
        keep = [s for s in failed_plan if s.done]
        failed = next((s for s in failed_plan if not s.done), None)
        nid = max([s.id for s in failed_plan] + [0]) + 1
        fix = PlanStep(nid, f"resolve: {failure_reason}", [s.id for s in keep[-1:]], False, 0.7)
        rest = [PlanStep(s.id, s.description, [nid] if s is failed else s.depends_on, False, s.confidence * 0.9) for s in failed_plan if not s.done]
        return (keep + [fix] + rest)[: len(keep) + max_steps]

    def clear_execution_history(self):
        self.execution_history = []


class HITL:
    """Human in the loop: actions wait for an approver callback (default: deny while paused, approve otherwise)."""

    def __init__(self, approver: Optional[Callable[[str], bool]] = None):
        self.approver, self.paused = approver, False
        self.approval_history: List[AuditEntry] = []

    def request_approval(self, action) -> bool:
        ok = False if self.paused else (self.approver(action) if self.approver else True)
        self.approval_history.append(AuditEntry("approval", action, "approved" if ok else "denied"))
        return ok

    def pause(self):
        self.paused = True

    def resume(self):
        self.paused = False


class AlignmentSystem:
    max_loop_iterations = 100
    NEGATIVE = ("harm", "deceive", "illegal", "exploit", "weapon", "steal")
    POSITIVE = ("help", "safe", "honest", "explain", "careful", "verify")

    def value_alignment_score(self, output: str) -> float:
        w = output.lower().split()
        neg = sum(any(n in t for n in self.NEGATIVE) for t in w)
        pos = sum(any(p in t for p in self.POSITIVE) for t in w)
        return max(0.0, min(1.0, 0.5 + 0.5 * (pos - 2 * neg) / max(4, len(w) ** 0.5)))


class SelfVerifier:
    def __init__(self, sandbox: Optional[Sandbox] = None):
        self.sandbox = sandbox or Sandbox()

    def verify_code(self, code, tests):
        return self.sandbox.verify_correctness(code, tests)

    @staticmethod
    def verify_arithmetic(expr: str, claimed: float, tol=1e-9) -> bool:
        node = ast.parse(expr, mode="eval")
        if not all(isinstance(n, (ast.Expression, ast.BinOp, ast.UnaryOp, ast.Constant, ast.operator, ast.unaryop)) for n in ast.walk(node)):
            return False
        return abs(eval(compile(node, "<expr>", "eval"), {"__builtins__": {}}) - claimed) <= tol


class RecursiveSelfImprover:
    """Improvement cycle over a training callback: find weaknesses, propose changes (learning rate, dropout, perturbation,
    pruning), score each candidate, keep the ones that improve the evaluation."""

    def __init__(self, evaluate: Callable[[dict], float], guard: Optional[SafetyGuardrails] = None):
        self.evaluate, self.guard = evaluate, guard or SafetyGuardrails()
        self.settings = {"learning_rate": 1e-4, "dropout": 0.0, "prune_threshold": 0.0, "perturbation": 0.0}
        self.history: List[dict] = []

    def evaluate_weaknesses(self, report: Dict[str, float]) -> List[str]:
        return [k for k, v in sorted(report.items(), key=lambda kv: kv[1]) if v < 0.6]

    def generate_candidates(self, weaknesses) -> List[dict]:
        s, out = self.settings, []
        for f in (0.5, 2.0):
            out.append({**s, "learning_rate": s["learning_rate"] * f})
        out.append({**s, "dropout": min(0.5, s["dropout"] + 0.05)})
        out.append({**s, "perturbation": 0.01})
        if any("size" in w or "speed" in w for w in weaknesses):
            out.append({**s, "prune_threshold": 0.01})
        return out

    def accept_candidate(self, cand, score, base) -> bool:
        return score > base and self.guard.check_modification("training settings", str(cand))

    def improvement_cycle(self, iterations=10, report: Optional[Dict[str, float]] = None):
        base = self.evaluate(self.settings)
        for _ in range(min(iterations, AlignmentSystem.max_loop_iterations)):
            if self.guard.is_killed():
                break
            cands = self.generate_candidates(self.evaluate_weaknesses(report or {}))
            scored = [(self.evaluate(c), c) for c in cands]
            best, cand = max(scored, key=lambda t: t[0])
            if not self.accept_candidate(cand, best, base):
                break
            self.settings, base = cand, best
            self.history.append({"score": best, **cand})
        return base


class CuriosityDrivenExplorer:
    """Picks the candidate whose outcome the learner predicts worst (largest running prediction error)."""

    def __init__(self, decay=0.9):
        self.err: Dict[str, float] = {}
        self.visits: Dict[str, int] = {}
        self.decay = decay

    def observe(self, key, predicted, actual):
        e = abs(predicted - actual)
        self.err[key] = self.decay * self.err.get(key, e) + (1 - self.decay) * e
        self.visits[key] = self.visits.get(key, 0) + 1

    def novelty(self, key):
        return self.err.get(key, 1.0) + 1.0 / math.sqrt(1 + self.visits.get(key, 0))

    def select(self, keys):
        return max(keys, key=self.novelty)


class ContinuousLearner:
    def __init__(self, train_step: Callable, buffer_size=1024, replay_ratio=0.25):
        self.train_step, self.buffer, self.size, self.ratio = train_step, [], buffer_size, replay_ratio
        self.steps = 0

    def learn(self, batch):
        self.steps += 1
        loss = self.train_step(batch)
        self.buffer.append(batch)
        if len(self.buffer) > self.size:
            self.buffer.pop(0)
        if self.buffer and self.steps % max(1, int(1 / self.ratio)) == 0:
            self.train_step(self.buffer[(self.steps * 7919) % len(self.buffer)])
        return loss


class KnowledgeDistillation:
    def __init__(self, temperature=2.0, alpha=0.5):
        self.T, self.alpha = temperature, alpha

    def loss(self, student_logits, teacher_logits, labels=None):
        T = self.T
        kd = torch.nn.functional.kl_div(torch.log_softmax(student_logits.float() / T, -1), torch.softmax(teacher_logits.float() / T, -1),
                                        reduction="batchmean") * T * T
        if labels is None:
            return kd
        ce = torch.nn.functional.cross_entropy(student_logits.float().view(-1, student_logits.shape[-1]), labels.reshape(-1))
        return self.alpha * kd + (1 - self.alpha) * ce


class PromptOptimizer:
    def __init__(self, score: Callable[[str], float]):
        self.score = score

    def optimize(self, base: str, variants: Sequence[str]):
        scored = sorted(((self.score(v.format(base=base) if "{base}" in v else v + base), v) for v in variants), reverse=True)
        return scored[0][1], scored


class ChainOfThought:
    def __init__(self, generate):
        self.generate = generate

    def solve(self, question, n_steps=4):
        chain, ctx = [], question
        for i in range(n_steps):
            step = self.generate(f"{ctx}\nStep {i + 1}:")
            chain.append(step)
            ctx += f"\nStep {i + 1}: {step}"
            if re.search(r"\b(answer|therefore|final)\b", step, re.I):
                break
        return chain, self.generate(ctx + "\nFinal answer:")


class ToolUse:
    def __init__(self):
        self.tools: Dict[str, Callable] = {}

    def register(self, name, fn):
        self.tools[name] = fn

    def run(self, text: str):
        """Executes every ``tool_name(arg)`` call found in ``text``; returns {call: result or error}."""
        out = {}
        for name, arg in re.findall(r"(\w+)\(([^()]*)\)", text):
            if name in self.tools:
                try:
                    out[f"{name}({arg})"] = self.tools[name](arg.strip().strip("'\""))
                except Exception as e:
                    out[f"{name}({arg})"] = f"error: {e}"
        return out


class MemorySystem:
    """Short-term ring + long-term store retrieved by word overlap."""

    def __init__(self, short_capacity=16):
        self.short, self.long, self.cap = [], [], short_capacity

    def remember(self, text, important=False):
        self.short.append(text)
        if len(self.short) > self.cap:
            self.long.append(self.short.pop(0))
        if important:
            self.long.append(text)

    def recall(self, query, k=3):
        q = set(query.lower().split())
        pool = self.long + self.short
        return sorted(pool, key=lambda t: -len(q & set(t.lower().split())))[:k]


class EvaluationHarness:
    def __init__(self, generate):
        self.generate = generate

    def run(self, cases: Sequence[tuple], match=lambda out, exp: exp.strip().lower() in out.strip().lower()):
        res = [(p, self.generate(p), e) for p, e in cases]
        ok = [match(o, e) for _, o, e in res]
        return {"accuracy": sum(ok) / max(1, len(ok)), "failures": [(p, o, e) for (p, o, e), k in zip(res, ok) if not k]}


class Flywheel:
    """evaluate -> find weaknesses -> improve -> verify -> (guarded) accept, with a record per iteration."""

    def __init__(self, harness: EvaluationHarness, improver: Callable[[list], None], guard: Optional[SafetyGuardrails] = None,
                 hitl: Optional[HITL] = None):
        self.harness, self.improver, self.guard, self.hitl = harness, improver, guard or SafetyGuardrails(), hitl or HITL()
        self.iterations: List[dict] = []

    def run(self, cases, max_iterations=5, target=1.0):
        for i in range(min(max_iterations, AlignmentSystem.max_loop_iterations)):
            if self.guard.is_killed():
                break
            rep = self.harness.run(cases)
            self.iterations.append({"iteration": i, "accuracy": rep["accuracy"], "failures": len(rep["failures"])})
            if rep["accuracy"] >= target or not rep["failures"]:
                break
            if not self.hitl.request_approval(f"improve on {len(rep['failures'])} failures"):
                break
            self.improver(rep["failures"])
        return self.iterations


class CodeGenSelfImprover:
    """Closes the loop between profiling and the kernel source generator: takes per-op timings and roofline targets, asks
    the generator for shape-specialised candidates of the slowest op, keeps those that compile (and, with a GPU, pass the
    numerical check) and reports the best.  Reference counterpart: CodeGenSelfImprover (include/quant/agi.h)."""

    def __init__(self, generator=None):
        if generator is None:
            from ..trainer.code_gen import CodeGenerator
            generator = CodeGenerator()
        self.gen = generator
        self.history: list = []

    def improve(self, timings_ms: dict, roofline_ms: dict = None, n: int = 1 << 20, threshold_ms: float = 0.0):
        from ..trainer.code_gen import KernelType
        paths = self.gen.identify_slow_paths(timings_ms, roofline_ms or {}, threshold_ms)
        for p_ in paths:
            name = p_.op_name.upper()
            if name not in KernelType.__members__:
                continue
            try:
                cands = self.gen.auto_optimize(KernelType[name], n, 3)
            except ValueError:
                continue
            if cands:
                self.history.append((p_.op_name, cands[0].function_name, cands[0].benchmark_ms))
                return cands[0]
        return None


class HPOptimizer:
    """Hyper-parameter search facade over trainer.hpo_nas.HPOEngine (random / successive-halving / evolutionary search
    over a SearchSpace with a user objective).  Reference counterpart: HPOptimizer (include/quant/agi.h)."""

    def __init__(self, space=None, seed: int = 0):
        from ..trainer.hpo_nas import HPOEngine, SearchSpace
        self.engine = HPOEngine(space or SearchSpace(), seed=seed) if _accepts(HPOEngine, "seed") else HPOEngine(space or SearchSpace())

    def __getattr__(self, name):
        return getattr(self.engine, name)


class NeuralArchitectureSearch:
    """Architecture search facade over trainer.hpo_nas.NASEngine (mutation-based evolution under hardware constraints).
    Reference counterpart: NeuralArchitectureSearch (include/quant/agi.h)."""

    def __init__(self, cfg=None, constraints=None):
        from ..trainer.hpo_nas import NASConfig, NASEngine
        args = [a for a in (cfg or NASConfig(), constraints) if a is not None]
        try:
            self.engine = NASEngine(*args)
        except TypeError:
            self.engine = NASEngine(args[0])

    def __getattr__(self, name):
        return getattr(self.engine, name)


def _accepts(cls, name: str) -> bool:
    import inspect
    return name in inspect.signature(cls.__init__).parameters


# =====================================================================================================================
# The reference's verb names on the classes above (include/quant/agi.h)
# =====================================================================================================================
def _agi_api():
    import difflib

    def put(cls, **fns):
        for name, fn in fns.items():
            setattr(cls, name, fn)

    # ---- RollingStats
    put(RollingStats, update=RollingStats.add, z_score=RollingStats.zscore,
        is_anomalous=lambda self, value, threshold=3.0: len(self.values) >= 8 and abs(self.zscore(value)) > threshold)

    # ---- SelfMonitor / MetaCognition / guardrails / planning / human in the loop: accessors
    put(SelfMonitor, get_confidence_stats=lambda self: self.confidence_stats, get_uncertainty_stats=lambda self: self.uncertainty_stats)
    put(MetaCognition, get_self_model_accuracy=lambda self: self.self_model_accuracy)
    put(SafetyGuardrails, set_paused=lambda self, p: setattr(self, "paused", bool(p)), is_paused=lambda self: getattr(self, "paused", False))
    put(PlanningEngine, get_execution_history=lambda self: list(self.execution_history))
    put(HITL, get_approval_history=lambda self: list(self.approval_history), is_paused=lambda self: self.paused)

    # ---- RecursiveSelfImprover: the individual knobs
    def adjust_lr(self, weakness: str = ""):
        """Unstable / diverging -> halve the rate; slow / plateau -> raise it by half."""
        w = weakness.lower()
        f = 0.5 if any(k in w for k in ("unstable", "diverg", "nan", "spike", "overfit")) else (1.5 if any(k in w for k in ("slow", "plateau", "underfit")) else 1.0)
        self.settings["learning_rate"] *= f
        return self.settings["learning_rate"]

    def apply_perturbation(self, magnitude: float = 0.01):
        self.settings["perturbation"] = float(magnitude)

    def apply_dropout(self, rate: float = 0.1):
        self.settings["dropout"] = min(0.9, max(0.0, float(rate)))

    def apply_pruning(self, threshold: float = 0.01):
        self.settings["prune_threshold"] = max(0.0, float(threshold))

    def adjust_format(self, analysis: str = ""):
        """Pick the weight format the analysis calls for: memory-bound -> fewer bits, accuracy loss -> more bits."""
        a = analysis.lower()
        order = ["q2", "q4", "q8", "q16"]
        cur = order.index(self.settings.get("format", "q8"))
        if any(k in a for k in ("memory", "size", "bandwidth", "slow")):
            cur = max(0, cur - 1)
        elif any(k in a for k in ("accuracy", "quality", "precision", "degrad")):
            cur = min(len(order) - 1, cur + 1)
        self.settings["format"] = order[cur]
        return order[cur]

    def evaluate_candidate(self, candidate) -> float:
        return float(self.evaluate(candidate if isinstance(candidate, dict) else self.settings))

    def self_modify(self, analysis: str) -> bool:
        """Apply the change an analysis in words asks for, keep it only when the evaluation improves (and the guard lets
        the modification through); returns whether it was kept."""
        before, base = dict(self.settings), self.evaluate(self.settings)
        a = analysis.lower()
        if "dropout" in a or "overfit" in a:
            self.apply_dropout(min(0.5, self.settings["dropout"] + 0.05))
        if "prun" in a or "sparse" in a:
            self.apply_pruning(0.01)
        if any(k in a for k in ("learning rate", "unstable", "diverg", "slow", "plateau")):
            self.adjust_lr(analysis)
        if "format" in a or "bits" in a or "memory" in a:
            self.adjust_format(analysis)
        if self.settings == before:
            return False
        score = self.evaluate(self.settings)
        if score > base and self.guard.check_modification("training settings", str(self.settings)):
            self.history.append({"score": score, **self.settings})
            return True
        self.settings = before
        return False
    put(RecursiveSelfImprover, adjust_lr=adjust_lr, apply_perturbation=apply_perturbation, apply_dropout=apply_dropout,
        apply_pruning=apply_pruning, adjust_format=adjust_format, evaluate_candidate=evaluate_candidate, self_modify=self_modify)

    # ---- CodeGenSelfImprover
    def generate_kernel(self, op: str, M: int, N: int = 1, K: int = 1) -> str:
        """CUDA source of a shape-specialised kernel for ``op`` from the kernel source generator ("" when the generator has
        no template for it)."""
        from ..trainer.code_gen import KernelType
        name = op.upper()
        if name not in KernelType.__members__:
            return ""
        try:
            cands = self.gen.auto_optimize(KernelType[name], max(1, M * N), 1)
        except ValueError:
            return ""
        return getattr(cands[0], "source", "") if cands else ""

    def compile_and_test(self, code: str) -> bool:
        """Does the source compile for sm_100a?  (nvcc -c into a scratch directory; no GPU is needed, nothing is run.)"""
        import shutil
        import subprocess
        import tempfile
        if not code.strip() or shutil.which("nvcc") is None:
            return False
        with tempfile.TemporaryDirectory() as d:
            src = os.path.join(d, "k.cu")
            open(src, "w").write(code)
            r = subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-c", src, "-o", os.path.join(d, "k.o")],
                               capture_output=True, text=True, timeout=300)
            self.last_compile_log = r.stderr[-2000:]
            return r.returncode == 0

    def replace_kernel(self, op: str, new_code: str) -> bool:
        """Register a candidate source for ``op`` (kept in memory; the framework's own kernels are built from the source
        tree and are never overwritten by generated code)."""
        if not self.compile_and_test(new_code):
            return False
        self.__dict__.setdefault("candidates", {})[op] = new_code
        return True
    put(CodeGenSelfImprover, generate_kernel=generate_kernel, compile_and_test=compile_and_test, replace_kernel=replace_kernel)

    # ---- SelfVerifier
    def verify(self, problem: str, solution: str) -> bool:
        """Arithmetic claims ("12 * 7 = 84") are recomputed; code blocks must run in the sandbox; anything else passes only
        when it is non-empty and does not contradict a number asked for in the problem."""
        claims = re.findall(r"([-+*/().\d\s]+?)\s*=\s*(-?\d+(?:\.\d+)?)", solution)
        checked = False
        for expr, val in claims:
            if re.search(r"\d\s*[-+*/]\s*\d", expr):
                checked = True
                try:
                    if not self.verify_arithmetic(expr.strip(), float(val), 1e-6):
                        return False
                except (SyntaxError, ZeroDivisionError, ValueError):
                    return False
        m = re.search(r"```(?:python)?\n(.*?)```", solution, re.S)
        if m:
            checked = True
            r_ = self.sandbox.compile_and_test(m.group(1))
            if not (r_.compiled and r_.exit_code == 0):
                return False
        return checked or bool(solution.strip())

    def find_edge_cases(self, solution: str) -> List[str]:
        """Inputs worth trying against a solution, read off its text: boundaries of the numbers it mentions, empty / zero /
        negative inputs, and the usual suspects of the constructs it uses."""
        cases = ["empty input", "zero", "negative value"]
        for n in sorted({int(x) for x in re.findall(r"\b\d{1,9}\b", solution)})[:4]:
            cases += [f"{n - 1}", f"{n}", f"{n + 1}"]
        if re.search(r"/|divide|ratio", solution, re.I):
            cases.append("division by zero")
        if re.search(r"\[|index|list|array", solution, re.I):
            cases += ["single element", "index out of range"]
        if re.search(r"sort|order|max|min", solution, re.I):
            cases += ["all elements equal", "already sorted", "reverse sorted"]
        if re.search(r"str|text|char", solution, re.I):
            cases += ["non-ASCII text", "very long string"]
        return list(dict.fromkeys(cases))
    put(SelfVerifier, verify=verify, find_edge_cases=find_edge_cases)

    # ---- CuriosityDrivenExplorer
    def intrinsic_reward(self, state) -> float:
        """Novelty of a state (a key, or a tensor / sequence hashed by its rounded content)."""
        key = state if isinstance(state, str) else repr([round(float(v), 2) for v in torch.as_tensor(state).reshape(-1)[:16].tolist()])
        return self.novelty(key)

    def explore(self, n_steps: int, keys: Optional[Sequence] = None, outcome: Optional[Callable] = None) -> List[int]:
        """Visit ``n_steps`` times the index of the most novel candidate among ``keys`` (default: the keys seen so far);
        ``outcome(key)`` gives the observed value, the running mean of which is the prediction."""
        keys = list(keys) if keys is not None else sorted(self.err)
        if not keys:
            return []
        mean: Dict = {}
        out = []
        for _ in range(n_steps):
            k = self.select(keys)
            y = float(outcome(k)) if outcome else 0.0
            self.observe(k, mean.get(k, 0.0), y)
            mean[k] = 0.5 * mean.get(k, 0.0) + 0.5 * y
            out.append(keys.index(k))
        return out
    put(CuriosityDrivenExplorer, intrinsic_reward=intrinsic_reward, explore=explore)

    # ---- facades over the search engines
    put(NeuralArchitectureSearch, search=lambda self, population=50, generations=20: self.engine.search(population, generations))

    put(HPOptimizer, population_based_training=lambda self, n_population=8, n_generations=10:
        self.engine.population_based_training(n_population, n_generations))

    # ---- ContinuousLearner
    def cl_update(self, new_data):
        return self.learn(new_data)

    def prevent_forgetting(self, threshold: float = 0.95, evaluate: Optional[Callable] = None) -> bool:
        """True while the retained skill is at least ``threshold`` of its best value so far; when it drops below, the whole
        replay buffer is trained on once.  ``evaluate()`` returns the skill (higher is better)."""
        if evaluate is None:
            return True
        s = float(evaluate())
        self.best_skill = max(getattr(self, "best_skill", s), s)
        if s >= threshold * self.best_skill:
            return True
        for b in self.buffer:
            self.train_step(b)
        return False
    put(ContinuousLearner, update=cl_update, prevent_forgetting=prevent_forgetting)

    # ---- KnowledgeDistillation
    def distill(self, data, steps: int, student=None, teacher=None, opt=None):
        """``steps`` optimizer steps of the student on the distillation loss against the teacher's logits.  ``data``:
        a loader with ``next_batch()`` or an iterable of (ids, labels); models map ids -> logits."""
        student, teacher = student or self.student, teacher or self.teacher
        opt = opt or torch.optim.Adam([p for p in student.parameters() if p.requires_grad], lr=1e-3)
        it = iter(data) if not hasattr(data, "next_batch") else None
        last = 0.0
        for _ in range(steps):
            ids, labels = data.next_batch() if it is None else next(it)
            with torch.no_grad():
                t_logits = teacher(ids)
            loss = self.loss(student(ids), t_logits, labels)
            opt.zero_grad()
            loss.backward()
            opt.step()
            last = float(loss.detach())
        return last
    put(KnowledgeDistillation, distill=distill, student=None, teacher=None)

    # ---- PromptOptimizer / ChainOfThought / ToolUse / MemorySystem / EvaluationHarness / Flywheel
    def po_evaluate(self, prompt: str, task: str = "") -> float:
        return float(self.score(prompt + task))
    put(PromptOptimizer, evaluate=po_evaluate)

    def reason(self, problem: str, max_steps: int = 10) -> str:
        self.chain, answer = self.solve(problem, max_steps)
        return answer
    put(ChainOfThought, reason=reason, get_chain=lambda self: list(getattr(self, "chain", [])))

    def call_tool(self, tool_name: str, args: str = "") -> str:
        if tool_name not in self.tools:
            return f"error: unknown tool {tool_name}"
        try:
            return str(self.tools[tool_name](args))
        except Exception as e:
            return f"error: {e}"
    put(ToolUse, call_tool=call_tool, get_available_tools=lambda self: sorted(self.tools))

    def mem_store(self, key, value=None):
        """Text form: ``store(text)``.  Vector form: ``store(key_vector, value)`` for retrieval by similarity."""
        if value is None:
            return self.remember(str(key))
        self.__dict__.setdefault("vectors", []).append((torch.as_tensor(key).float().reshape(-1), value))

    def mem_retrieve(self, query, k: int = 5):
        if isinstance(query, str):
            return self.recall(query, k)
        q = torch.as_tensor(query).float().reshape(-1)
        vs = self.__dict__.get("vectors", [])
        sims = [float(torch.nn.functional.cosine_similarity(q, kv, dim=0)) for kv, _ in vs]
        return [vs[i][1] for i in sorted(range(len(vs)), key=lambda i: -sims[i])[:k]]

    def consolidate(self, max_long: int = 1000):
        """Short-term entries move to the long-term store; near-duplicates (difflib ratio > 0.9) are merged."""
        self.long += self.short
        self.short = []
        kept: List[str] = []
        for t in self.long:
            if not any(difflib.SequenceMatcher(None, t, u).ratio() > 0.9 for u in kept[-50:]):
                kept.append(t)
        self.long = kept[-max_long:]
    put(MemorySystem, store=mem_store, retrieve=mem_retrieve, consolidate=consolidate)

    def eh_evaluate(self, benchmark_name: str, n_samples: int = 100) -> dict:
        """Accuracy on a named benchmark: case sets registered with ``register(name, cases)``, else the generated stand-ins
        of the self-evaluation suite."""
        from .self_eval import _builtin_benchmark
        cases = self.__dict__.get("benchmarks", {}).get(benchmark_name) or _builtin_benchmark(benchmark_name, n_samples)
        rep = self.run(cases[:n_samples])
        return {"benchmark": benchmark_name, "accuracy": rep["accuracy"], "samples": len(cases[:n_samples]), "failures": rep["failures"]}

    def eh_register(self, name: str, cases):
        self.__dict__.setdefault("benchmarks", {})[name] = list(cases)

    def evaluate_all(self, n_samples: int = 20):
        names = sorted(self.__dict__.get("benchmarks", {})) or ["mmlu", "arc", "hellaswag", "gsm8k"]
        return [self.evaluate(n, n_samples) for n in names]
    put(EvaluationHarness, evaluate=eh_evaluate, register=eh_register, evaluate_all=evaluate_all)

    def get_no_improvement_count(self) -> int:
        """Iterations at the end of the record whose accuracy did not beat the best before them."""
        n, best = 0, -1.0
        for it in self.iterations:
            n = 0 if it["accuracy"] > best else n + 1
            best = max(best, it["accuracy"])
        return n

    def self_play_for_test(self, cases=None) -> str:
        """One evaluate-and-improve round on a tiny built-in case set; returns a one-line summary."""
        cases = cases or [("2+2", "4"), ("3+5", "8")]
        it = self.run(cases, max_iterations=1)
        return f"iteration {it[-1]['iteration']}: accuracy {it[-1]['accuracy']:.2f}, failures {it[-1]['failures']}" if it else "no iteration ran"
    put(Flywheel, get_history=lambda self: list(self.iterations), get_no_improvement_count=get_no_improvement_count,
        get_log_path=lambda self: getattr(self, "log_path", ""), self_play_for_test=self_play_for_test)


_agi_api()
