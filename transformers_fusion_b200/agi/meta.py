"""Meta-cognition engine: reasoning chains with per-step confidence, confidence calibration (reliability bins, ECE),
goal decomposition with progress tracking, feedback log and self-assessment.
Reference counterpart: include/quant/meta_cognition.h:26-158, src/agi/meta_cognition.cpp."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class ReasoningStep:
    index: int
    content: str
    confidence: float = 1.0
    verified: bool = False


@dataclass
class ReasoningChain:
    goal: str
    steps: List[ReasoningStep] = field(default_factory=list)
    conclusion: str = ""

    def confidence(self):
        c = 1.0
        for s in self.steps:
            c *= s.confidence
        return c if self.steps else 0.0


@dataclass
class CalibrationBin:
    lo: float
    hi: float
    count: int = 0
    mean_confidence: float = 0.0
    accuracy: float = 0.0


@dataclass
class SubGoal:
    id: int
    description: str
    parent: int = -1
    done: bool = False
    weight: float = 1.0


@dataclass
class SelfAssessment:
    calibration_error: float = 0.0
    accuracy: float = 0.0
    overconfidence: float = 0.0
    goals_completed: float = 0.0
    insights: List[str] = field(default_factory=list)


class MetaCognitionEngine:
    def __init__(self, n_bins=10):
        self.records: List[tuple] = []          # (confidence, correct)
        self.n_bins = n_bins
        self.chains: List[ReasoningChain] = []
        self.goals: Dict[int, SubGoal] = {}
        self.feedback: List[dict] = []

    # ---- reasoning
    def begin_chain(self, goal):
        self.chains.append(ReasoningChain(goal))
        return self.chains[-1]

    def add_step(self, chain: ReasoningChain, content, confidence=1.0, verified=False):
        chain.steps.append(ReasoningStep(len(chain.steps), content, confidence, verified))

    def weakest_step(self, chain):
        return min(chain.steps, key=lambda s: s.confidence) if chain.steps else None

    # ---- calibration
    def record_confidence(self, confidence, correct):
        self.records.append((float(confidence), bool(correct)))

    def calibration_bins(self) -> List[CalibrationBin]:
        bins = [CalibrationBin(i / self.n_bins, (i + 1) / self.n_bins) for i in range(self.n_bins)]
        for c, ok in self.records:
            b = bins[min(self.n_bins - 1, int(c * self.n_bins))]
            b.mean_confidence = (b.mean_confidence * b.count + c) / (b.count + 1)
            b.accuracy = (b.accuracy * b.count + float(ok)) / (b.count + 1)
            b.count += 1
        return bins

    def expected_calibration_error(self):
        n = max(1, len(self.records))
        return sum(b.count / n * abs(b.accuracy - b.mean_confidence) for b in self.calibration_bins())

    def calibrate(self, confidence):
        """Map a raw confidence to the accuracy observed in its bin (identity until the bin has data)."""
        b = self.calibration_bins()[min(self.n_bins - 1, int(confidence * self.n_bins))]
        return b.accuracy if b.count >= 5 else confidence

    # ---- goals
    def decompose_goal(self, description, parts: List[str], parent=-1):
        gid = len(self.goals)
        self.goals[gid] = SubGoal(gid, description, parent)
        ids = []
        for p in parts:
            i = len(self.goals)
            self.goals[i] = SubGoal(i, p, gid, weight=1.0 / max(1, len(parts)))
            ids.append(i)
        return gid, ids

    def complete(self, gid):
        self.goals[gid].done = True
        p = self.goals[gid].parent
        if p >= 0 and all(g.done for g in self.goals.values() if g.parent == p):
            self.complete(p)

    def progress(self, gid):
        kids = [g for g in self.goals.values() if g.parent == gid]
        if not kids:
            return float(self.goals[gid].done)
        return sum(g.weight * self.progress(g.id) for g in kids) / sum(g.weight for g in kids)

    # ---- feedback / assessment
    def add_feedback(self, source, text, score):
        self.feedback.append({"source": source, "text": text, "score": float(score), "t": time.time()})

    def assess(self) -> SelfAssessment:
        a = SelfAssessment()
        if self.records:
            a.accuracy = sum(ok for _, ok in self.records) / len(self.records)
            a.calibration_error = self.expected_calibration_error()
            a.overconfidence = sum(c for c, _ in self.records) / len(self.records) - a.accuracy
        roots = [g for g in self.goals.values() if g.parent < 0]
        a.goals_completed = sum(self.progress(g.id) for g in roots) / len(roots) if roots else 0.0
        if a.overconfidence > 0.1:
            a.insights.append("confidence exceeds accuracy: lower stated confidence or verify more steps")
        if self.feedback and sum(f["score"] for f in self.feedback) / len(self.feedback) < 0.5:
            a.insights.append("recent feedback is mostly negative")
        return a


# ---- the reference's verbs (include/quant/meta_cognition.h: MetaCognitionEngine) ---------------------------------------
STRATEGIES = ("DIRECT", "CHAIN_OF_THOUGHT", "DECOMPOSE", "ANALOGY", "VERIFY_THEN_ANSWER")


@dataclass
class FeedbackEntry:
    task: str
    strategy_used: str = "DIRECT"
    performance_score: float = 0.0
    succeeded: bool = False
    failure_reason: str = ""
    duration_ms: int = 0


@dataclass
class GoalDecomposition:
    root: int
    subgoals: List[int] = field(default_factory=list)
    depends_on: Dict[int, List[int]] = field(default_factory=dict)


def _meta_api():
    E = MetaCognitionEngine
    import re

    def task_type_classify(task: str) -> str:
        t = task.lower()
        if re.search(r"\d\s*[-+*/x]\s*\d|solve|calculate|sum|how many", t):
            return "math"
        if re.search(r"\b(code|function|bug|compile|python|implement)\b", t):
            return "code"
        if re.search(r"\b(plan|steps|schedule|organi[sz]e|design)\b", t):
            return "planning"
        if re.search(r"\b(why|explain|because|cause)\b", t):
            return "explanation"
        return "general"

    def analyze_reasoning(self, input_text: str, output_text: str) -> ReasoningChain:
        """Cut an answer into steps (sentences / numbered lines); a step's confidence drops with hedging words and rises
        when the step restates terms of the question; contradictions between consecutive steps are marked."""
        chain = self.begin_chain(input_text)
        parts = [p.strip() for p in re.split(r"(?<=[.!?])\s+|\n+", output_text) if p.strip()]
        q_terms = set(re.findall(r"\w{4,}", input_text.lower()))
        for p in parts:
            hedges = len(re.findall(r"\b(maybe|perhaps|probably|might|guess|unsure|possibly|i think)\b", p.lower()))
            overlap = len(q_terms & set(re.findall(r"\w{4,}", p.lower()))) / max(1, len(q_terms))
            self.add_step(chain, p, max(0.05, min(1.0, 0.75 + 0.25 * overlap - 0.2 * hedges)))
        chain.conclusion = parts[-1] if parts else ""
        self.identify_reasoning_errors(chain)
        return chain

    @staticmethod
    def check_step_consistency(prev: ReasoningStep, curr: ReasoningStep) -> bool:
        """False when the later step negates the earlier one ("x is y" followed by "x is not y") or states a different value
        for the same left-hand side ("x = 3" then "x = 4")."""
        a, b = prev.content.lower(), curr.content.lower()
        strip = lambda s: re.sub(r"\b(not|never|no)\b|n't", "", s)
        if strip(a).split() == strip(b).split() and (("not" in b.split() or "n't" in b or "never" in b.split()) != ("not" in a.split() or "n't" in a or "never" in a.split())):
            return False
        ea, eb = re.findall(r"(\w+)\s*=\s*(-?\d+(?:\.\d+)?)", a), dict(re.findall(r"(\w+)\s*=\s*(-?\d+(?:\.\d+)?)", b))
        return not any(k in eb and eb[k] != v for k, v in ea)

    def calculate_chain_consistency(self, chain: ReasoningChain) -> float:
        """Share of the steps after the first that contradict none of the steps before them."""
        if len(chain.steps) < 2:
            return 1.0
        ok = sum(all(self.check_step_consistency(a, b) for a in chain.steps[:i]) for i, b in enumerate(chain.steps) if i)
        return ok / (len(chain.steps) - 1)

    def identify_reasoning_errors(self, chain: ReasoningChain):
        """Mark every step that contradicts an earlier one (``verified`` False, confidence halved, the earlier step named)."""
        for i, b in enumerate(chain.steps):
            if getattr(b, "error", ""):
                continue
            for a in chain.steps[:i]:
                if not self.check_step_consistency(a, b):
                    b.verified, b.confidence = False, b.confidence * 0.5
                    b.error = f"contradicts step {a.index}"
                    break

    @staticmethod
    def find_first_error_step(chain: ReasoningChain) -> int:
        return next((s.index for s in chain.steps if getattr(s, "error", "")), -1)

    def diagnose_error(self, chain: ReasoningChain, error_step: int) -> str:
        if not 0 <= error_step < len(chain.steps):
            return "no error step"
        s = chain.steps[error_step]
        why = getattr(s, "error", "") or ("low confidence" if s.confidence < 0.5 else "no inconsistency found")
        return f"step {error_step} ({s.content[:60]!r}): {why}; later steps that build on it should be re-derived"

    # calibration with the reference's names
    def _record(self, predicted, correct, task=""):
        self.records.append((float(predicted), bool(correct)))
        self.__dict__.setdefault("conf_tasks", []).append(task)

    def get_expected_calibration_error(self): return self.expected_calibration_error()

    def get_calibration_bins(self, num_bins: int = 10):
        old, self.n_bins = self.n_bins, num_bins
        try:
            return self.calibration_bins()
        finally:
            self.n_bins = old

    def get_current_confidence(self) -> float:
        """Mean stated confidence over the last 20 records, mapped through the calibration curve."""
        last = [c for c, _ in self.records[-20:]]
        return self.calibrate(sum(last) / len(last)) if last else 0.5

    def get_confidence_history(self): return list(self.records)
    def get_history(self): return list(self.chains)

    # goals
    def decompose(self, goal: str, max_subgoals: int = 20) -> GoalDecomposition:
        """Split a goal stated in text into sequential subgoals (each depends on the one before it)."""
        parts = [p.strip() for p in re.split(r"\s*(?:;|\.|,? and then |,? then |\n)\s*", goal) if p.strip()][:max_subgoals]
        root, ids = self.decompose_goal(goal, parts or [goal])
        return GoalDecomposition(root, ids, {i: ([ids[k - 1]] if k else []) for k, i in enumerate(ids)})

    def check_subgoal_completion(self, decomp: GoalDecomposition) -> bool:
        return all(self.goals[i].done for i in decomp.subgoals)

    def get_ready_subgoals(self, decomp: GoalDecomposition) -> List[int]:
        return [i for i in decomp.subgoals if not self.goals[i].done and all(self.goals[d].done for d in decomp.depends_on.get(i, []))]

    # strategies and feedback
    def record_feedback(self, entry: FeedbackEntry):
        self.__dict__.setdefault("entries", []).append(entry)
        self.add_feedback(entry.strategy_used, entry.failure_reason or entry.task, entry.performance_score)

    def get_recent_feedback(self, count: int = 50): return list(self.__dict__.get("entries", []))[-count:]

    def get_best_strategy_for_task_type(self, task_type: str) -> str:
        """The strategy with the best mean score on this type of task so far (DIRECT without evidence)."""
        score: Dict[str, List[float]] = {}
        for e in self.__dict__.get("entries", []):
            if task_type_classify(e.task) == task_type:
                score.setdefault(e.strategy_used, []).append(e.performance_score)
        return max(score, key=lambda k: sum(score[k]) / len(score[k])) if score else "DIRECT"

    def select_strategy(self, task: str, difficulty: float = 0.5) -> str:
        """Evidence first (the best recorded strategy for this type of task); otherwise by type and difficulty."""
        tt = task_type_classify(task)
        best = self.get_best_strategy_for_task_type(tt)
        if best != "DIRECT" or any(task_type_classify(e.task) == tt for e in self.__dict__.get("entries", [])):
            return best
        if difficulty >= 0.75:
            return "DECOMPOSE"
        if tt in ("math", "code"):
            return "VERIFY_THEN_ANSWER" if difficulty >= 0.5 else "CHAIN_OF_THOUGHT"
        return "CHAIN_OF_THOUGHT" if difficulty >= 0.4 else "DIRECT"

    def generate_feedback_summary(self) -> str:
        es = self.__dict__.get("entries", [])
        if not es:
            return "no feedback recorded"
        ok = sum(e.succeeded for e in es)
        by = {}
        for e in es:
            by.setdefault(e.strategy_used, []).append(e.performance_score)
        lines = [f"{len(es)} tasks, {ok} succeeded ({100 * ok / len(es):.0f}%)"]
        lines += [f"  {k}: mean score {sum(v) / len(v):.2f} over {len(v)}" for k, v in sorted(by.items())]
        return "\n".join(lines)

    def extract_improvement_patterns(self) -> List[str]:
        """Failure reasons that repeat, most frequent first, and strategies that fail more often than they succeed."""
        es = self.__dict__.get("entries", [])
        reasons: Dict[str, int] = {}
        for e in es:
            if not e.succeeded and e.failure_reason:
                reasons[e.failure_reason] = reasons.get(e.failure_reason, 0) + 1
        out = [f"recurring failure: {r} (x{n})" for r, n in sorted(reasons.items(), key=lambda kv: -kv[1]) if n >= 2]
        for s in sorted({e.strategy_used for e in es}):
            mine = [e for e in es if e.strategy_used == s]
            if len(mine) >= 2 and sum(e.succeeded for e in mine) * 2 < len(mine):
                out.append(f"strategy {s} fails more often than it succeeds")
        return out

    def assess_self(self, lookback_count: int = 100) -> SelfAssessment:
        keep = self.records
        self.records = keep[-lookback_count:]
        try:
            a = self.assess()
        finally:
            self.records = keep
        a.insights += self.extract_improvement_patterns()
        return a

    def generate_insight(self, task: str, result: str) -> dict:
        chain = self.analyze_reasoning(task, result)
        first = self.find_first_error_step(chain)
        return {"task_type": task_type_classify(task), "chain_confidence": chain.confidence(), "consistency": self.calculate_chain_consistency(chain),
                "first_error_step": first, "diagnosis": self.diagnose_error(chain, first) if first >= 0 else "",
                "suggested_strategy": self.select_strategy(task, 1.0 - chain.confidence())}

    def reset(self):
        self.records, self.chains, self.goals, self.feedback = [], [], {}, []
        self.entries, self.conf_tasks = [], []

    E.task_type_classify = staticmethod(task_type_classify)
    orig_record = E.record_confidence
    E.record_confidence = lambda self, predicted, correct, task="": _record(self, predicted, correct, task)
    for name, fn in list(locals().items()):
        if name not in ("E", "re", "task_type_classify", "orig_record", "_record") and not name.startswith("_") and (callable(fn) or isinstance(fn, staticmethod)):
            setattr(E, name, fn)


_meta_api()
