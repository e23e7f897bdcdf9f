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
