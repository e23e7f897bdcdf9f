"""Tabular world model over symbolic states: transition counts with Laplace smoothing, next-state / reward prediction with
uncertainty, beam planning, model-predictive control, counterfactual queries and a bounded state memory.
Reference counterpart: include/quant/world_model.h:20-177, src/agi/world_model.cpp."""
from __future__ import annotations

import math
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Sequence, Tuple


@dataclass
class PredictionResult:
    next_state: Hashable
    probability: float
    expected_reward: float
    entropy: float


@dataclass
class MPCPlan:
    actions: List[Hashable]
    expected_return: float
    states: List[Hashable]


@dataclass
class CounterfactualResult:
    factual_return: float
    counterfactual_return: float
    difference: float


class WorldModel:
    def __init__(self, discount=0.95, memory_size=4096):
        self.counts: Dict[Tuple, Dict[Hashable, int]] = defaultdict(lambda: defaultdict(int))
        self.reward_sum: Dict[Tuple, float] = defaultdict(float)
        self.visits: Dict[Tuple, int] = defaultdict(int)
        self.actions = set()
        self.gamma = discount
        self.memory: List[Tuple] = []
        self.memory_size = memory_size

    def observe(self, state, action, next_state, reward=0.0):
        k = (state, action)
        self.counts[k][next_state] += 1
        self.reward_sum[k] += reward
        self.visits[k] += 1
        self.actions.add(action)
        self.memory.append((state, action, next_state, reward))
        if len(self.memory) > self.memory_size:
            self.memory.pop(0)

    def distribution(self, state, action) -> Dict[Hashable, float]:
        c = self.counts.get((state, action))
        if not c:
            return {}
        tot = sum(c.values())
        return {s: n / tot for s, n in c.items()}

    def predict(self, state, action) -> PredictionResult:
        d = self.distribution(state, action)
        if not d:
            return PredictionResult(state, 0.0, 0.0, float("inf"))
        s, p = max(d.items(), key=lambda kv: kv[1])
        ent = -sum(q * math.log(q) for q in d.values())
        return PredictionResult(s, p, self.reward_sum[(state, action)] / self.visits[(state, action)], ent)

    def uncertainty(self, state, action):
        """(epistemic ~ 1/sqrt(visits), aleatoric = transition entropy)."""
        n = self.visits.get((state, action), 0)
        return 1.0 / math.sqrt(1 + n), (self.predict(state, action).entropy if n else float("inf"))

    def rollout_return(self, state, actions: Sequence) -> Tuple[float, List]:
        total, g, states = 0.0, 1.0, [state]
        for a in actions:
            pr = self.predict(state, a)
            if pr.probability == 0.0:
                break
            total += g * pr.expected_reward
            g *= self.gamma
            state = pr.next_state
            states.append(state)
        return total, states

    def plan_beam(self, state, horizon=5, beam=8) -> MPCPlan:
        beams = [([], 0.0, state, 1.0)]
        for _ in range(horizon):
            nxt = []
            for acts, ret, s, g in beams:
                for a in self.actions:
                    pr = self.predict(s, a)
                    if pr.probability > 0:
                        nxt.append((acts + [a], ret + g * pr.expected_reward, pr.next_state, g * self.gamma))
            if not nxt:
                break
            beams = sorted(nxt, key=lambda b: -b[1])[:beam]
        acts, ret, _, _ = max(beams, key=lambda b: b[1])
        return MPCPlan(acts, ret, self.rollout_return(state, acts)[1])

    def mpc_action(self, state, horizon=5, beam=8):
        p = self.plan_beam(state, horizon, beam)
        return p.actions[0] if p.actions else None

    def counterfactual(self, state, factual_actions, alternative_actions) -> CounterfactualResult:
        f, _ = self.rollout_return(state, factual_actions)
        c, _ = self.rollout_return(state, alternative_actions)
        return CounterfactualResult(f, c, c - f)

    def stats(self):
        return {"state_action_pairs": len(self.visits), "transitions": sum(self.visits.values()), "actions": len(self.actions),
                "memory": len(self.memory)}
