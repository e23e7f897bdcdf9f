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


# ---- the reference's verbs on the tabular model (include/quant/world_model.h: WorldModel) -------------------------------
@dataclass
class Transition:
    state: Hashable
    action: Hashable
    next_state: Hashable
    reward: float = 0.0


@dataclass
class UncertaintyEstimate:
    epistemic_uncertainty: float = 0.0
    aleatoric_uncertainty: float = 0.0
    total_uncertainty: float = 0.0
    ensemble_size: int = 0
    disagreement_magnitude: float = 0.0


def _wm_api():
    W = WorldModel

    def add_transition(self, t: Transition):
        self.observe(t.state, t.action, t.next_state, t.reward)
        st = self.__dict__.setdefault("_st", {"predictions": 0, "planning_calls": 0, "planning_ms": 0.0, "err": 0.0, "err_n": 0})
        return st

    update_transition_model = add_transition

    def train_on_transitions(self, transitions, epochs: int = 1):
        """Counts need one pass; ``epochs`` is accepted for signature parity."""
        for t in transitions:
            self.add_transition(t)

    def get_transition_buffer(self):
        return [Transition(*m) for m in self.memory]

    def simulate_step(self, state, action):
        """Most likely next state (the state itself when the pair was never seen)."""
        return self.predict(state, action).next_state

    def predict_reward(self, state, action) -> float:
        self._count("predictions")
        return self.predict(state, action).expected_reward

    def simulate_trajectory(self, start_state, actions):
        out, s = [], start_state
        for a in actions:
            pr = self.predict(s, a)
            if pr.probability == 0.0:
                break
            out.append(Transition(s, a, pr.next_state, pr.expected_reward))
            s = pr.next_state
        return out

    def _count(self, key, inc=1):
        st = self.__dict__.setdefault("_st", {"predictions": 0, "planning_calls": 0, "planning_ms": 0.0, "err": 0.0, "err_n": 0})
        st[key] += inc

    def estimate_uncertainty(self, state, action, ensemble_size: int = 5) -> UncertaintyEstimate:
        """Epistemic part from the visit count, aleatoric part from the transition entropy; the "ensemble" is
        ``ensemble_size`` bootstrap resamples of the observed next states, whose disagreement is reported."""
        import random
        ep, al = self.uncertainty(state, action)
        c = self.counts.get((state, action)) or {}
        pool = [s for s, n in c.items() for _ in range(n)]
        rng = random.Random(hash((state, action)) & 0xFFFF)
        votes = [max(set(smp), key=smp.count) for smp in ([rng.choice(pool) for _ in pool] for _ in range(ensemble_size))] if pool else []
        dis = self.compute_ensemble_disagreement(votes)
        al = 0.0 if math.isinf(al) else al
        return UncertaintyEstimate(ep, al, ep + al, ensemble_size if pool else 0, dis)

    def compute_ensemble_disagreement(self, predictions) -> float:
        """1 - share of the most common prediction (0 = all members agree)."""
        preds = list(predictions)
        if not preds:
            return 0.0
        return 1.0 - max(preds.count(p) for p in set(preds)) / len(preds)

    def predict_with_uncertainty(self, state, action):
        self._count("predictions")
        return self.predict(state, action), self.estimate_uncertainty(state, action)

    def beam_search_plan(self, current_state, horizon: int, beam_width: int = 10, n_actions: int = 10) -> MPCPlan:
        import time
        t0 = time.perf_counter()
        p = self.plan_beam(current_state, horizon, beam_width)
        self._count("planning_calls")
        self._count("planning_ms", (time.perf_counter() - t0) * 1e3)
        return p

    def model_predictive_control(self, current_state, horizon: int, n_samples: int = 50) -> MPCPlan:
        """Random-shooting MPC: ``n_samples`` action sequences are rolled out in the model, the best one is returned
        (its first action is what a controller executes before planning again)."""
        import random
        import time
        t0 = time.perf_counter()
        rng = random.Random(len(self.memory))
        acts = sorted(self.actions, key=repr)
        best = MPCPlan([], -float("inf"), [current_state])
        for _ in range(n_samples if acts else 0):
            seq = [rng.choice(acts) for _ in range(horizon)]
            ret, states = self.rollout_return(current_state, seq)
            if ret > best.expected_return:
                best = MPCPlan(seq[: len(states) - 1], ret, states)
        self._count("planning_calls")
        self._count("planning_ms", (time.perf_counter() - t0) * 1e3)
        return best if best.actions else MPCPlan([], 0.0, [current_state])

    def plan_actions(self, current_state, horizon: int):
        return self.beam_search_plan(current_state, horizon).actions

    def plan(self, horizon: int):
        """Planned states from the current state."""
        return self.beam_search_plan(self.get_current_state(), horizon).states

    def counterfactual_analysis(self, actual_state, actual_action, counterfactual_action) -> CounterfactualResult:
        return self.counterfactual(actual_state, [actual_action], [counterfactual_action])

    def batch_counterfactual(self, state, actual_action, alternatives):
        return [self.counterfactual_analysis(state, actual_action, a) for a in alternatives]

    # ---- state memory: keyed states with importance and access counts
    def store_state(self, state, importance: float = 1.0, key=None, vector=None):
        mem = self.__dict__.setdefault("_states", [])
        mem.append({"state": state, "key": key if key is not None else repr(state), "vector": list(vector) if vector is not None else None,
                    "importance_weight": float(importance), "access_count": 0, "last_accessed": len(mem)})

    def get_memory(self):
        return self.__dict__.setdefault("_states", [])

    def retrieve_most_relevant(self, query):
        """By key (a string: longest common prefix, then importance) or by vector (cosine similarity)."""
        mem = self.get_memory()
        if not mem:
            return None
        if isinstance(query, str):
            def score(e):
                k, n = e["key"], 0
                while n < min(len(k), len(query)) and k[n] == query[n]:
                    n += 1
                return (n, e["importance_weight"])
        else:
            q = list(query)
            qn = math.sqrt(sum(x * x for x in q)) or 1.0

            def score(e):
                v = e["vector"]
                if v is None:
                    return (-1.0, e["importance_weight"])
                vn = math.sqrt(sum(x * x for x in v)) or 1.0
                return (sum(a * b for a, b in zip(q, v)) / (qn * vn), e["importance_weight"])
        best = max(mem, key=score)
        best["access_count"] += 1
        best["last_accessed"] = self.__dict__["_clock"] = self.__dict__.get("_clock", 0) + 1
        return best["state"]

    def consolidate_memory(self, target_size: int = 1000):
        """Keep the ``target_size`` entries with the highest importance x (1 + accesses)."""
        mem = self.get_memory()
        mem.sort(key=lambda e: -(e["importance_weight"] * (1 + e["access_count"])))
        del mem[target_size:]

    def get_current_state(self):
        return self.__dict__.get("_current")

    def set_current_state(self, state):
        self._current = state

    def get_stats(self) -> dict:
        st = self.__dict__.setdefault("_st", {"predictions": 0, "planning_calls": 0, "planning_ms": 0.0, "err": 0.0, "err_n": 0})
        return {"total_transitions": sum(self.visits.values()), "total_predictions": st["predictions"],
                "memory_entries": len(self.get_memory()), "planning_calls": st["planning_calls"],
                "avg_planning_time_ms": st["planning_ms"] / max(1, st["planning_calls"])}

    def reset_stats(self):
        self._st = {"predictions": 0, "planning_calls": 0, "planning_ms": 0.0, "err": 0.0, "err_n": 0}

    for name, fn in list(locals().items()):
        if callable(fn) and name != "W":
            setattr(W, name, fn)


_wm_api()
