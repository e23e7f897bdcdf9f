"""Multi-agent system: agents with roles and metrics, a shared blackboard, direct messages, subtask assignment by load,
weighted voting and a hierarchical plan.  Reference counterpart: include/quant/multi_agent.h:47-201, src/agi/multi_agent.cpp."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


@dataclass
class AgentMessage:
    sender: int
    receiver: int
    topic: str
    content: str
    timestamp: float = field(default_factory=time.time)


@dataclass
class Subtask:
    id: int
    description: str
    assigned_to: int = -1
    done: bool = False
    result: str = ""
    depends_on: List[int] = field(default_factory=list)


@dataclass
class AgentMetrics:
    tasks_completed: int = 0
    tasks_failed: int = 0
    messages_sent: int = 0
    total_time_s: float = 0.0


@dataclass
class AgentState:
    id: int
    role: str
    fn: Callable[[str], str]
    weight: float = 1.0
    busy: bool = False
    metrics: AgentMetrics = field(default_factory=AgentMetrics)


@dataclass
class BlackboardEntry:
    key: str
    value: str
    author: int
    version: int = 1


@dataclass
class Vote:
    agent: int
    option: str
    weight: float = 1.0


class MultiAgentSystem:
    def __init__(self):
        self.agents: Dict[int, AgentState] = {}
        self.blackboard: Dict[str, BlackboardEntry] = {}
        self.inboxes: Dict[int, List[AgentMessage]] = {}
        self.subtasks: Dict[int, Subtask] = {}

    def add_agent(self, role, fn, weight=1.0) -> int:
        i = len(self.agents)
        self.agents[i] = AgentState(i, role, fn, weight)
        self.inboxes[i] = []
        return i

    # ---- communication
    def send(self, sender, receiver, topic, content):
        self.inboxes[receiver].append(AgentMessage(sender, receiver, topic, content))
        self.agents[sender].metrics.messages_sent += 1

    def broadcast(self, sender, topic, content):
        for r in self.agents:
            if r != sender:
                self.send(sender, r, topic, content)

    def receive(self, agent, topic=None):
        box = self.inboxes[agent]
        for i, m in enumerate(box):
            if topic is None or m.topic == topic:
                return box.pop(i)
        return None

    def post(self, author, key, value):
        e = self.blackboard.get(key)
        self.blackboard[key] = BlackboardEntry(key, value, author, e.version + 1 if e else 1)

    def read(self, key):
        e = self.blackboard.get(key)
        return e.value if e else None

    # ---- work
    def add_subtask(self, description, depends_on=()):
        i = len(self.subtasks)
        self.subtasks[i] = Subtask(i, description, depends_on=list(depends_on))
        return i

    def assign(self, role: Optional[str] = None):
        """Give every unassigned, ready subtask to the least loaded agent (of ``role`` when given)."""
        load = {a.id: sum(1 for s in self.subtasks.values() if s.assigned_to == a.id and not s.done) for a in self.agents.values()}
        for s in self.subtasks.values():
            if s.assigned_to >= 0 or s.done or not all(self.subtasks[d].done for d in s.depends_on):
                continue
            cands = [a for a in self.agents.values() if role is None or a.role == role]
            if not cands:
                continue
            a = min(cands, key=lambda x: load[x.id])
            s.assigned_to = a.id
            load[a.id] += 1

    def step(self):
        """Run every assigned, unfinished subtask once; results go to the blackboard under 'subtask/<id>'."""
        ran = 0
        for s in self.subtasks.values():
            if s.assigned_to < 0 or s.done:
                continue
            a = self.agents[s.assigned_to]
            t0 = time.perf_counter()
            try:
                ctx = " | ".join(self.subtasks[d].result for d in s.depends_on)
                s.result = a.fn(s.description + (f" (given: {ctx})" if ctx else ""))
                s.done = True
                a.metrics.tasks_completed += 1
                self.post(a.id, f"subtask/{s.id}", s.result)
            except Exception as e:
                a.metrics.tasks_failed += 1
                s.assigned_to = -1                      # goes back to the pool
                s.result = f"error: {e}"
            a.metrics.total_time_s += time.perf_counter() - t0
            ran += 1
        return ran

    def run(self, max_rounds=10):
        for _ in range(max_rounds):
            self.assign()
            if self.step() == 0:
                break
        return all(s.done for s in self.subtasks.values())

    # ---- decisions
    def vote(self, question: str, options: List[str]):
        votes = []
        for a in self.agents.values():
            ans = a.fn(f"{question} Options: {', '.join(options)}")
            pick = next((o for o in options if o.lower() in ans.lower()), None)
            if pick:
                votes.append(Vote(a.id, pick, a.weight))
        tally = {o: sum(v.weight for v in votes if v.option == o) for o in options}
        return max(tally, key=tally.get), tally, votes

    def hierarchical_plan(self, goal, planner: int, max_parts=5):
        text = self.agents[planner].fn(f"Split into at most {max_parts} parts, one per line: {goal}")
        parts = [l.strip("-*0123456789. ").strip() for l in text.splitlines() if l.strip()][:max_parts]
        prev, ids = None, []
        for p in parts:
            prev = self.add_subtask(p, [prev] if prev is not None else [])
            ids.append(prev)
        return ids
