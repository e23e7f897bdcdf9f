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


# ---- the reference's verbs (include/quant/multi_agent.h: MultiAgentSystem) ---------------------------------------------
@dataclass
class ProposalVote:
    agent_id: int
    proposal: str
    approve: bool
    confidence: float = 1.0
    rationale: str = ""


@dataclass
class HierarchicalPlan:
    goal: str
    high_level_steps: List[str] = field(default_factory=list)
    subtask_ids: List[int] = field(default_factory=list)
    completed: bool = False
    overall_progress: float = 0.0


def _mas_api():
    M = MultiAgentSystem
    TOPOLOGIES = ("STAR", "RING", "FULL")

    def configure(self, topology: str = "STAR"):
        """Who may talk to whom directly: STAR (everyone with agent 0), RING (neighbours by id), FULL."""
        topology = topology.upper()
        assert topology in TOPOLOGIES, topology
        self.topology = topology

    def _connected(self, a: int, b: int) -> bool:
        topo, ids = getattr(self, "topology", "FULL"), sorted(self.agents)
        if topo == "FULL" or a == b:
            return True
        if topo == "STAR":
            return a == ids[0] or b == ids[0]
        ia, ib = ids.index(a), ids.index(b)
        return abs(ia - ib) in (1, len(ids) - 1)

    def set_max_queue_size(self, n: int): self.max_queue = int(n)
    def set_communication_delay(self, delay_ms: int): self.delay_ms = int(delay_ms)
    def agent_count(self) -> int: return len(self.agents)
    def get_agent(self, agent_id: int): return self.agents[agent_id]

    def remove_agent(self, agent_id: int):
        """The agent leaves; its unfinished subtasks return to the pool."""
        self.agents.pop(agent_id, None)
        self.inboxes.pop(agent_id, None)
        for s in self.subtasks.values():
            if s.assigned_to == agent_id and not s.done:
                s.assigned_to = -1

    def send_message(self, msg: AgentMessage) -> bool:
        """Deliver along the topology (a message between unconnected agents is relayed through agent 0 in a star and is
        refused otherwise); a full inbox drops its oldest message."""
        if msg.receiver not in self.inboxes or msg.sender not in self.agents:
            return False
        if not _connected(self, msg.sender, msg.receiver):
            return False
        if getattr(self, "delay_ms", 0):
            msg.timestamp += self.delay_ms / 1e3                    # delivery time, for receivers that order by it
        box = self.inboxes[msg.receiver]
        box.append(msg)
        while len(box) > getattr(self, "max_queue", 1 << 30):
            box.pop(0)
        self.agents[msg.sender].metrics.messages_sent += 1
        self.__dict__.setdefault("history", []).append(f"{msg.sender}->{msg.receiver} [{msg.topic}] {msg.content}")
        return True

    def communicate_direct(self, sender: int, receiver: int, content: str) -> bool:
        return self.send_message(AgentMessage(sender, receiver, "direct", content))

    def receive_messages(self, agent_id: int) -> List[AgentMessage]:
        out, self.inboxes[agent_id] = self.inboxes.get(agent_id, []), []
        return out

    def get_histories(self) -> List[str]:
        return list(self.__dict__.get("history", []))

    # ---- tasks
    def assign_task(self, agent_id: int, task: str) -> int:
        i = self.add_subtask(task)
        self.subtasks[i].assigned_to = agent_id
        return i

    def assign_task_to_role(self, role: str, task: str) -> int:
        i = self.add_subtask(task)
        cands = [a for a in self.agents.values() if a.role == role]
        if cands:
            self.subtasks[i].assigned_to = min(cands, key=lambda a: sum(1 for s in self.subtasks.values() if s.assigned_to == a.id and not s.done)).id
        return i

    def get_task_status(self, task_id: int) -> str:
        s = self.subtasks.get(task_id)
        if s is None:
            return "unknown"
        return "done" if s.done else ("failed" if s.result.startswith("error:") and s.assigned_to < 0 else ("assigned" if s.assigned_to >= 0 else "pending"))

    def decompose_task(self, complex_task: str, max_subtasks: int = 5) -> List[int]:
        """Split on sentence / clause boundaries ("then", ";", ".", " and then ") into a chain of dependent subtasks; a
        planner agent (role "planner"), when present, does the splitting instead."""
        import re
        planner = next((a.id for a in self.agents.values() if a.role == "planner"), None)
        if planner is not None:
            return self.hierarchical_plan(complex_task, planner, max_subtasks)
        parts = [p.strip() for p in re.split(r"\s*(?:;|\.|,? and then |,? then )\s*", complex_task) if p.strip()][:max_subtasks]
        prev, ids = None, []
        for p in parts or [complex_task]:
            prev = self.add_subtask(p, [prev] if prev is not None else [])
            ids.append(prev)
        return ids

    def get_subtasks(self) -> List[Subtask]:
        return [self.subtasks[i] for i in sorted(self.subtasks)]

    def assign_subtask(self, subtask_id: int, agent_id: int):
        self.subtasks[subtask_id].assigned_to = agent_id

    def get_ready_subtasks(self) -> List[Subtask]:
        return [s for s in self.get_subtasks() if not s.done and all(self.subtasks[d].done for d in s.depends_on)]

    # ---- votes on proposals
    def submit_vote(self, agent_id: int, proposal: str, approve: bool, confidence: float = 1.0, rationale: str = ""):
        self.__dict__.setdefault("votes", []).append(ProposalVote(agent_id, proposal, bool(approve), float(confidence), rationale))

    def get_votes(self) -> List[ProposalVote]:
        return list(self.__dict__.get("votes", []))

    def reset_votes(self):
        self.votes = []

    def check_consensus(self, threshold: float = 0.6) -> bool:
        """Confidence- and weight-weighted share of approvals among the votes cast reaches the threshold."""
        vs = self.get_votes()
        if not vs:
            return False
        w = lambda v: v.confidence * (self.agents[v.agent_id].weight if v.agent_id in self.agents else 1.0)
        tot = sum(w(v) for v in vs)
        return tot > 0 and sum(w(v) for v in vs if v.approve) / tot >= threshold

    # ---- blackboard
    def write_blackboard(self, key: str, value: str, agent_id: int): self.post(agent_id, key, value)
    def read_blackboard(self, key: str): return self.read(key) or ""

    def search_blackboard(self, prefix: str) -> List[BlackboardEntry]:
        return [e for k, e in sorted(self.blackboard.items()) if k.startswith(prefix)]

    def cleanup_blackboard(self, keep_prefixes=("plan/",)):
        """Drop the results of finished subtasks (and anything else not under a kept prefix)."""
        self.blackboard = {k: e for k, e in self.blackboard.items() if any(k.startswith(p) for p in keep_prefixes)}

    # ---- plans and supervision
    def create_plan(self, goal: str, max_subtasks: int = 5) -> HierarchicalPlan:
        ids = self.decompose_task(goal, max_subtasks)
        plan = HierarchicalPlan(goal, [self.subtasks[i].description for i in ids], ids)
        self.post(-1, f"plan/{goal[:40]}", "; ".join(plan.high_level_steps))
        return plan

    def get_plan_progress(self, plan: HierarchicalPlan) -> float:
        return sum(self.subtasks[i].done for i in plan.subtask_ids) / max(1, len(plan.subtask_ids))

    def execute_plan(self, plan: HierarchicalPlan, max_rounds: int = 10) -> bool:
        for _ in range(max_rounds):
            self.assign()
            self.supervisor_monitor()
            if self.step() == 0:
                break
        plan.overall_progress = self.get_plan_progress(plan)
        plan.completed = plan.overall_progress == 1.0
        return plan.completed

    def supervisor_monitor(self) -> List[int]:
        """Subtasks that failed and lost their agent are handed out again; returns their ids."""
        failed = [s.id for s in self.subtasks.values() if not s.done and s.assigned_to < 0 and s.result.startswith("error:")]
        for i in failed:
            self.supervisor_reassign_failed(i)
        return failed

    def supervisor_reassign_failed(self, subtask_id: int):
        """To the agent with the best record that has not just failed it (fewest failures, then least load)."""
        s = self.subtasks[subtask_id]
        tried = self.__dict__.setdefault("_tried", {}).setdefault(subtask_id, set())
        cands = [a for a in self.agents.values() if a.id not in tried] or list(self.agents.values())
        if not cands:
            return
        load = lambda a: sum(1 for t in self.subtasks.values() if t.assigned_to == a.id and not t.done)
        a = min(cands, key=lambda a: (a.metrics.tasks_failed, load(a), a.id))
        tried.add(a.id)
        s.assigned_to, s.result = a.id, ""

    def supervisor_resolve_conflicts(self) -> List[str]:
        """Blackboard keys written more than once: the last writer wins (that is what the board already holds); the keys
        are reported so that the supervisor can look at them."""
        return sorted(k for k, e in self.blackboard.items() if e.version > 1)

    def supervisor_escalate(self, issue: str):
        self.__dict__.setdefault("escalations", []).append(issue)
        self.post(-1, f"escalation/{len(self.escalations)}", issue)

    # ---- metrics and driving loops
    def update_metrics(self, agent_id: int):
        a = self.agents[agent_id]
        a.busy = any(s.assigned_to == agent_id and not s.done for s in self.subtasks.values())

    def get_metrics(self, agent_id: int) -> AgentMetrics: return self.agents[agent_id].metrics
    def get_all_metrics(self) -> List[AgentMetrics]: return [self.agents[i].metrics for i in sorted(self.agents)]

    def metrics_summary(self) -> str:
        return "\n".join(f"agent {a.id} ({a.role}): done {a.metrics.tasks_completed}, failed {a.metrics.tasks_failed}, "
                          f"messages {a.metrics.messages_sent}, busy {a.metrics.total_time_s:.3f}s" for a in self.agents.values())

    def run_round(self, max_rounds: int = 10) -> bool:
        return self.run(max_rounds)

    def run_episode(self, steps: int) -> int:
        """``steps`` assign-and-work rounds regardless of progress; returns how many subtask runs happened."""
        ran = 0
        for _ in range(steps):
            self.assign()
            self.supervisor_monitor()
            ran += self.step()
        return ran

    for name, fn in list(locals().items()):
        if callable(fn) and name not in ("M",) and not name.startswith("_"):
            setattr(M, name, fn)


_mas_api()
