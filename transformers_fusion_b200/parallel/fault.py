"""Failure detection and elastic recovery, all on the host.

* ``Heartbeat``               - a watchdog thread per rank that stamps ``hb/<rank>`` in a key-value store (the
  ``torch.distributed`` TCP store, or any object with set/get) every ``interval`` and reports peers whose stamp is older
  than ``fault_timeout`` (defaults 1 s / 5 s as in the reference's ClusterConfig).
* ``FaultToleranceManager``   - node table, ``on_node_failure`` / ``on_node_recovery`` callbacks, counters and the text
  checkpoint ``nodes:N;failed:N;failed_node{id};node{id,addr,port,ne};stats{routed=,dropped=,failures=}``.
* ``redistribute_experts``    - contiguous re-assignment of experts over the surviving ranks.
* ``reshard_flat``            - elastic restart: re-cut a flat ZeRO / FSDP state (one shard per old rank) for a new world size.
* ``device_wait_status``      - reads the device status word that every bounded wait in the kernels writes on expiry, so a
  stuck peer shows up as an error code on the host instead of a hung GPU.
* ``FaultInjector``           - host-side injection only: drop / delay control-plane messages, skip posting a flag,
  raise in a rank, truncate a file.  Nothing here makes a GPU fault.

Reference counterparts: expert::FaultToleranceManager (src/model/expert_parallel.cpp:1058-1234), ExpertParallelManager
handle_node_failure / redistribute_experts_after_failure / compute_redistribution (:835-868,1479), ClusterConfig
(include/quant/expert_parallel.h:61-76)."""
from __future__ import annotations

import os
import random
import re
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch


@dataclass
class ClusterConfig:
    heartbeat_interval_ms: int = 1000
    fault_timeout_ms: int = 5000
    max_retries: int = 3
    num_experts: int = 0


class DictStore:
    """In-process stand-in for the TCP store (tests, single process)."""

    def __init__(self):
        self.d, self.lock = {}, threading.Lock()

    def set(self, k, v):
        with self.lock:
            self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        with self.lock:
            return self.d[k]

    def check(self, keys):
        with self.lock:
            return all(k in self.d for k in keys)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, fault_timeout_s: float = 5.0,
                 on_failure: Optional[Callable[[int], None]] = None, on_recovery: Optional[Callable[[int], None]] = None,
                 clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout = interval_s, fault_timeout_s
        self.on_failure, self.on_recovery, self.clock = on_failure, on_recovery, clock
        self.failed = set()
        self._stop = threading.Event()
        self._thread = None
        self.paused = False                     # fault injection: a rank that stops beating

    def beat(self):
        if not self.paused:
            self.store.set(f"hb/{self.rank}", repr(self.clock()))

    def check_peers(self) -> List[int]:
        """Ranks whose last beat is older than the timeout (or that never beat)."""
        now = self.clock()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                ok = self.store.check([f"hb/{r}"]) if hasattr(self.store, "check") else True
                last = float(self.store.get(f"hb/{r}").decode()) if ok else -1e30
            except Exception:
                last = -1e30
            if now - last > self.timeout:
                dead.append(r)
        for r in dead:
            if r not in self.failed:
                self.failed.add(r)
                if self.on_failure:
                    self.on_failure(r)
        for r in list(self.failed):
            if r not in dead:
                self.failed.discard(r)
                if self.on_recovery:
                    self.on_recovery(r)
        return dead

    def start(self):
        def loop():
            while not self._stop.wait(self.interval):
                self.beat()
                self.check_peers()
        self.beat()
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2 * self.interval + 1)


@dataclass
class NodeInfo:
    id: int
    addr: str = "127.0.0.1"
    port: int = 0
    num_experts: int = 0
    alive: bool = True


class FaultToleranceManager:
    def __init__(self, cfg: Optional[ClusterConfig] = None):
        self.cfg = cfg or ClusterConfig()
        self.nodes: Dict[int, NodeInfo] = {}
        self.failed: List[int] = []
        self.stats = {"routed": 0, "dropped": 0, "failures": 0}
        self.failure_cbs: List[Callable[[int], None]] = []
        self.recovery_cbs: List[Callable[[int], None]] = []

    def add_node(self, node: NodeInfo):
        self.nodes[node.id] = node

    def remove_node(self, node_id: int):
        self.nodes.pop(node_id, None)
        if node_id in self.failed:
            self.failed.remove(node_id)

    def on_node_failure(self, node_id: int):
        n = self.nodes.get(node_id)
        if n is None or not n.alive:
            return
        n.alive = False
        self.failed.append(node_id)
        self.stats["failures"] += 1
        for cb in self.failure_cbs:
            cb(node_id)

    def on_node_recovery(self, node_id: int):
        n = self.nodes.get(node_id)
        if n is None or n.alive:
            return
        n.alive = True
        self.failed.remove(node_id)
        for cb in self.recovery_cbs:
            cb(node_id)

    def alive_nodes(self) -> List[int]:
        return sorted(i for i, n in self.nodes.items() if n.alive)

    def get_failed_nodes(self) -> List[int]:
        return list(self.failed)

    # ---- periodic health check (reference: FaultToleranceManager::start_heartbeat, include/quant/expert_parallel.h:240)
    def start_heartbeat(self, interval_ms: int, probe: Optional[Callable[[int], bool]] = None):
        """Every ``interval_ms`` a daemon thread asks ``probe(node_id)`` (default: the node's ``alive`` flag as last set
        by the transport) about every known node; a node whose probe fails is reported through ``on_node_failure``, one
        that answers again through ``on_node_recovery``."""
        self.stop_heartbeat()
        self._hb_stop = threading.Event()
        self._hb_probe = probe

        def loop():
            while not self._hb_stop.wait(max(1, interval_ms) / 1e3):
                self.heartbeat_once()
        self._hb_thread = threading.Thread(target=loop, name="tfb-fault-heartbeat", daemon=True)
        self._hb_thread.start()

    def heartbeat_once(self):
        """One round of the health check (what the heartbeat thread runs; callable directly from tests)."""
        probe = getattr(self, "_hb_probe", None)
        for i in list(self.nodes):
            ok = probe(i) if probe is not None else self.nodes[i].alive
            if not ok and i not in self.failed:
                self.on_node_failure(i)
            elif ok and i in self.failed:
                self.on_node_recovery(i)

    def stop_heartbeat(self):
        t = getattr(self, "_hb_thread", None)
        if t is not None:
            self._hb_stop.set()
            t.join(timeout=2.0)
            self._hb_thread = None

    def heartbeat_running(self) -> bool:
        t = getattr(self, "_hb_thread", None)
        return t is not None and t.is_alive()

    def check_node_health(self, node_id: int) -> bool:
        n = self.nodes.get(node_id)
        return bool(n and n.alive)

    def checkpoint_state(self) -> str:
        parts = [f"nodes:{len(self.nodes)}", f"failed:{len(self.failed)}"]
        parts += [f"failed_node{{{i}}}" for i in self.failed]
        parts += [f"node{{{n.id},{n.addr},{n.port},{n.num_experts}}}" for n in sorted(self.nodes.values(), key=lambda x: x.id)]
        parts.append("stats{routed=%d,dropped=%d,failures=%d}" % (self.stats["routed"], self.stats["dropped"], self.stats["failures"]))
        return ";".join(parts)

    def restore_state(self, text: str) -> bool:
        try:
            nodes, failed = {}, []
            for m in re.finditer(r"node\{(\d+),([^,}]*),(\d+),(\d+)\}", text):
                if text[max(0, m.start() - 7):m.start()] == "failed_":
                    continue
                nodes[int(m.group(1))] = NodeInfo(int(m.group(1)), m.group(2), int(m.group(3)), int(m.group(4)))
            for m in re.finditer(r"failed_node\{(\d+)\}", text):
                failed.append(int(m.group(1)))
            st = re.search(r"stats\{routed=(\d+),dropped=(\d+),failures=(\d+)\}", text)
            head = re.match(r"nodes:(\d+);failed:(\d+)", text)
            if not head or int(head.group(1)) != len(nodes) or int(head.group(2)) != len(failed) or not st:
                return False
            for i in failed:
                if i in nodes:
                    nodes[i].alive = False
            self.nodes, self.failed = nodes, failed
            self.stats = {"routed": int(st.group(1)), "dropped": int(st.group(2)), "failures": int(st.group(3))}
            return True
        except (ValueError, AttributeError):
            return False

    def save(self, path):
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            f.write(self.checkpoint_state())
        os.replace(tmp, path)

    def load(self, path) -> bool:
        try:
            return self.restore_state(open(path).read())
        except OSError:
            return False


def redistribute_experts(num_experts: int, alive_ranks: List[int]) -> Dict[int, List[int]]:
    """Contiguous blocks of experts over the surviving ranks (the first ``num_experts % n`` ranks get one more)."""
    n = len(alive_ranks)
    if n == 0:
        raise RuntimeError("no rank left to host the experts")
    base, extra = divmod(num_experts, n)
    out, e = {}, 0
    for i, r in enumerate(sorted(alive_ranks)):
        k = base + (1 if i < extra else 0)
        out[r] = list(range(e, e + k))
        e += k
    return out


def compute_redistribution(old: Dict[int, List[int]], new: Dict[int, List[int]]):
    """[(expert, from_rank or None when its owner is gone, to_rank)] for every expert that changes owner."""
    owner_old = {e: r for r, es in old.items() for e in es}
    moves = []
    for r, es in new.items():
        for e in es:
            if owner_old.get(e) != r:
                moves.append((e, owner_old.get(e) if owner_old.get(e) in new else None, r))
    return sorted(moves)


def reshard_flat(shards: List[torch.Tensor], new_world: int, pad_multiple: int = 1024) -> List[torch.Tensor]:
    """Old per-rank shards of one flat buffer -> new equal shards (zero padded so that the length divides evenly)."""
    flat = torch.cat([s.reshape(-1) for s in shards])
    gran = new_world * pad_multiple
    n = (flat.numel() + gran - 1) // gran * gran
    if n > flat.numel():
        flat = torch.cat([flat, torch.zeros(n - flat.numel(), dtype=flat.dtype)])
    return list(flat.chunk(new_world))


STATUS_NAMES = {0: "ok", 1: "timeout_full", 2: "timeout_empty", 3: "timeout_tmem_full", 4: "timeout_tmem_empty", 5: "timeout_drain",
                6: "timeout_flag"}


def device_wait_status(device=None, reset=True):
    """(code, name) of the first bounded wait that gave up on ``device`` since the last reset (0 = none)."""
    from ..ops import _lib
    w = _lib.status_word(device)
    code = int(w[0].item())
    if reset and code:
        w.zero_()
    return code, STATUS_NAMES.get(code, f"status_{code}")


class FaultInjector:
    """Host-side fault injection for tests."""

    def __init__(self, seed=0):
        self.rng = random.Random(seed)
        self.drop_prob, self.delay_s = 0.0, 0.0
        self.dropped = 0

    def wrap_store(self, store):
        inj = self

        class Lossy:
            def set(self, k, v):
                if inj.rng.random() < inj.drop_prob:
                    inj.dropped += 1
                    return
                if inj.delay_s:
                    time.sleep(inj.delay_s)
                store.set(k, v)

            def get(self, k):
                return store.get(k)

            def check(self, keys):
                return store.check(keys)
        return Lossy()

    @staticmethod
    def truncate_file(path, keep_fraction=0.5):
        n = os.path.getsize(path)
        with open(path, "r+b") as f:
            f.truncate(int(n * keep_fraction))

    @staticmethod
    def corrupt_file(path, offset, nbytes=1):
        with open(path, "r+b") as f:
            f.seek(offset)
            b = f.read(nbytes)
            f.seek(offset)
            f.write(bytes(x ^ 0xFF for x in b))

    @staticmethod
    def raise_in_rank(rank, target_rank, exc=RuntimeError("injected failure")):
        if rank == target_rank:
            raise exc
