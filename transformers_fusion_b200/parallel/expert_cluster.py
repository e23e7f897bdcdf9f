"""Expert-parallel cluster management (control plane) and the host statement of token dispatch.

* ``ExpertDispatcher``       - top-k routing with renormalised weights, per-expert / per-node token counts, the all-to-all
  plan (counts and bytes per destination), host-side ``dispatch_tokens`` / ``gather_results`` (the oracle of the fused
  device kernels in parallel/ep.py), load-balance and z losses, contiguous expert-to-node assignment.
* ``TCPCommBackend``         - length-framed messages over TCP (64-byte header, 64 KiB chunks): the control plane between
  nodes; bulk tensor data travels over NVLink through the symmetric heap, never through this class.
* ``ExpertParallelManager``  - node table, join / leave, heartbeats, failure handling with expert redistribution, expert
  checkpoint / restore, gradient averaging over the control plane for small tensors.
* ``LoadBalanceMetrics`` / ``RoutingHistogram`` - coefficient of variation, Gini, entropy of the expert load.

Reference counterparts: src/model/expert_parallel.cpp (TCPCommBackend :92-311, assign_experts_to_nodes :319,
ExpertDispatcher :354-555, ExpertParallelManager :614-952, LoadBalanceMetrics :1345), include/quant/expert_parallel.h."""
from __future__ import annotations

import math
import socket
import struct
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .fault import ClusterConfig, FaultToleranceManager, NodeInfo, compute_redistribution, redistribute_experts

MSG_TOKEN_DATA, MSG_EXPERT_OUTPUT, MSG_HEARTBEAT, MSG_JOIN, MSG_LEAVE, MSG_GRADIENT_SYNC, MSG_CHECKPOINT = range(1, 8)
_HDR = struct.Struct("<4sIIIQQ32x")          # magic, type, src, dst, payload bytes, sequence number; padded to 64 bytes
CHUNK = 64 << 10


@dataclass
class RoutingDecision:
    expert_indices: torch.Tensor      # [T, k]
    expert_weights: torch.Tensor      # [T, k] renormalised over the chosen experts
    tokens_per_expert: torch.Tensor   # [E]
    tokens_per_node: torch.Tensor     # [nodes]
    probs: torch.Tensor               # [T, E] full softmax
    lse: torch.Tensor                 # [T]


@dataclass
class AllToAllPlan:
    send_counts: List[int]            # token copies this node sends to each node
    recv_counts: List[int]
    send_bytes: List[int]
    total_bytes: int


def assign_experts_to_nodes(num_experts: int, num_nodes: int) -> List[List[int]]:
    """Contiguous blocks; the first ``num_experts % num_nodes`` nodes hold one expert more."""
    m = redistribute_experts(num_experts, list(range(num_nodes)))
    return [m[i] for i in range(num_nodes)]


class ExpertDispatcher:
    def __init__(self, num_experts: int, num_nodes: int = 1, node_id: int = 0, top_k: int = 2, hidden: int = 0, elem_bytes: int = 4):
        self.E, self.nodes, self.node, self.k, self.hidden, self.eb = num_experts, num_nodes, node_id, top_k, hidden, elem_bytes
        self.assignment = assign_experts_to_nodes(num_experts, num_nodes)
        self._refresh()

    def _refresh(self):
        self.owner = torch.empty(self.E, dtype=torch.long)
        for n, es in enumerate(self.assignment):
            for e in es:
                self.owner[e] = n

    def assign_experts_to_nodes(self, num_nodes: int):
        """Contiguous blocks over ``num_nodes`` nodes (replaces the current assignment)."""
        self.nodes = max(1, int(num_nodes))
        self.assignment = assign_experts_to_nodes(self.E, self.nodes)
        self._refresh()
        return self.assignment

    def get_expert_assignment(self, expert: int) -> int:
        """Node that holds ``expert``."""
        return int(self.owner[expert])

    def get_all_assignments(self) -> List[int]:
        """Owner node of every expert, by expert id."""
        return self.owner.tolist()

    def redistribute_expert(self, expert: int, to_node: int):
        for es in self.assignment:
            if expert in es:
                es.remove(expert)
        self.assignment[to_node].append(expert)
        self._refresh()

    def route_tokens(self, logits: torch.Tensor, top_k: Optional[int] = None) -> RoutingDecision:
        k = top_k or self.k
        lf = logits.float()
        lse = torch.logsumexp(lf, -1)
        probs = torch.softmax(lf, -1)
        w, idx = probs.topk(k, -1)
        w = w / w.sum(-1, keepdim=True)
        tpe = torch.bincount(idx.reshape(-1), minlength=self.E)
        tpn = torch.zeros(self.nodes, dtype=torch.long).index_add_(0, self.owner[idx.reshape(-1).cpu()], torch.ones(idx.numel(), dtype=torch.long))
        return RoutingDecision(idx, w, tpe, tpn, probs, lse)

    def plan_all_to_all(self, r: RoutingDecision, all_node_counts: Optional[List[List[int]]] = None) -> AllToAllPlan:
        """``all_node_counts[src][dst]`` (when every node's row is known) gives the receive side too."""
        send = r.tokens_per_node.tolist()
        recv = [row[self.node] for row in all_node_counts] if all_node_counts else [0] * self.nodes
        by = [c * self.hidden * self.eb for c in send]
        return AllToAllPlan(send, recv, by, sum(b for n, b in enumerate(by) if n != self.node))

    def dispatch_tokens(self, x: torch.Tensor, r: RoutingDecision):
        """Host oracle: {node: (token rows [n, H], expert id per row, (token, slot) origin per row)}."""
        out = {}
        idx = r.expert_indices.cpu()
        T, k = idx.shape
        tok = torch.arange(T).repeat_interleave(k)
        slot = torch.arange(k).repeat(T)
        flat = idx.reshape(-1)
        for n in range(self.nodes):
            sel = (self.owner[flat] == n).nonzero().reshape(-1)
            order = sel[torch.argsort(flat[sel], stable=True)]
            out[n] = (x[tok[order]], flat[order], torch.stack([tok[order], slot[order]], 1))
        return out

    def gather_results(self, outputs: Dict[int, torch.Tensor], dispatched, r: RoutingDecision, T: int):
        """Weighted sum of the experts' outputs back into token order."""
        H = next(iter(outputs.values())).shape[1]
        y = torch.zeros((T, H), dtype=torch.float32)
        w = r.expert_weights.cpu().float()
        for n, o in outputs.items():
            origin = dispatched[n][2]
            y.index_add_(0, origin[:, 0], o.float() * w[origin[:, 0], origin[:, 1]][:, None])
        return y

    def compute_load_balance(self, r: RoutingDecision) -> Tuple[float, float]:
        """(load-balance loss E * sum f_i P_i, z loss mean lse^2)."""
        f = r.tokens_per_expert.float() / max(1, int(r.tokens_per_expert.sum()))
        P = r.probs.mean(0).cpu()
        return float(self.E * (f * P).sum()), float((r.lse ** 2).mean())


@dataclass
class LoadBalanceMetrics:
    cv: float = 0.0
    gini: float = 0.0
    entropy: float = 0.0
    max_load: int = 0
    min_load: int = 0

    @classmethod
    def compute(cls, counts) -> "LoadBalanceMetrics":
        c = torch.as_tensor(counts, dtype=torch.float64)
        n, tot = c.numel(), float(c.sum())
        if tot == 0:
            return cls()
        mean = tot / n
        cv = float(c.std(unbiased=False) / mean)
        s = torch.sort(c).values
        gini = float((2 * (torch.arange(1, n + 1, dtype=torch.float64) * s).sum() / (n * tot)) - (n + 1) / n)
        p = c / tot
        ent = float(-(p[p > 0] * torch.log(p[p > 0])).sum())
        return cls(cv, gini, ent, int(c.max()), int(c.min()))


class RoutingHistogram:
    def __init__(self, num_experts):
        self.counts = torch.zeros(num_experts, dtype=torch.long)
        self.steps = 0

    def update(self, expert_indices):
        self.counts += torch.bincount(expert_indices.reshape(-1).cpu(), minlength=self.counts.numel())
        self.steps += 1

    def metrics(self):
        return LoadBalanceMetrics.compute(self.counts)

    def utilization(self):
        return (self.counts > 0).float().mean().item()


class TCPCommBackend:
    """Framed messages between nodes.  ``listen`` starts an accept thread that queues whole messages; ``send`` connects
    (once per destination), writes the 64-byte header and the payload in 64 KiB chunks."""

    def __init__(self, node_id: int, timeout_s: float = 5.0):
        self.node, self.timeout = node_id, timeout_s
        self.server: Optional[socket.socket] = None
        self.port = 0
        self.inbox: List[Tuple[int, int, int, bytes]] = []       # (type, src, seq, payload)
        self.cv = threading.Condition()
        self.conns: Dict[Tuple[str, int], socket.socket] = {}
        self.seq = 0
        self._stop = False
        self.threads: List[threading.Thread] = []
        self.peers: Dict[int, Tuple[str, int]] = {}             # node id -> address, filled by connect()
        self._tx: Dict[int, int] = {}
        self._rx: Dict[int, int] = {}
        self._pending: List[threading.Thread] = []
        self._send_lock = threading.Lock()

    def listen(self, port: int = 0, host: str = "127.0.0.1") -> int:
        self.server = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.server.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.server.bind((host, port))
        self.server.listen(16)
        self.server.settimeout(0.2)
        self.port = self.server.getsockname()[1]
        t = threading.Thread(target=self._accept, daemon=True)
        t.start()
        self.threads.append(t)
        return self.port

    def _accept(self):
        while not self._stop:
            try:
                c, _ = self.server.accept()
            except (socket.timeout, OSError):
                continue
            c.settimeout(self.timeout)
            t = threading.Thread(target=self._reader, args=(c,), daemon=True)
            t.start()
            self.threads.append(t)

    @staticmethod
    def _read_exact(c, n):
        buf = bytearray()
        while len(buf) < n:
            part = c.recv(min(CHUNK, n - len(buf)))
            if not part:
                return None
            buf += part
        return bytes(buf)

    def _reader(self, c):
        try:
            while not self._stop:
                try:
                    hdr = self._read_exact(c, _HDR.size)
                except socket.timeout:
                    continue
                if hdr is None:
                    return
                magic, typ, src, dst, nbytes, seq = _HDR.unpack(hdr)
                if magic != b"TFEP" or nbytes > (1 << 32):
                    return                                   # not ours / corrupt: drop the connection
                payload = self._read_exact(c, nbytes) if nbytes else b""
                if payload is None:
                    return
                with self.cv:
                    self.inbox.append((typ, src, seq, payload))
                    self._rx[src] = self._rx.get(src, 0) + _HDR.size + len(payload)
                    self.cv.notify_all()
        except OSError:
            return
        finally:
            c.close()

    def send(self, addr, typ: int, payload: bytes = b"", dst: int = 0) -> bool:
        """``addr``: an (host, port) pair, or the node id of a peer registered with ``connect``."""
        if isinstance(addr, int):
            if addr not in self.peers:
                return False
            addr, dst = self.peers[addr], addr
        with self._send_lock:
            ok = self._send_locked(addr, typ, payload, dst)
        if ok:
            self._tx[dst] = self._tx.get(dst, 0) + _HDR.size + len(payload)
        return ok

    def _send_locked(self, addr: Tuple[str, int], typ: int, payload: bytes, dst: int) -> bool:
        try:
            c = self.conns.get(addr)
            if c is None:
                c = socket.create_connection(addr, timeout=self.timeout)
                self.conns[addr] = c
            self.seq += 1
            c.sendall(_HDR.pack(b"TFEP", typ, self.node, dst, len(payload), self.seq))
            for o in range(0, len(payload), CHUNK):
                c.sendall(payload[o:o + CHUNK])
            return True
        except OSError:
            self.conns.pop(addr, None)
            return False

    def recv(self, typ: Optional[int] = None, timeout_s: Optional[float] = None):
        end = time.time() + (timeout_s if timeout_s is not None else self.timeout)
        with self.cv:
            while True:
                for i, m in enumerate(self.inbox):
                    if typ is None or m[0] == typ:
                        return self.inbox.pop(i)
                rest = end - time.time()
                if rest <= 0:
                    return None
                self.cv.wait(rest)

    # ---- node-id addressed form (reference: TCPCommBackend, include/quant/expert_parallel.h:91-111)
    def connect(self, address: str, port: int, node_id: Optional[int] = None) -> bool:
        """Open the connection to a peer now and remember it under ``node_id`` (default: the next free id)."""
        nid = node_id if node_id is not None else (max(self.peers) + 1 if self.peers else 0)
        addr = (address, int(port))
        try:
            if addr not in self.conns:
                self.conns[addr] = socket.create_connection(addr, timeout=self.timeout)
        except OSError:
            return False
        self.peers[nid] = addr
        return True

    def disconnect(self, node_id: int):
        addr = self.peers.pop(node_id, None)
        c = self.conns.pop(addr, None) if addr else None
        if c is not None:
            try:
                c.close()
            except OSError:
                pass

    def is_connected(self, node_id: int) -> bool:
        return node_id in self.peers and self.peers[node_id] in self.conns

    def bytes_sent(self, node_id: int) -> int: return self._tx.get(node_id, 0)
    def bytes_received(self, node_id: int) -> int: return self._rx.get(node_id, 0)

    def send_async(self, node_id, typ: int, payload: bytes = b"") -> "threading.Thread":
        """Send on a helper thread; ``wait_all`` joins every outstanding one.  The thread's ``ok`` attribute holds the result."""
        def run():
            t.ok = self.send(node_id, typ, payload)
        t = threading.Thread(target=run, daemon=True)
        t.ok = None
        t.start()
        self._pending.append(t)
        return t

    def recv_async(self, typ: Optional[int] = None, timeout_s: Optional[float] = None) -> "threading.Thread":
        """Wait for a message on a helper thread; after ``wait_all`` (or ``join``) its ``message`` attribute holds it (None on
        time-out)."""
        def run():
            t.message = self.recv(typ, timeout_s)
        t = threading.Thread(target=run, daemon=True)
        t.message = None
        t.start()
        self._pending.append(t)
        return t

    def wait_all(self):
        pend, self._pending = self._pending, []
        for t in pend:
            t.join()

    def shutdown(self):
        self.wait_all()
        self.close()

    def close(self):
        self._stop = True
        self.peers.clear()
        for c in self.conns.values():
            try:
                c.close()
            except OSError:
                pass
        if self.server:
            self.server.close()


@dataclass
class ExpertParallelStats:
    total_tokens_routed: int = 0
    total_tokens_dropped: int = 0
    total_comm_bytes: int = 0
    total_expert_forward_calls: int = 0
    avg_load_imbalance: float = 0.0
    max_load_imbalance: float = 0.0
    node_failures_handled: int = 0
    expert_redistributions: int = 0
    total_forward_time_ms: float = 0.0
    total_comm_time_ms: float = 0.0


@dataclass
class MoEOutput:
    output: torch.Tensor                       # [T, H]: the weighted sum over the experts THIS node holds
    router_logits: torch.Tensor
    expert_weights: torch.Tensor
    expert_indices: torch.Tensor
    load_balance_loss: float = 0.0
    z_loss: float = 0.0
    tokens_dropped: int = 0


def _run_expert(expert, x: torch.Tensor) -> torch.Tensor:
    """``expert``: a callable, or (gate_up [2F, H], down [H, F]) weights of a SwiGLU expert."""
    if callable(expert):
        return expert(x)
    gate_up, down = expert
    gu = x.float() @ gate_up.float().t()
    F_ = gu.shape[1] // 2
    return ((torch.nn.functional.silu(gu[:, :F_]) * gu[:, F_:]) @ down.float().t()).to(x.dtype)


class ExpertParallelManager:
    def __init__(self, cfg: Optional[ClusterConfig] = None, num_experts: int = 0, hidden_size: int = 0, top_k: int = 2):
        self.cfg = cfg or ClusterConfig(num_experts=num_experts)
        self.E = num_experts or self.cfg.num_experts
        self.hidden, self.top_k = hidden_size, top_k
        self.ft = FaultToleranceManager(self.cfg)
        self.comm: Optional[TCPCommBackend] = None
        self.node_id = 0
        self.assignment: Dict[int, List[int]] = {}
        self.last_seen: Dict[int, float] = {}
        self.ft.failure_cbs.append(self._on_failure)
        self.stats = ExpertParallelStats()
        self.router: Optional[torch.Tensor] = None       # [E, H]; made on first use (or set by the caller)
        self._imbalance_n = 0

    # ---- accessors of the reference's manager (include/quant/expert_parallel.h:150-158)
    def is_cluster_active(self) -> bool: return self.comm is not None and self.comm.server is not None
    def local_node_id(self) -> int: return self.node_id
    def num_nodes(self) -> int: return max(1, len(self.ft.alive_nodes()))
    def get_nodes(self) -> List[NodeInfo]: return sorted(self.ft.nodes.values(), key=lambda n: n.id)
    def get_stats(self) -> ExpertParallelStats: return self.stats
    def reset_stats(self): self.stats = ExpertParallelStats(); self._imbalance_n = 0

    def restore_nodes(self, nodes: List[NodeInfo]):
        self.ft.nodes = {n.id: n for n in nodes}
        self.ft.failed = [n.id for n in nodes if not n.alive]
        self._reassign()

    def restore_stats(self, stats: ExpertParallelStats): self.stats = stats

    # ---- forward over the experts this node holds
    def forward_expert_parallel(self, x: torch.Tensor, local_experts, training: bool = True) -> MoEOutput:
        """Route all T tokens over all experts, run those routed to an expert of THIS node and return their weighted sum
        (the sum of the nodes' outputs is the layer's output).  ``local_experts``: {expert id: expert} or a list indexed
        by expert id; an expert is a callable or a (gate_up, down) pair.  Reference:
        src/model/expert_parallel.cpp:683-758 (which walks token by token; here each expert runs once on its rows)."""
        t0 = time.perf_counter()
        T, H = x.shape[0], x.shape[-1]
        xf = x.reshape(T, H)
        if self.router is None:
            g = torch.Generator().manual_seed(1234)
            self.router = (torch.randn(self.E, H, generator=g) * H ** -0.5).to(xf.device)
        logits = xf.float() @ self.router.float().t()
        nodes = sorted(self.ft.alive_nodes()) or [self.node_id]
        disp = ExpertDispatcher(self.E, 1, 0, self.top_k, H)
        r = disp.route_tokens(logits, self.top_k)
        mine = set(self.local_experts()) if self.assignment else set(range(self.E))
        experts = local_experts if isinstance(local_experts, dict) else dict(enumerate(local_experts or []))
        out = torch.zeros((T, H), dtype=torch.float32, device=xf.device)
        calls = 0
        for e in sorted(mine):
            if e not in experts:
                continue
            tok, slot = (r.expert_indices == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            y = _run_expert(experts[e], xf[tok])
            out.index_add_(0, tok, y.float() * r.expert_weights[tok, slot].float()[:, None])
            calls += 1
        lb, z = disp.compute_load_balance(r)
        st = self.stats
        st.total_tokens_routed += T
        st.total_expert_forward_calls += calls
        st.total_forward_time_ms += (time.perf_counter() - t0) * 1e3
        remote = sum(int(c) for e, c in enumerate(r.tokens_per_expert.tolist()) if e not in mine)
        st.total_comm_bytes += remote * H * xf.element_size() * (2 if len(nodes) > 1 else 0)
        cnt = r.tokens_per_expert.float()
        imb = float(cnt.max() / cnt.mean().clamp(min=1e-9))            # busiest expert against the mean load
        self._imbalance_n += 1
        st.avg_load_imbalance += (imb - st.avg_load_imbalance) / self._imbalance_n
        st.max_load_imbalance = max(st.max_load_imbalance, imb)
        return MoEOutput(out.to(x.dtype).reshape(x.shape), logits, r.expert_weights, r.expert_indices, lb, z, 0)

    def expert_parallel_mlp(self, x: torch.Tensor, local_experts) -> torch.Tensor:
        """The output tensor of ``forward_expert_parallel`` alone."""
        return self.forward_expert_parallel(x, local_experts, training=False).output

    def rebalance_experts(self):
        """Contiguous reassignment over the nodes that are alive now."""
        self._reassign()
        self.stats.expert_redistributions += 1
        return self.assignment

    def redistribute_experts_after_failure(self, failed_node: int):
        """Experts of ``failed_node`` go to the surviving nodes; returns the moves [(expert, from, to)]."""
        n = self.ft.nodes.get(failed_node)
        if n is not None and n.alive:
            self.ft.on_node_failure(failed_node)          # triggers _reassign through the failure callback
        else:
            self._reassign()
        self.stats.expert_redistributions += 1
        return list(getattr(self, "last_moves", []))

    def all_reduce_gradients(self, grad: torch.Tensor, timeout_s: float = 5.0) -> torch.Tensor:
        """Average ``grad`` over the alive nodes through the control plane, in place (small tensors only; bulk gradients
        travel over NVLink through the fused collectives).  Reference: src/model/expert_parallel.cpp:777-806."""
        t0 = time.perf_counter()
        avg = self._average_over_nodes(grad, timeout_s)
        grad.copy_(avg.to(grad.dtype))
        self.stats.total_comm_time_ms += (time.perf_counter() - t0) * 1e3
        return grad

    # ---- membership
    def init_cluster(self, node_id: int, port: int = 0) -> int:
        self.node_id = node_id
        self.comm = TCPCommBackend(node_id)
        p = self.comm.listen(port)
        self.add_node(NodeInfo(node_id, "127.0.0.1", p))
        return p

    def join_cluster(self, addr: str, port: int) -> bool:
        me = self.ft.nodes[self.node_id]
        return self.comm.send((addr, port), MSG_JOIN, f"{me.id},{me.addr},{me.port}".encode())

    def leave_cluster(self):
        for n in self.ft.nodes.values():
            if n.id != self.node_id:
                self.comm.send((n.addr, n.port), MSG_LEAVE, str(self.node_id).encode())
        self.comm.close()

    def add_node(self, node: NodeInfo):
        self.ft.add_node(node)
        self.last_seen[node.id] = time.time()
        self._reassign()

    def remove_node(self, node_id: int):
        self.ft.remove_node(node_id)
        self._reassign()

    def _reassign(self):
        alive = self.ft.alive_nodes()
        if alive and self.E:
            new = redistribute_experts(self.E, alive)
            self.last_moves = compute_redistribution(self.assignment, new) if self.assignment else []
            self.assignment = new
            for n in self.ft.nodes.values():
                n.num_experts = len(new.get(n.id, []))

    def process_messages(self, timeout_s=0.05):
        """Drain control messages: joins, leaves, heartbeats."""
        n = 0
        while True:
            m = self.comm.recv(None, timeout_s)
            if m is None:
                return n
            typ, src, _, payload = m
            n += 1
            if typ == MSG_JOIN:
                i, a, p = payload.decode().split(",")
                self.add_node(NodeInfo(int(i), a, int(p)))
            elif typ == MSG_LEAVE:
                self.remove_node(int(payload.decode()))
            elif typ == MSG_HEARTBEAT:
                self.last_seen[src] = time.time()
                if src in self.ft.failed:
                    self.ft.on_node_recovery(src)
                    self._reassign()

    def send_heartbeats(self):
        for n in self.ft.nodes.values():
            if n.id != self.node_id:
                self.comm.send((n.addr, n.port), MSG_HEARTBEAT, b"", n.id)

    def check_failures(self, now: Optional[float] = None) -> List[int]:
        now = now if now is not None else time.time()
        dead = [i for i, t in self.last_seen.items() if i != self.node_id and now - t > self.cfg.fault_timeout_ms / 1e3
                and self.ft.check_node_health(i)]
        for i in dead:
            self.handle_node_failure(i)
        return dead

    def handle_node_failure(self, node_id: int):
        self.ft.on_node_failure(node_id)
        self.stats.node_failures_handled += 1

    def _on_failure(self, node_id):
        self._reassign()

    def local_experts(self) -> List[int]:
        return self.assignment.get(self.node_id, [])

    # ---- expert state
    def checkpoint_experts(self, path: str, expert_tensors: Dict[int, Dict[str, torch.Tensor]]):
        torch.save({"assignment": self.assignment, "experts": expert_tensors, "cluster": self.ft.checkpoint_state()}, path)

    def restore_experts(self, path: str) -> Dict[int, Dict[str, torch.Tensor]]:
        st = torch.load(path, map_location="cpu", weights_only=False)
        self.ft.restore_state(st["cluster"])
        self.assignment = st["assignment"]
        return st["experts"]

    # ---- small-tensor gradient averaging over the control plane
    def sync_gradients(self, grads, timeout_s: float = 5.0):
        """A tensor: its average over the nodes.  A mapping / list of tensors (the gradients of the local experts): each
        is averaged in place, as the reference's ``sync_gradients(local_experts)`` does."""
        if isinstance(grads, dict):
            return {k: self.all_reduce_gradients(g, timeout_s) for k, g in grads.items()}
        if isinstance(grads, (list, tuple)):
            return [self.all_reduce_gradients(g, timeout_s) for g in grads]
        return self._average_over_nodes(grads, timeout_s)

    def _average_over_nodes(self, grads: torch.Tensor, timeout_s: float = 5.0) -> torch.Tensor:
        peers = [n for n in self.ft.nodes.values() if n.id != self.node_id and n.alive]
        payload = grads.detach().float().cpu().numpy().tobytes()
        for n in peers:
            self.comm.send((n.addr, n.port), MSG_GRADIENT_SYNC, payload, n.id)
            self.stats.total_comm_bytes += len(payload)
        acc, got = grads.detach().float().cpu().clone(), 1
        for _ in peers:
            m = self.comm.recv(MSG_GRADIENT_SYNC, timeout_s)
            if m is None:
                break
            import numpy as np
            acc += torch.from_numpy(np.frombuffer(m[3], dtype=np.float32).copy()).view(acc.shape)
            got += 1
        return (acc / got).to(grads.device)


class PipelineStage:
    """One stage of the expert pipeline: the experts it runs, where, and its pending input / last output."""

    def __init__(self, stage_id: int):
        self.stage_id, self.expert_ids, self.node_id, self.ready = stage_id, [], -1, False
        self.input_buffer = self.output_buffer = None


class PipelineScheduler:
    """Chains expert-parallel stages: stage i's output becomes stage i + 1's input; ``execute_pipeline`` runs every stage
    that has input pending, in order, through its manager's ``forward_expert_parallel``.  ``micro_batch_size`` splits a
    scheduled input into micro-batches that flow through the stages one after another, so stage i can work on micro-batch
    j + 1 while stage i + 1 holds micro-batch j (the order a multi-node deployment overlaps).

    Reference counterpart: PipelineScheduler / PipelineStage (include/quant/expert_parallel.h:197-228,
    src/model/expert_parallel.cpp:975-1051)."""

    def __init__(self, num_stages: int, micro_batch_size: int):
        import threading
        self.num_stages, self.micro_batch_size = num_stages, max(1, micro_batch_size)
        self._stages = [PipelineStage(i) for i in range(num_stages)]
        self._lock = threading.Lock()
        self.current_step = 0

    def schedule_forward(self, x, stage_id: int):
        with self._lock:
            if 0 <= stage_id < self.num_stages:
                self._stages[stage_id].input_buffer, self._stages[stage_id].ready = x, True

    def schedule_backward(self, grad_output, stage_id: int):
        with self._lock:
            if 0 <= stage_id < self.num_stages:
                self._stages[stage_id].output_buffer = grad_output

    def execute_pipeline(self, managers, all_experts=None):
        """``managers[i]``: object with ``forward_expert_parallel(x, experts)`` (ExpertParallelManager) or a plain callable
        for stage i.  Returns the last stage's output (micro-batches concatenated) or None when nothing was pending."""
        import torch
        with self._lock:
            first = self._stages[0]
            if not first.ready or first.input_buffer is None:
                pending = [s for s in self._stages if s.ready and s.input_buffer is not None]
                if not pending:
                    return None
                start, chunks = pending[0].stage_id, [pending[0].input_buffer]
            else:
                start, chunks = 0, list(torch.split(first.input_buffer, self.micro_batch_size, 0))
            outs = []
            for mb in chunks:
                x = mb
                for st in range(start, self.num_stages):
                    s = self._stages[st]
                    if st >= len(managers) or managers[st] is None:
                        break
                    fn = managers[st]
                    ex = all_experts[st] if all_experts is not None and st < len(all_experts) else None
                    y = fn.forward_expert_parallel(x, ex) if hasattr(fn, "forward_expert_parallel") else fn(x)
                    y = getattr(y, "output", y)
                    s.input_buffer, s.output_buffer, s.ready = x, y, False
                    x = y
                    self.current_step += 1
                outs.append(x)
            return torch.cat(outs, 0) if len(outs) > 1 else outs[0]

    def get_stage(self, stage_id: int):
        with self._lock:
            return self._stages[stage_id] if 0 <= stage_id < self.num_stages else PipelineStage(-1)

    def all_stages_done(self) -> bool:
        with self._lock:
            return not any(s.ready for s in self._stages)

    def reset(self):
        with self._lock:
            for s in self._stages:
                s.ready, s.input_buffer, s.output_buffer = False, None, None
            self.current_step = 0
