import time

import pytest
import torch

from transformers_fusion_b200.parallel import expert_cluster as X
from transformers_fusion_b200.parallel.fault import ClusterConfig


def test_dispatch_roundtrip_matches_dense_mixture():
    torch.manual_seed(0)
    T, H, E, k = 40, 8, 6, 2
    d = X.ExpertDispatcher(E, num_nodes=3, node_id=1, top_k=k, hidden=H)
    assert d.assignment == [[0, 1], [2, 3], [4, 5]]
    x, logits = torch.randn(T, H), torch.randn(T, E)
    W = torch.randn(E, H, H)
    r = d.route_tokens(logits)
    assert torch.allclose(r.expert_weights.sum(-1), torch.ones(T)) and int(r.tokens_per_expert.sum()) == T * k
    assert int(r.tokens_per_node.sum()) == T * k
    disp = d.dispatch_tokens(x, r)
    outs = {n: torch.stack([rows[i] @ W[int(e)] for i, e in enumerate(eids)]) if len(eids) else torch.zeros(0, H)
            for n, (rows, eids, _) in disp.items()}
    y = d.gather_results(outs, disp, r, T)
    ref = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            ref[t] += r.expert_weights[t, j] * (x[t] @ W[int(r.expert_indices[t, j])])
    assert torch.allclose(y, ref, atol=1e-5)
    plan = d.plan_all_to_all(r, [[0, 3, 0], r.tokens_per_node.tolist(), [0, 5, 0]])
    assert plan.send_counts == r.tokens_per_node.tolist() and plan.recv_counts == [3, int(r.tokens_per_node[1]), 5]
    assert plan.total_bytes == (plan.send_counts[0] + plan.send_counts[2]) * H * 4
    lb, z = d.compute_load_balance(r)
    assert lb > 0.9 and z > 0
    d.redistribute_expert(5, 0)
    assert d.assignment[0] == [0, 1, 5] and int(d.owner[5]) == 0


def test_load_metrics():
    even = X.LoadBalanceMetrics.compute([10, 10, 10, 10])
    skew = X.LoadBalanceMetrics.compute([40, 0, 0, 0])
    assert even.cv == 0 and abs(even.gini) < 1e-9 and even.entropy == pytest.approx(1.3862943, rel=1e-5)
    assert skew.cv > 1.5 and skew.gini == pytest.approx(0.75) and skew.entropy == 0
    h = X.RoutingHistogram(4)
    h.update(torch.tensor([[0, 1], [0, 2]]))
    assert h.counts.tolist() == [2, 1, 1, 0] and h.utilization() == 0.75


def test_cluster_join_heartbeat_failure_and_grad_sync(tmp_path):
    cfg = ClusterConfig(heartbeat_interval_ms=50, fault_timeout_ms=2000)
    a, b = X.ExpertParallelManager(cfg, 8), X.ExpertParallelManager(cfg, 8)
    pa = a.init_cluster(0)
    pb = b.init_cluster(1)
    try:
        assert b.join_cluster("127.0.0.1", pa) and a.join_cluster("127.0.0.1", pb)
        a.process_messages(0.3), b.process_messages(0.3)
        assert a.assignment == {0: [0, 1, 2, 3], 1: [4, 5, 6, 7]} and b.local_experts() == [4, 5, 6, 7]
        b.send_heartbeats()
        assert a.process_messages(0.3) >= 1 and a.check_failures() == []
        # gradient averaging over the control plane
        import threading
        res = {}
        t = threading.Thread(target=lambda: res.setdefault("b", b.sync_gradients(torch.full((4,), 3.0))))
        t.start()
        ga = a.sync_gradients(torch.full((4,), 1.0))
        t.join()
        assert torch.allclose(ga, torch.full((4,), 2.0)) and torch.allclose(res["b"], torch.full((4,), 2.0))
        # node 1 goes silent (host-side fault): after the timeout its experts move to node 0
        dead = a.check_failures(now=time.time() + 5.0)
        assert dead == [1] and a.assignment == {0: list(range(8))} and all(src is None for _, src, _ in a.last_moves)
        a.checkpoint_experts(str(tmp_path / "e.pt"), {0: {"w": torch.ones(2)}})
        c = X.ExpertParallelManager(cfg, 8)
        ex = c.restore_experts(str(tmp_path / "e.pt"))
        assert c.assignment == {0: list(range(8))} and torch.equal(ex[0]["w"], torch.ones(2)) and c.ft.failed == [1]
        # the node comes back
        b.send_heartbeats()
        a.process_messages(0.3)
        assert a.ft.failed == [] and a.assignment[1] == [4, 5, 6, 7]
    finally:
        a.comm.close(), b.comm.close()


def test_tcp_backend_rejects_foreign_bytes():
    s = X.TCPCommBackend(0, timeout_s=0.5)
    port = s.listen()
    import socket
    c = socket.create_connection(("127.0.0.1", port))
    c.sendall(b"GET / HTTP/1.1\r\n" + b"x" * 80)
    c.close()
    good = X.TCPCommBackend(1, timeout_s=0.5)
    assert good.send(("127.0.0.1", port), X.MSG_TOKEN_DATA, b"z" * 200000)
    m = s.recv(X.MSG_TOKEN_DATA, 2.0)
    assert m is not None and m[1] == 1 and len(m[3]) == 200000 and s.recv(None, 0.1) is None
    s.close(), good.close()


def test_pipeline_scheduler_chains_stages_and_micro_batches():
    import torch
    from transformers_fusion_b200.parallel.expert_cluster import PipelineScheduler
    sch = PipelineScheduler(3, micro_batch_size=2)
    calls = []

    class Stage:
        def __init__(self, k):
            self.k = k

        def forward_expert_parallel(self, x, experts):
            calls.append((self.k, x.shape[0]))
            return x + self.k
    x = torch.zeros(5, 4)
    assert sch.execute_pipeline([Stage(1), Stage(10), Stage(100)]) is None and sch.all_stages_done()
    sch.schedule_forward(x, 0)
    assert not sch.all_stages_done()
    y = sch.execute_pipeline([Stage(1), Stage(10), Stage(100)])
    assert torch.equal(y, x + 111) and sch.all_stages_done()
    assert calls[:3] == [(1, 2), (10, 2), (100, 2)] and len(calls) == 9          # three micro-batches through three stages
    assert torch.equal(sch.get_stage(2).output_buffer, torch.full((1, 4), 111.0))
    sch.reset()
    assert sch.get_stage(0).input_buffer is None and sch.current_step == 0


def test_manager_forward_over_local_experts_sums_to_the_dense_mixture():
    """Two managers that hold half of the experts each: their partial outputs add up to the dense top-k mixture, stats
    are counted, a failure moves the experts, and real managers can be chained by the pipeline scheduler."""
    from transformers_fusion_b200.parallel.fault import NodeInfo
    E, H, F_, T = 4, 16, 24, 12
    g = torch.Generator().manual_seed(0)
    experts = {e: (torch.randn(2 * F_, H, generator=g) * 0.2, torch.randn(H, F_, generator=g) * 0.2) for e in range(E)}
    x = torch.randn(T, H, generator=g)
    router = torch.randn(E, H, generator=g)
    mgrs = []
    for node in (0, 1):
        m = X.ExpertParallelManager(ClusterConfig(), E, hidden_size=H, top_k=2)
        m.node_id, m.router = node, router
        m.restore_nodes([NodeInfo(0, "127.0.0.1", 1), NodeInfo(1, "127.0.0.1", 2)])
        mgrs.append(m)
    assert mgrs[0].local_experts() == [0, 1] and mgrs[1].local_experts() == [2, 3] and mgrs[0].num_nodes() == 2
    outs = [m.forward_expert_parallel(x, {e: experts[e] for e in m.local_experts()}) for m in mgrs]
    # dense statement of the same layer
    probs = torch.softmax(x @ router.t(), -1)
    w, idx = probs.topk(2, -1)
    w = w / w.sum(-1, keepdim=True)
    want = torch.zeros(T, H)
    for t in range(T):
        for k in range(2):
            want[t] += w[t, k] * X._run_expert(experts[int(idx[t, k])], x[t:t + 1])[0]
    assert torch.allclose(outs[0].output + outs[1].output, want, atol=1e-5)
    assert torch.equal(outs[0].expert_indices, idx) and outs[0].load_balance_loss >= 1.0 - 1e-4 and outs[0].z_loss > 0
    st = mgrs[0].get_stats()
    assert st.total_tokens_routed == T and 1 <= st.total_expert_forward_calls <= 2 and st.max_load_imbalance >= 1.0
    assert st.total_comm_bytes > 0 and torch.equal(mgrs[0].expert_parallel_mlp(x, experts), outs[0].output)
    # node 1 fails: its experts move to node 0, which then computes the whole mixture
    moves = mgrs[0].redistribute_experts_after_failure(1)
    assert sorted(e for e, _, _ in moves) == [2, 3] and mgrs[0].local_experts() == [0, 1, 2, 3]
    assert torch.allclose(mgrs[0].forward_expert_parallel(x, experts).output, want, atol=1e-5)
    assert mgrs[0].get_stats().expert_redistributions == 1
    mgrs[0].reset_stats()
    assert mgrs[0].get_stats().total_tokens_routed == 0
    # dispatcher bookkeeping
    d = X.ExpertDispatcher(8, 2, 0)
    assert d.get_all_assignments() == [0, 0, 0, 0, 1, 1, 1, 1]
    d.assign_experts_to_nodes(4)
    assert d.get_expert_assignment(7) == 3 and d.get_all_assignments() == [0, 0, 1, 1, 2, 2, 3, 3]
    # scheduler over real managers: stage 2 consumes stage 1's mixture
    sch = X.PipelineScheduler(2, micro_batch_size=T)
    sch.schedule_forward(x, 0)
    y = sch.execute_pipeline([mgrs[0], mgrs[0]], [experts, experts])
    assert torch.allclose(y, mgrs[0].forward_expert_parallel(want, experts).output, atol=1e-4)


def test_fault_manager_heartbeat_thread_reports_failure_and_recovery():
    from transformers_fusion_b200.parallel.fault import FaultToleranceManager, NodeInfo
    ft = FaultToleranceManager(ClusterConfig())
    for i in range(3):
        ft.add_node(NodeInfo(i, "127.0.0.1", 1000 + i))
    seen = []
    ft.failure_cbs.append(lambda i: seen.append(("down", i)))
    ft.recovery_cbs.append(lambda i: seen.append(("up", i)))
    health = {0: True, 1: True, 2: True}
    ft.start_heartbeat(10, probe=lambda i: health[i])
    assert ft.heartbeat_running()
    health[2] = False
    deadline = time.time() + 3.0
    while ("down", 2) not in seen and time.time() < deadline:
        time.sleep(0.01)
    assert seen == [("down", 2)] and ft.get_failed_nodes() == [2] and not ft.check_node_health(2)
    health[2] = True
    while ("up", 2) not in seen and time.time() < deadline:
        time.sleep(0.01)
    ft.stop_heartbeat()
    assert seen == [("down", 2), ("up", 2)] and ft.get_failed_nodes() == [] and not ft.heartbeat_running()


def test_tcp_backend_node_addressing_async_and_byte_counters():
    s = X.TCPCommBackend(0, timeout_s=1.0)
    port = s.listen()
    c = X.TCPCommBackend(1, timeout_s=1.0)
    try:
        assert not c.is_connected(0) and not c.send(0, X.MSG_TOKEN_DATA, b"x") and c.connect("127.0.0.1", port, node_id=0) and c.is_connected(0)
        waiter = s.recv_async(X.MSG_TOKEN_DATA, 2.0)
        sends = [c.send_async(0, X.MSG_TOKEN_DATA, b"a" * 1000) for _ in range(3)]
        c.wait_all(), s.wait_all()
        assert all(t.ok for t in sends) and waiter.message is not None and waiter.message[1] == 1 and len(waiter.message[3]) == 1000
        assert s.recv(X.MSG_TOKEN_DATA, 1.0) is not None and s.recv(X.MSG_TOKEN_DATA, 1.0) is not None
        assert c.bytes_sent(0) == 3 * (1000 + 64) == s.bytes_received(1) and c.bytes_sent(7) == 0
        c.disconnect(0)
        assert not c.is_connected(0) and not c.send(0, X.MSG_TOKEN_DATA, b"x")
        assert not c.connect("127.0.0.1", 1, node_id=5)          # nothing listens on port 1
    finally:
        c.shutdown(), s.shutdown()
