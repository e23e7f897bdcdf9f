"""Expert parallelism composed with data-parallel replicas: the trainer sums the gradients of an expert over the ranks that
hold a copy of it and counts each distinct expert once in the clipping norm.  Checked on two CPU ranks (gloo) that both
hold every expert, where the result must equal one process training on the combined batch."""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_expert_replicas_match_single_process(tmp_path):
    import torch
    worker = os.path.join(HERE, "_mp_ep_replica_worker.py")
    env = {k: v for k, v in os.environ.items() if k not in ("WORLD_SIZE", "RANK", "LOCAL_RANK")}
    r = subprocess.run([sys.executable, worker, str(tmp_path)], capture_output=True, text=True, timeout=280, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    port = 29700 + os.getpid() % 90
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), worker, str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    ref = json.load(open(tmp_path / "w1_rank0.json"))
    r0 = json.load(open(tmp_path / "w2_rank0.json"))
    r1 = json.load(open(tmp_path / "w2_rank1.json"))
    assert r0["losses"] == r1["losses"]
    for a, b in zip(r0["losses"], ref["losses"]):
        assert abs(a - b) < 1e-4, (r0["losses"], ref["losses"])
    assert abs(r0["norm"] - ref["norm"]) < 1e-4 * max(1.0, ref["norm"])
    pr, p0, p1 = (torch.load(tmp_path / f) for f in ("w1_rank0.pt", "w2_rank0.pt", "w2_rank1.pt"))
    assert max(float((a - b).abs().max()) for a, b in zip(p0, pr)) < 1e-5
    assert all(torch.equal(a, b) for a, b in zip(p0, p1))
