"""DistributedContext / RingAllReduce over gloo (CPU, 3 ranks) and the fused symmetric-memory collectives on GPUs."""
import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(n, backend, tmp_path, env=None):
    port = 29700 + (os.getpid() % 90) + (7 if backend == "nccl" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mp_coll_worker.py"), str(tmp_path), backend]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, **(env or {})))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return [json.load(open(os.path.join(tmp_path, f"rank{i}.json"))) for i in range(n)]


def test_host_collectives_gloo(tmp_path):
    for res in _launch(3, "gloo", tmp_path, {"CUDA_VISIBLE_DEVICES": ""}):
        for k, v in res.items():
            assert v < 1e-5, (k, v)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fused_collectives(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    g = torch.cuda.device_count()
    n = 2 if g < 4 else (4 if g < 8 else 8)
    for res in _launch(n, "nccl", tmp_path, {"NCCL_NVLS_ENABLE": "0"}):
        assert res["status"] == 0, res
        for k, v in res.items():
            if k.startswith("sc_"):
                assert v <= 1.0, (k, v)
            elif k != "status":
                assert v < 1e-4, (k, v)


def test_parameter_server():
    from transformers_fusion_b200.parallel.collectives import ParameterServer
    ps = ParameterServer(num_shards=2, lr=0.1)
    ps.push("w", torch.ones(4))
    w, ver = ps.pull("w")
    assert ver == 1 and ps.update_gradient("w", torch.ones(4), ver)
    assert torch.allclose(ps.pull("w")[0], torch.full((4,), 0.9))
    assert ps.update_gradient("w", torch.ones(4), ver)                      # one version stale: half step
    assert torch.allclose(ps.pull("w")[0], torch.full((4,), 0.85))
    for _ in range(6):
        ps.push("w", ps.pull("w")[0])
    assert not ps.update_gradient("w", torch.ones(4), ver) and ps.dropped == 1
    a = ParameterServer(async_mode=True, lr=1.0)
    a.push("k", torch.zeros(2))
    for _ in range(10):
        a.update_gradient("k", torch.ones(2), a.pull("k")[1])
    a.flush()
    a.stop()
    assert a.pull("k")[0].min() < -2
