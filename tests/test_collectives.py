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


def test_first_generation_wrappers_and_parameter_server_on_gloo(tmp_path):
    import json
    import subprocess
    import sys as _sys
    here = os.path.dirname(os.path.abspath(__file__))
    port = 29870 + (os.getpid() % 50)
    cmd = [_sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "_mp_wrappers_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = [json.load(open(os.path.join(tmp_path, f"rank{i}.json"))) for i in range(2)]
    assert [x["is_main"] for x in res] == [True, False] and res[0]["mode0"] == "DDP"
    for i, x in enumerate(res):
        assert x["tp_err"] < 1e-4 and x["tp_mode"] == "TENSOR_PARALLEL"
        assert x["split"] == ([0.0, 1.0, 2.0, 3.0] if i == 0 else [4.0, 5.0, 6.0, 7.0])
        assert x["ps_avg"] == [0.5] * 4 and x["ring"] == [i, 2]
        assert x["ddp"] == [1, 2, i, 2, True] and x["ddp_reset"] == 0 and x["wrapper_ctx"]
    assert res[0]["pp_err"] is None and res[1]["pp_err"] < 1e-4
    assert res[0]["ps_node"] == [True, 0, 1] and res[1]["ps_node"] == [False, -1, 1]


def test_parameter_server_management_verbs():
    import torch
    from transformers_fusion_b200.parallel.collectives import ParameterServer
    ps = ParameterServer(num_shards=3, lr=0.1)
    f = ps.push_async("a", torch.ones(3))
    f.result(5)
    ps.push("b", torch.full((2,), 2.0))
    assert ps.list_params() == ["a", "b"] and ps.owns_param("a") and not ps.owns_param("zz") and ps.get_param("zz") is None
    assert ps.get_version("a") == 1 and ps.get_version("zz") == -1
    assert 0 <= ParameterServer.shard_for("a", 3) < 3 and ParameterServer.shard_for("a", 3) == ParameterServer.shard_for("a", 3)
    t, v = ps.pull_async("a").result(5)
    assert v == 1 and ps.update_gradient_async("a", torch.ones(3), v).result(5)
    assert torch.allclose(ps.get_param("a"), torch.full((3,), 0.9))
    ps.apply_weight_decay(0.5)
    assert torch.allclose(ps.get_param("b"), torch.ones(2))
    ps.accumulate_gradient("b", torch.ones(2)), ps.accumulate_gradient("b", torch.ones(2))
    ps.apply_momentum(0.9, 0.1)
    assert torch.allclose(ps.get_param("b"), torch.full((2,), 0.8))
    ps.accumulate_gradient("b", torch.zeros(2))
    ps.apply_momentum(0.9, 0.1)                                   # the velocity carries on: v = 0.9 * 2
    assert torch.allclose(ps.get_param("b"), torch.full((2,), 0.8 - 0.18))
    ps.set_max_stale_gradients(0)
    assert not ps.update_gradient("a", torch.ones(3), 0)          # computed against version 0, now 2: too stale
    ps.remove_param("a")
    assert ps.list_params() == ["b"]
    ps.clear_params()
    assert ps.list_params() == []
    ps.barrier(), ps.shutdown()
