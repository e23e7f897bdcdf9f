"""Expert parallelism with the fused dispatch / combine kernels on >= 2 GPUs."""
import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_expert_parallel_matches_single_rank(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    n = 2 if torch.cuda.device_count() < 4 else 4
    port = 29700 + (os.getpid() % 90)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_mp_ep_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for i in range(n):
        res = json.load(open(os.path.join(tmp_path, f"rank{i}.json")))
        assert res["status"] == 0, res
        for key, v in res.items():
            if key != "status":
                assert v < 4e-2, (key, v, res)


def test_assign_experts_contiguous():
    from transformers_fusion_b200.parallel.ep import assign_experts
    assert assign_experts(8, 4) == [[0, 1], [2, 3], [4, 5], [6, 7]]


@pytest.mark.gpu
def test_ep_model_training(tmp_path):
    """Expert-parallel MoE model on 2 GPUs: forward loss equals the unsharded model's, training reduces it, replicated
    weights stay in step."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = 29950 + (os.getpid() % 40)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mp_epmodel_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for i in range(2):
        res = json.load(open(os.path.join(tmp_path, f"rank{i}.json")))
        assert res["status"] == 0 and res["local_experts"] == 2
        assert abs(res["ep_loss"] - res["ref_loss"]) < 0.03 * abs(res["ref_loss"]), res
        assert res["g_qkv"] < 0.05 and res["g_down_has_remote_tokens"]
        assert res["losses"][-1] < res["losses"][0] - 0.2, res["losses"]
        assert res["replicated_in_sync"]
