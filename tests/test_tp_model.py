"""Tensor-parallel + sequence-parallel dense model against the single-rank model: gloo ranks on CPU (collective +
GEMM path) and, on a multi-GPU box, NCCL ranks with the fused all-gather->GEMM / GEMM->reduce-scatter kernels."""
import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(tmp_path, n, where, extra_env=None):
    port = 29700 + (os.getpid() % 90) + (5 if where == "cuda" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mp_tpmodel_worker.py"), str(tmp_path), where]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, env=dict(os.environ, **(extra_env or {})))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return [json.load(open(os.path.join(tmp_path, f"rank{i}.json"))) for i in range(n)]


def _check(results, tol):
    for res in results:
        for k in ("loss_err", "g_qkv", "g_o", "g_down", "g_gate_up", "g_attn_norm", "g_final_norm", "g_embed"):
            assert res[k] < tol, (k, res[k])
        assert res["losses"][-1] < res["losses"][0] - 0.02, res["losses"]
        assert abs(res["gathered_loss"] - res["losses"][-1]) < 0.5        # one more update lies between the two
    assert all(abs(a - b) < 1e-4 * max(1, abs(a)) for a, b in zip(results[0]["losses"], results[1]["losses"]))


def test_tp_model_matches_dense_cpu(tmp_path):
    _check(_run(tmp_path, 2, "cpu"), 2e-4)


@pytest.mark.gpu
def test_tp_model_matches_dense_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = _run(tmp_path, 2, "cuda", {"NCCL_NVLS_ENABLE": "0"})
    assert all(r["status"] == 0 for r in res)
    _check(res, 4e-2)
