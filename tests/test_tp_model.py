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


def test_head_partitioner_and_parallel_linear_accessors():
    import torch
    from transformers_fusion_b200.parallel.tp import ColumnParallelLinear, HeadPartitioner, RowParallelLinear, SequenceParallel, TensorParallelManager
    hp = HeadPartitioner(8, 2, 4, rank=2, head_dim=4)
    assert (hp.head_start(), hp.head_end(), hp.heads_per_rank()) == (4, 6, 2) and hp.q_heads(2) == [4, 5] and hp.kv_heads(2) == [1]
    x = torch.arange(2 * 32.0).view(2, 32)
    loc = hp.partition_heads(x)
    assert loc.shape == (2, 8) and loc[0].tolist() == list(range(16, 24))
    one = HeadPartitioner(8, 8, 1, head_dim=4)
    assert torch.equal(one.merge_heads(one.partition_heads(x)), x) and one.sync_output(x.clone()).equal(x)
    w = torch.randn(12, 8)
    col, row = ColumnParallelLinear(w, 1, 2), RowParallelLinear(w, 1, 2)
    assert col.local_out_features() == 6 and torch.equal(col.local_weight().data, w[6:]) and col.local_bias() is None
    assert row.local_in_features() == 4 and torch.equal(row.local_weight().data, w[:, 4:])
    sp = SequenceParallel(1, 2)
    assert sp.world_size() == 2 and sp.world_rank() == 1 and sp.allreduce(x) is x
    m = TensorParallelManager(None, 4, 3)
    assert m.world_size() == 4 and m.world_rank() == 3
