"""Fused tensor-parallel GEMMs on >= 2 GPUs against the single-device product."""
import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fused_tp_gemms(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    n = 2 if torch.cuda.device_count() < 4 else 4
    port = 29900 + (os.getpid() % 90)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_mp_tp_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for i in range(n):
        res = json.load(open(os.path.join(tmp_path, f"rank{i}.json")))
        assert res["status"] == 0, res
        for k, v in res.items():
            if k.endswith(("_0", "_1", "_2")):
                assert v < 2e-2, (k, v)


def test_split_helpers():
    from transformers_fusion_b200.parallel import tp
    w = torch.arange(24.0).view(6, 4)
    shards = [tp.column_parallel_split(w, 4, r) for r in range(4)]
    assert [s.shape[0] for s in shards] == [2, 2, 2, 0] and torch.equal(tp.reconstruct_weight(shards[:3]), w)
    assert torch.equal(tp.reconstruct_weight([tp.row_parallel_split(w, 2, r) for r in range(2)], column=False), w)
    assert tp.partition_heads(8, 4, 3) == [6, 7] and tp.partition_heads(5, 4, 3) == []
    v = tp.communication_volume(4096, 4096, 4096, 2)
    assert v["all_gather"] == 2048 * 4096 * 2 and v["total"] == 2 * v["all_gather"]


def test_tensor_parallel_manager_api():
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.parallel import tp
    cfg = TransformerConfig(vocab_size=64, hidden_size=64, num_layers=1, num_heads=4, num_kv_heads=2, ffn_hidden_size=128, max_seq_len=16)
    m = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0)
    shards = [tp.TensorParallelManager(m, 2, r).parallelize_model() for r in range(2)]
    assert torch.equal(torch.cat([shards[r][0]["q"] for r in range(2)], 0), m.layers[0].qkv.data[:64])
    assert torch.equal(torch.cat([shards[r][0]["o"] for r in range(2)], 1), m.layers[0].o.data)
    assert torch.equal(torch.cat([shards[r]["lm_head"] for r in range(2)], 0), m.lm_head.data)
    mgr = tp.TensorParallelManager(m, 1, 0)
    x = torch.randn(4, 64)
    assert torch.allclose(mgr.column_parallel_linear(x, m.layers[0].o.data), x @ m.layers[0].o.data.t(), atol=1e-5)
    assert torch.allclose(mgr.row_parallel_linear(x, m.layers[0].o.data), x @ m.layers[0].o.data.t(), atol=1e-5)
    assert tp.TensorParallelManager.select_strategy(cfg, 1) == "none"
    assert tp.TensorParallelManager.select_strategy(TransformerConfig(hidden_size=4096, num_heads=32, num_layers=2), 8, 8192) == "tp+sp"
    assert tp.HeadPartitioner(8, 2, 4).kv_heads(3) == [1] and tp.HeadPartitioner(8, 2, 4).q_heads(0) == [0, 1]
    assert tp.SequenceParallel(1, 2).scatter(torch.arange(8).view(1, 8)).tolist() == [[4, 5, 6, 7]]
