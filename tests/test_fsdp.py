import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(n, backend, tmp_path, env):
    port = 29600 + (os.getpid() % 90) + (5 if backend == "nccl" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mp_fsdp_worker.py"), str(tmp_path), backend]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, **env))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return [json.load(open(os.path.join(tmp_path, f"rank{i}.json"))) for i in range(n)]


def test_zero3_matches_single_process_gloo(tmp_path):
    for res in _launch(2, "gloo", tmp_path, {"CUDA_VISIBLE_DEVICES": ""}):
        assert res["n_sharded"] >= 8 and res["savings"] > 0.3 and res["gathers"] > 20
        for a, b in zip(res["losses"], res["ref_losses"]):
            assert abs(a - b) < 2e-4, res
        assert res["param_err"] < 2e-4, res


@pytest.mark.gpu
@pytest.mark.multigpu
def test_zero3_fused_weight_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for res in _launch(2, "nccl", tmp_path, {"NCCL_NVLS_ENABLE": "0"}):
        assert res["status"] == 0, res
        for a, b in zip(res["losses"], res["ref_losses"]):
            assert abs(a - b) < 5e-2, res
        assert res["param_err"] < 5e-2, res
        assert res["losses"][-1] < res["losses"][0]


def test_offload_and_checkpointing_helpers():
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.parallel.fsdp import ActivationCheckpointing, CPUOffloadEngine, FullyShardedDataParallel
    eng = CPUOffloadEngine(pool_bytes=1 << 20, device="cpu")
    t = torch.arange(1000.0)
    eng.offload("m", t)
    assert torch.equal(eng.fetch("m"), t)
    with pytest.raises(MemoryError):
        eng.offload("big", torch.zeros(1 << 20))
    eng.release("m")
    assert eng.used == 0
    m = DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=3, num_heads=4, ffn_hidden_size=64, max_seq_len=16),
                   device="cpu", dtype=torch.float32, seed=0)
    ac = ActivationCheckpointing(m).enable()
    assert m.activation_checkpointing and ac.memory_saved_bytes(2, 16) > 0
    assert FullyShardedDataParallel.auto_wrap(m, 1000) == ["layers.0", "layers.1", "layers.2"]
