import json
import os
import subprocess
import sys

from transformers_fusion_b200.parallel.pp import DualPipe, split_model

HERE = os.path.dirname(os.path.abspath(__file__))


def test_split_model():
    assert split_model(12, 4) == [(0, 3), (3, 6), (6, 9), (9, 12)]
    assert split_model(10, 4) == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert split_model(8, 2, [3, 1]) == [(0, 6), (6, 8)]
    s = DualPipe(4, 8).schedule()
    assert len(s) == 4 + 3 and s[0][0] == [("down", 0, "F")] and s[0][3] == [("up", 4, "F")]


def test_pipeline_matches_single_process(tmp_path):
    port = 29800 + (os.getpid() % 90)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mp_pp_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=120, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = [json.load(open(os.path.join(tmp_path, f"rank{i}.json"))) for i in range(2)]
    for sched in ("gpipe", "1f1b"):
        assert res[1][f"{sched}_loss_err"] < 1e-4
        assert res[0][f"{sched}_grad_err"] < 1e-4 and res[1][f"{sched}_grad_err"] < 1e-4
    assert res[0]["1f1b_live"] == 2 and res[1]["1f1b_live"] == 1 and res[0]["gpipe_live"] == 4
    for r in res:
        assert r["tied_norm_err"] < 1e-4
        assert r["tied_grad_err"] < 1e-5 and r["tied_param_err"] < 1e-5
    assert res[1]["fwd_logits_err"] < 1e-4 and res[1]["fwd_loss_err"] < 1e-4
    assert all(r["two_call_loss"] and r["stage_params"] > 0 for r in res)


def test_stage_and_context_accessors():
    import torch
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.parallel.pp import PipelineParallel, PipelineStage
    m = DenseModel(TransformerConfig(vocab_size=32, hidden_size=16, num_layers=4, num_heads=2, ffn_hidden_size=32, max_seq_len=16), device="cpu",
                   dtype=torch.float32, seed=0)
    pp = PipelineParallel(m, 2, 1)
    st = pp.stage()
    assert isinstance(st, PipelineStage) and (st.layer_start, st.layer_end, st.device_id) == (2, 4, 0) and st.model_segment is m
    assert pp.context() is pp.ctx and pp.context().rank == 1
