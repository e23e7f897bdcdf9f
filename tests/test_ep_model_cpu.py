"""Model-level expert parallelism with replicated tokens (the reference's algorithm) on two gloo ranks."""
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_replicated_token_expert_parallel_matches_single_process(tmp_path):
    port = 29950 + (os.getpid() % 40)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mp_ep_model_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = [json.load(open(os.path.join(tmp_path, f"rank{i}.json"))) for i in range(2)]
    assert res[0]["local"] == [0, 1] and res[1]["local"] == [2, 3]
    for r_ in res:
        assert r_["logits_err"] < 1e-4 and r_["loss_err"] < 1e-5 and r_["grad_err"] < 1e-4, r_
        assert r_["foreign_grad"] == 0.0 and r_["n_local"] == 2
        assert r_["gathered"] == [0.0, 0.0, 1.0, 1.0]
