"""ZeRO-3 x tensor-parallel engine against a single-process run (CPU ranks over gloo here; GPU ranks in the gpu tests)."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(tmp_path, nproc, tp, comm, extra=(), env=None, timeout=240):
    port = 29300 + (os.getpid() * 7 + nproc * 3 + tp) % 500
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mp_sharded_worker.py"), str(tmp_path), str(tp), comm, *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env or dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return [json.load(open(os.path.join(tmp_path, f"rank{i}.json"))) for i in range(nproc)]


@pytest.mark.parametrize("nproc,tp,extra", [(4, 2, ()), (2, 1, ()), (2, 2, ("tied",)), (4, 1, ("tied",))])
def test_sharded_engine_matches_single_process_cpu(tmp_path, nproc, tp, extra):
    res = _run(tmp_path, nproc, tp, "gloo", extra)
    for r in res:
        assert max(r["loss_err"]) < 2e-4, r
        assert r["weight_err"] < 2e-3, r
        assert abs(r["grad_norm"] - r["ref_grad_norm"]) < 1e-3 * max(1.0, r["ref_grad_norm"]), r
        if nproc // tp > 1:
            assert r["gathers"] > 0       # (the toy matrices are padded to 128 rows per rank: no memory claim here)


def _gpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.gpu
@pytest.mark.parametrize("nproc,tp,comm", [(2, 1, "fused"), (2, 1, "fused_in_gemm"), (2, 2, "fused"), (4, 2, "fused"),
                                           (4, 2, "fused_in_gemm"), (4, 2, "nccl")])
def test_sharded_engine_matches_single_process_gpu(tmp_path, nproc, tp, comm):
    if _gpus() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    res = _run(tmp_path, nproc, tp, comm, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    for r in res:
        assert max(r["loss_err"]) < 5e-2, r
        assert r["weight_err"] < 8e-2, r
        assert abs(r["grad_norm"] - r["ref_grad_norm"]) < 5e-2 * max(1.0, r["ref_grad_norm"]), r
