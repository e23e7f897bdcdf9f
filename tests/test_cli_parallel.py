"""quant_train under torch.distributed.run on CPU (gloo): data-parallel ZeRO, tensor-parallel and pipeline-parallel meshes
all train, log from rank 0 only and leave a loadable checkpoint; bad meshes are refused with exit code 2."""
import json
import os
import subprocess
import sys

import pytest

from transformers_fusion_b200.parallel.launch import mesh_coords, mesh_groups

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_mesh_layout():
    tpg, dpg, ppg = mesh_groups(8, 2, 2, 2)
    assert tpg[0] == [0, 1] and tpg[-1] == [6, 7] and dpg[0] == [0, 2] and ppg[0] == [0, 4] and ppg[-1] == [3, 7]
    assert mesh_coords(5, 2, 2, 2) == (1, 0, 1)
    seen = sorted(r for g in tpg for r in g)
    assert seen == list(range(8)) and sorted(r for g in ppg for r in g) == list(range(8))
    with pytest.raises(AssertionError):
        mesh_groups(8, 3, 2, 1)


def _train(tmp_path, name, flags, nproc=2):
    data = tmp_path / "corpus.txt"
    if not data.exists():
        data.write_text("the quick brown fox jumps over the lazy dog. " * 400)
    cfgp = tmp_path / "cfg.json"
    cfgp.write_text(json.dumps({"hidden_size": 32, "num_layers": 2, "num_heads": 2, "num_kv_heads": 2, "ffn_hidden_size": 64}))
    model = str(tmp_path / f"{name}.quant")
    port = 29600 + (os.getpid() % 80) + len(name)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "transformers_fusion_b200.cli", "quant_train", "--model", model, "--data", str(data),
           "--config", str(cfgp), "--batch-size", "4", "--seq-length", "16", "--vocab-size", "280", "--max-steps", "12", "--epochs", "1",
           "--log-interval", "4", "--lr", "3e-3", "--optimizer", "adamw", "--device", "cpu"] + flags
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, cwd=ROOT)
    return r, model


@pytest.mark.parametrize("name,flags", [("dp", ["--zero-stage", "2"]), ("tp", ["--tp", "2"]), ("pp", ["--pp", "2"]), ("fsdp", ["--zero-stage", "3"])])
def test_train_cli_meshes(tmp_path, name, flags):
    r, model = _train(tmp_path, name, flags)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    steps = [l for l in r.stdout.splitlines() if l.startswith("Step ")]
    assert steps and len(steps) <= 4, r.stdout                  # rank 0 only
    first, last = (float(l.split("loss:")[1].split("|")[0]) for l in (steps[0], steps[-1]))
    assert last < first, (first, last)
    assert os.path.exists(model) and os.path.exists(model + ".vocab")
    from transformers_fusion_b200.quant.codec import load_model
    m = load_model(model)
    assert m.cfg.hidden_size == 32 and m.cfg.num_layers == 2


def test_train_cli_rejects_bad_mesh(tmp_path):
    r, _ = _train(tmp_path, "bad", ["--tp", "3"])
    assert r.returncode != 0 and "does not divide" in (r.stdout + r.stderr)


@pytest.mark.parametrize("name,flags", [("dp2tp2", ["--tp", "2", "--dp", "2"]), ("dp2pp2", ["--pp", "2", "--dp", "2"])])
def test_train_cli_two_dimensional_meshes(tmp_path, name, flags):
    """Four gloo ranks: data parallel x tensor parallel and data parallel x pipeline (the groups of mesh_groups in use)."""
    r, model = _train(tmp_path, name, flags, nproc=4)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    steps = [l for l in r.stdout.splitlines() if l.startswith("Step ")]
    first, last = (float(l.split("loss:")[1].split("|")[0]) for l in (steps[0], steps[-1]))
    assert last < first and os.path.exists(model)
    assert "dp=2" in r.stdout
