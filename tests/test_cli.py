"""Command-line tools end to end on CPU: train -> info -> quantize -> infer -> evaluate -> convert."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(tool, *args, expect=0):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, "-m", "transformers_fusion_b200.cli", tool, *map(str, args)], capture_output=True, text=True,
                       env=env, timeout=600)
    assert p.returncode == expect, p.stdout[-2000:] + p.stderr[-2000:]
    return p.stdout, p.stderr


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    d = tmp_path_factory.mktemp("cli")
    text = ("the quick brown fox jumps over the lazy dog. " * 40 + "pack my box with five dozen liquor jugs. " * 40) * 3
    (d / "data.txt").write_text(text)
    out, _ = run("quant_train", "--model", d / "m.quant", "--data", d / "data.txt", "--batch-size", 2, "--seq-length", 32, "--epochs", 1,
                 "--vocab-size", 300, "--hidden-size", 64, "--num-layers", 2, "--num-heads", 4, "--log-interval", 5, "--optimizer", "adamw",
                 "--max-steps", 30, "--lr", "3e-3", "--seed", 7)
    return d, out


def test_train_log_format(trained):
    d, out = trained
    assert "Using AdamW optimizer via UnifiedTrainer (dense)." in out
    lines = [l for l in out.splitlines() if l.startswith("Step ")]
    assert lines and all(" | loss: " in l and " | ppl: " in l and " | lr: " in l and " | tok/s: " in l for l in lines)
    first, last = (float(l.split("loss: ")[1].split(" |")[0]) for l in (lines[0], lines[-1]))
    assert last < first
    assert f"Training complete. Model saved to {d / 'm.quant'}" in out
    assert (d / "m.quant").exists() and (d / "m.quant.vocab").exists()


def test_numeric_flag_error():
    _, err = run("quant_train", "--data", "x", "--batch-size", "abc", expect=2)
    assert "Error: --batch-size has invalid numeric value 'abc'" in err
    _, err = run("quant_convert", "--input", "a", "--output", "b", "--bpw", "99", expect=2)
    assert "--bpw needs 0..32" in err


def test_info_quantize_infer_evaluate(trained):
    d, _ = trained
    out, _ = run("quant_info", d / "m.quant")
    assert "Magic: QUA1" in out and "tok_embeddings.weight" in out and "Total parameters:" in out
    out, _ = run("quant_quantize", "--input", d / "m.quant", "--output", d / "m8.quant", "--format", "q8", "--per-layer", "o_proj=q16")
    assert "Quantized" in out and (d / "m8.quant").stat().st_size < 0.5 * (d / "m.quant").stat().st_size
    out, _ = run("quant_info", d / "m8.quant")
    assert "format=Q_8" in out and "format=Q_16" in out
    _, err = run("quant_quantize", "--input", d / "m.quant", "--output", d / "x.quant", "--format", "zz9", expect=2)
    assert "unknown format" in err
    out, _ = run("quant_infer", d / "m8.quant", "the quick", "--seed", 3, "--max-tokens", 12)
    assert "tok/s]" in out
    out, _ = run("quant_evaluate", "--model", d / "m.quant", "--task", "all", "--data", d / "data.txt", "--context", 32, "--max-tokens", 400)
    assert "Perplexity:" in out and "Accuracy:" in out and "Classification accuracy:" in out and "Evaluation complete." in out
    ppl = float(out.split("Perplexity: ")[1].split(" ")[0])
    assert ppl < 200
    out, _ = run("quant_finetune", "--model", d / "m.quant", "--data", d / "data.txt", "--output", d / "ft.quant", "--batch-size", 2,
                 "--seq-length", 32, "--max-steps", 4)
    assert "Fine-tuning complete" in out and (d / "ft.quant").exists()


def test_convert_and_format_list(tmp_path):
    (tmp_path / "w.bin").write_bytes(np.random.default_rng(0).standard_normal(4096).astype(np.float32).tobytes())
    out, _ = run("quant_convert", "--input", tmp_path / "w.bin", "--output", tmp_path / "w.quant", "--bpw", 4)
    assert "Converted 1 tensors (4096 weights)" in out
    assert (tmp_path / "w.quant").stat().st_size < 4096 * 4 * 0.2
    out, _ = run("quant_format_list")
    assert "Q_G_8_K_M" in out and "Q_32" in out


def test_serve_engine_service_swaps_models_between_requests():
    """The serving bridge of quant_serve: a request runs on the engine that was current when it arrived, a swap waits for
    the old engine to drain, an unloaded service refuses."""
    import torch
    from transformers_fusion_b200.cli.serve import EngineService
    from transformers_fusion_b200.inference.engine import EngineConfig, InferenceEngine
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.tokenizer import ByteTokenizer

    def engine(seed):
        m = DenseModel(TransformerConfig(vocab_size=260, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=64,
                                         max_seq_len=64), device="cpu", dtype=torch.float32, seed=seed)
        return InferenceEngine(m, ByteTokenizer(), EngineConfig(max_batch=2, num_pages=32, max_seq_len=64))
    a, b = engine(1), engine(2)
    svc = EngineService(a, {"max_tokens": 8})
    try:
        first = "".join(svc.generate("hello", 6, 0.0, 1.0, 0, False))
        assert svc.last_usage[0] == 5 and svc.last_usage[1] >= 1
        svc.swap_engine(b)
        assert svc.engine is b and not a.has_pending()
        second = "".join(svc.generate("hello", 6, 0.0, 1.0, 0, False))
        assert isinstance(first, str) and isinstance(second, str)
        svc.swap_engine(a)
        assert "".join(svc.generate("hello", 6, 0.0, 1.0, 0, False)) == first       # greedy: the first model answers as before
        svc.swap_engine(None)
        import pytest as _pt
        with _pt.raises(RuntimeError):
            next(svc.generate("hello", 2, 0.0, 1.0, 0, False))
    finally:
        svc.stop()
