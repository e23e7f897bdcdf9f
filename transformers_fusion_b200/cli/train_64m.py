"""train_64m [--test] [--steps N]: trains the 67M-parameter configuration (14 layers, d512, 8 heads, ffn 2048, vocab 8192,
batch 8 x 2048) on a synthetic token stream in the native quantised-weight representation; ``--test`` runs 5 batches
(tools/train_64m.cpp:62-140).  ``bench_speed`` mode (``--bench``) times 20 plain training steps after 5 warm-up steps
(tools/bench_speed.cpp)."""
from __future__ import annotations

import argparse
import sys
import time

from .common import add_int, model_dtype, pick_device


def main(argv=None):
    ap = argparse.ArgumentParser(prog="train_64m")
    ap.add_argument("--test", action="store_true")
    ap.add_argument("--bench", action="store_true")
    add_int(ap, "--steps", 0)
    add_int(ap, "--batch", 8)
    add_int(ap, "--seq", 2048)
    add_int(ap, "--layers", 14)
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    import torch

    from ..models.config import TransformerConfig
    from ..models.dense import DenseModel
    from ..trainer.native_quant import NativeQUANTTrainer, NativeTrainConfig
    dev = pick_device(a.device)
    B, S = a.batch, a.seq
    cfg = TransformerConfig(vocab_size=8192, hidden_size=512, num_layers=a.layers, num_heads=8, head_dim=64, ffn_hidden_size=2048, max_seq_len=max(S, 16))
    print("================================================")
    print("  64M-parameter training run" + ("  (QUICK TEST MODE: %d tokens)" % (B * S * 5) if a.test else ""))
    print("================================================\n")
    model = DenseModel(cfg, device=dev, dtype=model_dtype(dev), seed=42)
    n = cfg.num_params()
    print(f"Model: {n} params ({n / 1e6:.1f}M)", flush=True)
    g = torch.Generator().manual_seed(42)

    def batch():
        ids = torch.randint(0, cfg.vocab_size - 1, (B, S), generator=g)
        return ids.to(dev), torch.roll(ids, -1, 1).to(dev)
    steps = a.steps or (5 if a.test else 1000)
    if a.bench:
        from ..trainer.engine import TrainEngine
        eng = TrainEngine(model, lr=1e-4, zero_stage=0)
        print("\n--- Benchmarking 20 steps ---", flush=True)
        for step in range(25):
            ids, lab = batch()
            if dev.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            loss = float(eng.step(ids, lab, 1e-4))
            if dev.type == "cuda":
                torch.cuda.synchronize()
            ms = (time.perf_counter() - t0) * 1e3
            if step >= 5:
                print(f"  step {step}: {ms:.0f} ms, {B * S / (ms / 1e3):.0f} tok/s", flush=True)
        return 0
    tr = NativeQUANTTrainer(model, NativeTrainConfig(warmup_steps=min(2, steps), lr_scale=1e-4, lr_weight=1e-4))
    t0 = time.perf_counter()
    for step in range(steps):
        m = tr.train_step(*batch())
        print(f"Step {step + 1} | loss: {m.loss:.6g} | native: {int(tr.native)} | frozen: {m.frozen_fraction:.3f} | "
              f"q8/q1/q4 blocks: {m.quant8_count}/{m.quant1_count}/{m.quant_count} | tok/s: {(step + 1) * B * S / (time.perf_counter() - t0):.6g}",
              flush=True)
    print("Training complete.")
    return 0


if __name__ == "__main__":
    sys.exit(main())
