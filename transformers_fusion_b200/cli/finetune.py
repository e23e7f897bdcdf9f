"""quant_finetune: ``--model --data --output(finetuned.quant) --lr(1e-5) --epochs(1) --batch-size(4)
--seq-length(512) --optimizer`` (tools/finetune.cpp:24-103); ``--lora-rank N`` trains rank adapters only."""
from __future__ import annotations

import argparse
import os
import sys

from .common import add_float, add_int, load_tokenizer, model_dtype, pick_device


def main(argv=None):
    ap = argparse.ArgumentParser(prog="quant_finetune")
    ap.add_argument("--model", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--output", default="finetuned.quant")
    add_float(ap, "--lr", 1e-5)
    add_int(ap, "--epochs", 1)
    add_int(ap, "--batch-size", 4)
    add_int(ap, "--seq-length", 512)
    ap.add_argument("--optimizer", default="adamw")
    ap.add_argument("--model-dir", default="")
    add_int(ap, "--lora-rank", 0)
    add_int(ap, "--max-steps", 10000)
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    for p in (a.model, a.data):
        if not os.path.exists(p):
            print(f"Error: cannot open '{p}'", file=sys.stderr)
            return 1
    from ..quant import codec
    from ..trainer.trainer import DataLoader, TrainConfig, Trainer
    dev = pick_device(a.device)
    model = codec.load_model(a.model, device=dev, dtype=model_dtype(dev))
    tok = load_tokenizer(a.model, a.model_dir)
    seq = min(a.seq_length, model.cfg.max_seq_len)
    cfg = TrainConfig(batch_size=a.batch_size, seq_length=seq, epochs=a.epochs, learning_rate=a.lr, optimizer=a.optimizer.lower(),
                      checkpoint_path=a.output, warmup_steps=0, zero_stage=0, max_steps=a.max_steps, save_interval=0)
    dl = DataLoader(tok, a.data, a.batch_size, seq, device=dev)
    if a.lora_rank > 0:
        from ..trainer.finetune import RankAdapterEngine
        eng = RankAdapterEngine(model, rank=a.lora_rank, lr=a.lr)
        for _ in range(min(a.max_steps, a.epochs * max(1, len(dl)))):
            loss = eng.train_step(*dl.next_batch())
        eng.merge_into_base()
        codec.save_model(model, a.output)
        eng.save_adapters(a.output + ".nrad")
    else:
        tr = Trainer(model, tok).compile(None, cfg)
        tr.set_log_callback(lambda m: print(f"Step {m.step} | loss: {m.loss:.6g} | lr: {m.learning_rate:.6g}", flush=True))
        tr.fit(dl)
    print(f"Fine-tuning complete. Model saved to {a.output}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
