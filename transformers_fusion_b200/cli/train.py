"""quant_train: dense pre-training from a text file.  Flags and log line follow tools/train.cpp:36-192
(``--model --data --config --batch-size --seq-length --epochs --lr --vocab-size --hidden-size
--num-layers --num-heads --log-interval --save-interval --optimizer adafactor|adamw --seed``); new:
``--dp/--zero-stage/--resume/--device/--max-steps`` and an honoured ``--config`` JSON."""
from __future__ import annotations

import argparse
import json
import os
import sys

from .common import add_float, add_int, load_tokenizer, model_dtype, pick_device, resolve_base_seed


def build_parser():
    ap = argparse.ArgumentParser(prog="quant_train", description="Usage: quant_train --model model.quant --data data.txt [options]")
    ap.add_argument("--model", default="model.quant")
    ap.add_argument("--data", default="")
    ap.add_argument("--config", default="")
    add_int(ap, "--batch-size", 8, "Batch size (default: 8)")
    add_int(ap, "--seq-length", 512, "Sequence length (default: 512)")
    add_int(ap, "--epochs", 3, "Number of epochs (default: 3)")
    add_float(ap, "--lr", 3e-4, "Learning rate (default: 3e-4)")
    add_int(ap, "--vocab-size", 32000)
    add_int(ap, "--hidden-size", 768)
    add_int(ap, "--num-layers", 12)
    add_int(ap, "--num-heads", 12)
    add_int(ap, "--log-interval", 10)
    add_int(ap, "--save-interval", 1000)
    ap.add_argument("--optimizer", default="adafactor", help="'adafactor' or 'adamw' (default: adafactor)")
    add_int(ap, "--seed", 0, "Base seed (0=default 42, or QUANT_SEED env)")
    add_int(ap, "--max-steps", 10000)
    add_int(ap, "--zero-stage", 0)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--kind", default="dense")
    return ap


def main(argv=None):
    args = build_parser().parse_args(argv)
    if not args.data or not os.path.exists(args.data):
        print(f"Error: cannot open data file '{args.data}'", file=sys.stderr)
        return 1
    import torch

    from ..models.config import TransformerConfig
    from ..models.dense import DenseModel
    from ..tokenizer import BPETokenizer
    from ..trainer.trainer import DataLoader, TrainConfig, Trainer
    seed = resolve_base_seed(args.seed)
    os.environ["QUANT_SEED"] = str(seed)
    torch.manual_seed(seed)
    over = json.load(open(args.config)) if args.config and os.path.exists(args.config) else {}
    dev = pick_device(args.device)
    # tokenizer: BPE trained on the first <= 64 MiB of the corpus (tools/train.cpp:119-156)
    text = open(args.data, "r", encoding="utf-8", errors="ignore").read(64 << 20)
    tok = BPETokenizer().train([text], args.vocab_size)
    tok.save(args.model + ".vocab")
    heads = over.get("num_heads", args.num_heads)
    cfg = TransformerConfig(vocab_size=max(tok.vocab_size, 8), hidden_size=over.get("hidden_size", args.hidden_size),
                            num_layers=over.get("num_layers", args.num_layers), num_heads=heads,
                            num_kv_heads=over.get("num_kv_heads", heads), ffn_hidden_size=over.get("ffn_hidden_size", 0),
                            max_seq_len=max(args.seq_length, over.get("max_seq_len", args.seq_length)))
    model = DenseModel(cfg, device=dev, dtype=model_dtype(dev), seed=seed)
    tcfg = TrainConfig(batch_size=args.batch_size, seq_length=args.seq_length, epochs=args.epochs, learning_rate=args.lr,
                       log_interval=args.log_interval, save_interval=args.save_interval, optimizer=args.optimizer.lower(),
                       checkpoint_path=args.model, max_steps=args.max_steps, seed=seed, zero_stage=args.zero_stage)
    tr = Trainer(model, tok).compile(None, tcfg)
    tr.set_log_callback(lambda m: print(f"Step {m.step} | loss: {m.loss:.6g} | ppl: {m.perplexity:.6g} | lr: {m.learning_rate:.6g}"
                                        f" | tok/s: {m.tokens_per_sec:.6g}", flush=True))
    print(f"Using {'AdamW' if args.optimizer.lower() == 'adamw' else args.optimizer.capitalize()} optimizer via UnifiedTrainer ({args.kind}).")
    dl = DataLoader(tok, args.data, args.batch_size, args.seq_length, device=dev)
    if args.resume and os.path.exists(args.model):
        tr.load_checkpoint(args.model, dl)
    tr.fit(dl)
    print(f"Training complete. Model saved to {args.model}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
