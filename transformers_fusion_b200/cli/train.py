"""quant_train: dense pre-training from a text file.  Flags and log line follow tools/train.cpp:36-192
(``--model --data --config --batch-size --seq-length --epochs --lr --vocab-size --hidden-size
--num-layers --num-heads --log-interval --save-interval --optimizer adafactor|adamw --seed``); new:
``--zero-stage/--resume/--device/--max-steps``, an honoured ``--config`` JSON, and the mesh flags ``--dp --tp --pp --ep``
for jobs started with ``python -m torch.distributed.run`` (one process per GPU; see parallel/launch.py)."""
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
    add_int(ap, "--dp", 0, "Data-parallel degree (0 = world size / (tp x pp))")
    add_int(ap, "--tp", 1, "Tensor-parallel degree (sequence parallel between the TP regions)")
    add_int(ap, "--pp", 1, "Pipeline stages (1F1B)")
    add_int(ap, "--ep", 1, "Expert-parallel degree (MoE models)")
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
    from ..parallel.launch import fit_parallel, init_parallel, shutdown
    seed = resolve_base_seed(args.seed)
    os.environ["QUANT_SEED"] = str(seed)
    torch.manual_seed(seed)
    over = json.load(open(args.config)) if args.config and os.path.exists(args.config) else {}
    try:
        st = init_parallel(args.dp, args.tp, args.pp, args.ep, args.device)
    except ValueError as e:
        print(f"Error: {e}", file=sys.stderr)
        return 2
    dev = st.device if st.world > 1 else pick_device(args.device)
    # tokenizer: BPE trained on the first <= 64 MiB of the corpus (tools/train.cpp:119-156); deterministic, so every
    # rank trains the same vocabulary and only rank 0 writes it
    text = open(args.data, "r", encoding="utf-8", errors="ignore").read(64 << 20)
    tok = BPETokenizer().train([text], args.vocab_size)
    if st.is_main:
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
    line = lambda step, loss, ppl, lr, tps: print(f"Step {step} | loss: {loss:.6g} | ppl: {ppl:.6g} | lr: {lr:.6g} | tok/s: {tps:.6g}",
                                                  flush=True)
    if st.is_main:
        print(f"Using {'AdamW' if args.optimizer.lower() == 'adamw' else args.optimizer.capitalize()} optimizer via UnifiedTrainer ({args.kind}).")
    if st.world > 1:
        if st.is_main:
            print(f"Parallel mesh: dp={st.dp} tp={st.tp} pp={st.pp} ep={st.ep} on {st.world} ranks")
        fit_parallel(model, tok, args.data, tcfg, st, line, args.resume)
        shutdown(st)
    else:
        tr = Trainer(model, tok).compile(None, tcfg)
        tr.set_log_callback(lambda m: line(m.step, m.loss, m.perplexity, m.learning_rate, m.tokens_per_sec))
        dl = DataLoader(tok, args.data, args.batch_size, args.seq_length, device=dev)
        if args.resume and os.path.exists(args.model):
            tr.load_checkpoint(args.model, dl)
        tr.fit(dl)
    if st.is_main:
        print(f"Training complete. Model saved to {args.model}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
