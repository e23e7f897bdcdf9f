"""quant_evaluate: ``--model --model-dir --task perplexity|accuracy|classification|generation|hellaswag|all
--data --batch-size --context --max-tokens`` (tools/evaluate.cpp:29-159)."""
from __future__ import annotations

import argparse
import os
import sys

from .common import add_int, load_tokenizer, model_dtype, pick_device


def main(argv=None):
    ap = argparse.ArgumentParser(prog="quant_evaluate", epilog="Tasks: perplexity, accuracy, classification, generation, hellaswag, all")
    ap.add_argument("--model", default="")
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--task", default="perplexity")
    ap.add_argument("--data", default="")
    add_int(ap, "--batch-size", 1)
    add_int(ap, "--context", 512)
    add_int(ap, "--max-tokens", 0)
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    if not a.model:
        print("Error: --model required", file=sys.stderr)
        return 1
    import torch

    from ..quant import codec
    from ..utils.metrics import ModelEvaluator, eval_classification, load_eval_tokens
    dev = pick_device(a.device)
    try:
        model = codec.load_model(a.model, device=dev, dtype=model_dtype(dev))
    except (ValueError, OSError, KeyError) as e:
        print(f"Error loading model: {e}", file=sys.stderr)
        return 1
    tok = load_tokenizer(a.model, a.model_dir or os.path.dirname(a.model))
    print(f"Tokenizer loaded ({tok.vocab_size} vocab)")
    print(f"Model loaded: {model.cfg.num_params()} params")
    toks = []
    if a.data:
        toks = [t % model.cfg.vocab_size for t in load_eval_tokens(a.data, a.max_tokens, tok)]
        print(f"Loaded {len(toks)} eval tokens")
    ev = ModelEvaluator(model, a.batch_size)
    ctx = min(a.context, model.cfg.max_seq_len)
    if a.task in ("perplexity", "all") and toks:
        r = ev.evaluate_perplexity(toks, "perplexity", ctx, max(1, ctx // 2))
        print(f"Perplexity: {r.perplexity:.6g} (tokens: {r.total_tokens})")
    if a.task in ("accuracy", "all") and toks:
        r = ev.evaluate_accuracy(toks, "accuracy", ctx)
        print(f"Accuracy: {r.accuracy * 100.0:.6g}% ({r.correct}/{r.total})")
    if a.task in ("generation", "all"):
        r = ev.evaluate_generation(min(32, ctx // 2), 128, "generation")
        print(f"Generation speed: {r.tokens_per_sec:.6g} tok/s")
    if a.task in ("classification", "all") and len(toks) > 1:
        n = min(len(toks) - 1, ctx)
        with torch.no_grad():
            logits = model.forward(torch.tensor([toks[:n]], device=dev))[0].float().cpu()
        cr = eval_classification(logits, toks[1:n + 1])
        print(f"Classification accuracy: {cr.accuracy * 100.0:.6g}% f1: {cr.f1_score:.6g} precision: {cr.precision:.6g} recall: {cr.recall:.6g}")
    if a.task in ("hellaswag", "all"):
        print("HellaSwag eval requires context/ending data -- skipped")
    print("Evaluation complete.")
    return 0


if __name__ == "__main__":
    sys.exit(main())
