"""quant_infer: ``<model.quant> [prompt] [--model-dir DIR] [--seed N]``; temperature .7, top_k 40, top_p .9,
max 512 tokens; prints the completion and tok/s (tools/infer.cpp:15-108)."""
from __future__ import annotations

import argparse
import sys
import time

from .common import add_int, load_tokenizer, model_dtype, pick_device, resolve_base_seed


def main(argv=None):
    ap = argparse.ArgumentParser(prog="quant_infer")
    ap.add_argument("model")
    ap.add_argument("prompt", nargs="?", default="Hello")
    ap.add_argument("--model-dir", default="")
    add_int(ap, "--seed", 0)
    add_int(ap, "--max-tokens", 512)
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8", "q4"])
    ap.add_argument("--weights", default="", choices=["", "int8", "int4", "mxfp8", "fp4", "ternary"],
                    help="serve the block matrices from this low-bit format with the fused-dequant GEMM")
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    from ..inference.engine import EngineConfig, InferenceEngine
    from ..inference.sampler import SamplerConfig
    from ..quant import codec
    dev = pick_device(a.device)
    try:
        model = codec.load_model(a.model, device=dev, dtype=model_dtype(dev))
    except (ValueError, OSError) as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    tok = load_tokenizer(a.model, a.model_dir)
    eng = InferenceEngine(model, tok, EngineConfig(kv_mode=a.kv, seed=resolve_base_seed(a.seed), num_pages=1024, weight_format=a.weights))
    t0 = time.perf_counter()
    n0 = eng.stats.generated_tokens
    text = eng.generate(a.prompt, min(a.max_tokens, model.cfg.max_seq_len - 1), SamplerConfig(0.7, 40, 0.9))
    dt = time.perf_counter() - t0
    print(text)
    print(f"[{eng.stats.generated_tokens - n0} tokens, {(eng.stats.generated_tokens - n0) / max(dt, 1e-9):.2f} tok/s]")
    return 0


if __name__ == "__main__":
    sys.exit(main())
