"""Shared pieces of the command-line tools: numeric flag parsing with the reference's error text and
exit code (include/quant/detail/cli_parse.h: ``Error: <flag> has invalid numeric value 'X'``, exit 2),
seed resolution (cli > QUANT_SEED > 42, src/core/random.cpp:113) and device selection."""
from __future__ import annotations

import argparse
import os
import sys


def _num(kind, flag):
    def parse(v):
        try:
            return kind(v)
        except ValueError:
            print(f"Error: {flag} has invalid numeric value '{v}'", file=sys.stderr)
            raise SystemExit(2)
    return parse


def add_int(ap, flag, default, help=""):
    ap.add_argument(flag, type=_num(int, flag), default=default, help=help)


def add_float(ap, flag, default, help=""):
    ap.add_argument(flag, type=_num(float, flag), default=default, help=help)


def resolve_base_seed(cli_seed: int = 0) -> int:
    if cli_seed:
        return int(cli_seed)
    env = os.environ.get("QUANT_SEED", "")
    try:
        return int(env) if env else 42
    except ValueError:
        return 42


def make_seed(base: int, stream: int, counter: int = 0) -> int:
    """splitmix64-style mixing of (base, stream, counter) (reference make_seed, src/core/random.cpp:41)."""
    z = (base + 0x9E3779B97F4A7C15 * (stream + 1) + counter) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


def pick_device(name: str = "auto"):
    import torch
    if name == "auto":
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return torch.device(name)


def model_dtype(device):
    import torch
    return torch.bfloat16 if device.type == "cuda" else torch.float32


def load_tokenizer(model_path: str, model_dir: str = ""):
    """Tokenizer next to the model: HF ``vocab.json`` + ``merges.txt`` in --model-dir, else ``<model>.vocab``
    (trained BPE), else raw bytes."""
    from ..tokenizer import BPETokenizer, ByteTokenizer, Qwen35Tokenizer
    if model_dir and os.path.exists(os.path.join(model_dir, "vocab.json")):
        return Qwen35Tokenizer.load_from_dir(model_dir)
    for cand in (model_path + ".vocab", os.path.splitext(model_path)[0] + ".vocab"):
        if os.path.exists(cand):
            return BPETokenizer().load(cand)
    return ByteTokenizer()
