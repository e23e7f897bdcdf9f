"""quant_convert: ``--input --output --format rawfp32|gguf|safetensors|auto --bpw N --verbose``
(tools/convert.cpp:27-56; safetensors files / model directories are accepted as well)."""
from __future__ import annotations

import argparse
import sys

from .common import add_float


def main(argv=None):
    ap = argparse.ArgumentParser(prog="quant_convert", description="Usage: quant_convert --input <file> --output <model.quant> [options]",
                                 epilog="Formats: 1.0(quant1) 1.50(quant) 4.0(quant4) 8.0(quant8) 16.0(fp16) 32.0(fp32)")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--format", default="rawfp32", help="Input format: rawfp32 (default), gguf, safetensors, auto")
    add_float(ap, "--bpw", 0.0, "Target bits-per-weight for FormatPlanner (0=no compression)")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    if not (0.0 <= a.bpw <= 32.0):
        print("Error: --bpw needs 0..32", file=sys.stderr)
        return 2
    from ..quant import importers
    try:
        rep = importers.convert(a.input, a.output, kind=a.format, target_bpw=a.bpw, verbose=a.verbose)
    except (ValueError, OSError) as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    print(f"Converted {rep['tensors']} tensors ({rep['weights']} weights) -> {a.output}: {rep['bytes']} bytes, {rep['bpw']:.3f} bpw")
    return 0


if __name__ == "__main__":
    sys.exit(main())
