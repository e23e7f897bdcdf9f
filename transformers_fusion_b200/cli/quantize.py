"""quant_quantize: ``--input --output --format(q8; q1..q32, qg1..qg24 + aliases) --per-layer name=fmt,...
--num-bits`` (tools/quantize.cpp:21-240).  Every tensor is re-encoded in 256-weight blocks; tables are
written before the blocks (the order the reader needs; the reference tool writes them after)."""
from __future__ import annotations

import argparse
import os
import sys

from .common import add_int


def main(argv=None):
    ap = argparse.ArgumentParser(prog="quant_quantize")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--format", default="q8")
    ap.add_argument("--per-layer", default="")
    add_int(ap, "--num-bits", 0)
    a = ap.parse_args(argv)
    from ..quant import codec
    fmt_name = a.format if not a.num_bits else f"q{a.num_bits}"
    fmt = codec.parse_format(fmt_name)
    if fmt < 0:
        print(f"Error: unknown format '{fmt_name}'", file=sys.stderr)
        return 2
    per = {}
    for item in filter(None, a.per_layer.split(",")):
        k, _, v = item.partition("=")
        if codec.parse_format(v) < 0:
            print(f"Error: unknown format '{v}' for layer '{k}'", file=sys.stderr)
            return 2
        per[k] = codec.parse_format(v)
    if not os.path.exists(a.input):
        print(f"Error: cannot open '{a.input}'", file=sys.stderr)
        return 1
    r = codec.QuantReader(a.input)
    w = codec.QuantWriter(a.output, r.config_bytes(), r.version)
    total_in = total_w = 0
    for name in r.tensor_names():
        t = r.read_tensor(name)
        f = fmt
        for k, v in per.items():
            if k in name:
                f = v
        if t.numel() < 1024 or name.endswith("norm.weight") or name.endswith(".bias"):
            f = codec.Q_32
        w.add_tensor(name, t, f)
        total_w += t.numel()
        total_in += t.numel() * 4
    w.close()
    out_bytes = os.path.getsize(a.output)
    print(f"Quantized {len(r.tensor_names())} tensors ({total_w} weights) to {codec.format_name(fmt)}: "
          f"{total_in / 1e6:.2f} MB -> {out_bytes / 1e6:.2f} MB ({8.0 * out_bytes / max(1, total_w):.3f} bpw)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
