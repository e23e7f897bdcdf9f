"""quant_info <model.quant>: header, tensor list with formats, parameter total (tools/info.cpp:10-70)."""
from __future__ import annotations

import sys


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1 or argv[0] in ("-h", "--help"):
        print("Usage: quant_info <model.quant>")
        return 0 if argv else 1
    from ..quant import codec
    try:
        r = codec.QuantReader(argv[0])
    except ValueError as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    L = codec.lib()
    print(f"QUANT Model: {argv[0]}")
    print("Magic: QUA1")
    print(f"Version: {r.version}")
    print(f"Flags: 0x{L.tfb_reader_flags(r._h):x}")
    print(f"Config size: {len(r.config_bytes())} bytes")
    names = r.tensor_names()
    print(f"Tensors: {len(names)}")
    total = 0
    for i, n in enumerate(names):
        numel = L.tfb_reader_tensor_numel(r._h, n.encode())
        if numel < 0:
            print(f"  [{i}] {n} (error: corrupt blocks)")
            continue
        fm = r.block_formats(n)
        extra = f" (+{len(fm) - 1} blocks)" if len(fm) > 1 else ""
        mixed = "" if len(set(fm.tolist())) <= 1 else " mixed:" + ",".join(sorted({codec.format_name(int(f)) for f in fm}))
        print(f"  [{i}] {n} numel={numel} format={codec.format_name(int(fm[0])) if len(fm) else '-'}{extra}{mixed}")
        total += numel
    print(f"Total parameters: {total}")
    if len(r.config_bytes()) == 128:
        from ..models.config import TransformerConfig
        c = TransformerConfig.from_bytes(r.config_bytes())
        print(f"Config: vocab={c.vocab_size} hidden={c.hidden_size} layers={c.num_layers} heads={c.num_heads} kv_heads={c.num_kv_heads} "
              f"ffn={c.ffn_hidden_size} act={c.activation} max_seq={c.max_seq_len}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
