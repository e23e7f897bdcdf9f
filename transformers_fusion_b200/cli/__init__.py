"""Command-line tools.  ``python -m transformers_fusion_b200.cli <tool> [args]`` or the launchers under
``bin/`` (one per tool, same names as the reference binaries: quant_train, quant_finetune, quant_quantize,
quant_convert, quant_infer, quant_serve, quant_server, quant_evaluate, quant_info, quant_bench,
quant_format_list, gle_report, train_64m, bench_speed, probe_mi_extraction, generate_comparison_visuals)."""
import importlib
import sys

TOOLS = {
    "quant_train": "train", "quant_finetune": "finetune", "quant_quantize": "quantize", "quant_convert": "convert",
    "quant_infer": "infer", "quant_serve": "serve", "quant_server": "serve", "quant_evaluate": "evaluate",
    "quant_info": "info", "quant_bench": "bench", "quant_format_list": "format_list", "gle_report": "gle_report",
    "train_64m": "train_64m", "bench_speed": "train_64m", "probe_mi_extraction": "probe_mi_extraction",
    "generate_comparison_visuals": "generate_comparison_visuals",
}


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help") or argv[0] not in TOOLS:
        print("usage: python -m transformers_fusion_b200.cli <tool> [args]\ntools: " + " ".join(sorted(TOOLS)))
        return 0 if argv and argv[0] in ("-h", "--help") else 2
    mod = importlib.import_module(f"{__name__}.{TOOLS[argv[0]]}")
    extra = ["--bench"] if argv[0] == "bench_speed" else []
    return mod.main(extra + argv[1:])
