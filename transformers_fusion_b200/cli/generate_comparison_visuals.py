"""generate_comparison_visuals: Markdown report with embedded SVG charts from a format-comparison CSV.

Input CSV (header + rows): ``dataset,format,bpw,mse,psnr[,enc_ms,dec_ms,...]`` - the table ``quant_bench`` style format
comparisons write.  For every dataset the report holds a PSNR-versus-bits-per-weight scatter (one dot per format,
coloured by family: reference baselines red, MX formats amber, grouped formats green, the rest blue) and a table sorted
by bits per weight.  Every number plotted comes from the CSV.

Reference counterpart: tools/generate_comparison_visuals.cpp:14-138 (reads bench_format_comparison.csv, writes
docs/COMPARISON_CHARTS.md)."""
from __future__ import annotations

import argparse
import csv
import os
import sys
from typing import Dict, List


def color(fmt: str) -> str:
    if fmt.startswith("[ref]"):
        return "#d33"
    if fmt.startswith(("MXQ", "Q_MX", "QG_MX", "mx")):
        return "#c6a700"
    if "_G" in fmt:
        return "#083"
    return "#06c"


def read_rows(path: str) -> List[dict]:
    rows = []
    with open(path, newline="") as f:
        rd = csv.reader(f)
        next(rd, None)
        for c in rd:
            if len(c) < 5:
                continue
            try:
                r = {"dataset": c[0], "format": c[1], "bpw": float(c[2]), "mse": float(c[3]), "psnr": float(c[4])}
                if len(c) > 6:
                    r["enc"], r["dec"] = float(c[5]), float(c[6])
            except ValueError:
                continue
            rows.append(r)
    return rows


def scatter_svg(rows: List[dict], w: int = 640, h: int = 360) -> str:
    xs, ys = [r["bpw"] for r in rows], [r["psnr"] for r in rows]
    x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
    sx = lambda v: 50 + (v - x0) / ((x1 - x0) or 1) * (w - 70)
    sy = lambda v: h - 40 - (v - y0) / ((y1 - y0) or 1) * (h - 60)
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" viewBox="0 0 {w} {h}">',
           f'<rect width="{w}" height="{h}" fill="#fff"/>', f'<line x1="50" y1="{h - 40}" x2="{w - 20}" y2="{h - 40}" stroke="#333"/>',
           f'<line x1="50" y1="20" x2="50" y2="{h - 40}" stroke="#333"/>',
           f'<text x="{w // 2}" y="{h - 8}" font-size="12" text-anchor="middle">bits per weight ({x0:g} .. {x1:g})</text>',
           f'<text x="14" y="{h // 2}" font-size="12" transform="rotate(-90 14 {h // 2})" text-anchor="middle">PSNR dB ({y0:.1f} .. {y1:.1f})</text>']
    for r in rows:
        out.append(f'<circle cx="{sx(r["bpw"]):.1f}" cy="{sy(r["psnr"]):.1f}" r="4" fill="{color(r["format"])}"><title>{r["format"]}: '
                   f'{r["bpw"]:g} bpw, {r["psnr"]:.2f} dB</title></circle>')
    out.append("</svg>")
    return "\n".join(out)


def render(rows: List[dict], source: str) -> str:
    by: Dict[str, List[dict]] = {}
    for r in rows:
        by.setdefault(r["dataset"], []).append(r)
    md = ["# Format comparison charts\n", f"> Generated from `{os.path.basename(source)}`; every value below is a measured round trip of the codec.\n"]
    for ds, rs in by.items():
        rs.sort(key=lambda r: (r["bpw"], -r["psnr"]))
        md += [f"## Dataset: {ds}\n", scatter_svg(rs), "", "| format | bpw | MSE | PSNR dB |", "|---|---|---|---|"]
        md += [f"| {r['format']} | {r['bpw']:g} | {r['mse']:.3e} | {r['psnr']:.2f} |" for r in rs]
        md.append("")
    return "\n".join(md)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="generate_comparison_visuals")
    ap.add_argument("--input", default="bench_format_comparison.csv")
    ap.add_argument("--output", default="docs/COMPARISON_CHARTS.md")
    a = ap.parse_args(argv)
    if not os.path.exists(a.input):
        print(f"ERROR: {a.input} is missing (write it with the format comparison benchmark first)", file=sys.stderr)
        return 1
    rows = read_rows(a.input)
    if not rows:
        print("ERROR: CSV has no rows", file=sys.stderr)
        return 2
    os.makedirs(os.path.dirname(os.path.abspath(a.output)), exist_ok=True)
    with open(a.output, "w") as f:
        f.write(render(rows, a.input))
    print(f"{a.output} generated ({len(rows)} CSV rows read)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
