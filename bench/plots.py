#!/usr/bin/env python
"""Bar charts of a benchmark history as SVG files, without a plotting library.

    python bench/plots.py [--history bench/results/history.jsonl] [--out bench/results]

For every (suite, model) in the history one chart per metric (samples/s, epochs/s, final loss, accuracy) with one bar per run
label (mean over repeats, min-max whisker), plus ``plots.md`` that embeds them. The reference produces the same
charts with matplotlib and an auto-written README (benchmarks/issue/plots.py, benchmarks/issue/readme.py)."""
from __future__ import annotations

import argparse
import json
import os
from collections import OrderedDict

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
METRICS = [("samples_per_sec", "samples / s"), ("epochs_per_sec", "epochs / s"), ("final_loss", "final loss"),
           ("accuracy", "accuracy")]
COLORS = ["#4c78a8", "#f58518", "#54a24b", "#e45756", "#72b7b2", "#b279a2", "#ff9da6", "#9d755d"]


def _fmt(v: float) -> str:
    a = abs(v)
    if a >= 1e6:
        return f"{v / 1e6:.2f}M"
    if a >= 1e3:
        return f"{v / 1e3:.1f}k"
    if a >= 10:
        return f"{v:.1f}"
    return f"{v:.4g}"


def _esc(s: str) -> str:
    return s.replace("&", "&amp;").replace("<", "&lt;").replace(">", "&gt;")


def bar_chart(title: str, ylabel: str, bars: list[tuple[str, float, float, float]]) -> str:
    """bars: (label, mean, lo, hi). Returns an SVG document."""
    W, H, L, R, T, B = 760, 380, 70, 20, 40, 110
    pw, ph = W - L - R, H - T - B
    top = max([hi for _, _, _, hi in bars] + [1e-12]) * 1.12
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="11">',
           f'<rect width="{W}" height="{H}" fill="white"/>',
           f'<text x="{W / 2}" y="20" text-anchor="middle" font-size="14">{_esc(title)}</text>',
           f'<text x="14" y="{T + ph / 2}" text-anchor="middle" transform="rotate(-90 14 {T + ph / 2})">{_esc(ylabel)}</text>']
    for i in range(5):
        v = top * i / 4
        y = T + ph - ph * i / 4
        out.append(f'<line x1="{L}" y1="{y:.1f}" x2="{L + pw}" y2="{y:.1f}" stroke="#ddd"/>')
        out.append(f'<text x="{L - 6}" y="{y + 4:.1f}" text-anchor="end">{_fmt(v)}</text>')
    n = max(1, len(bars))
    slot = pw / n
    bw = min(60.0, slot * 0.7)
    for i, (label, mean, lo, hi) in enumerate(bars):
        x = L + slot * i + (slot - bw) / 2
        h = ph * mean / top
        y = T + ph - h
        out.append(f'<rect x="{x:.1f}" y="{y:.1f}" width="{bw:.1f}" height="{h:.1f}" fill="{COLORS[i % len(COLORS)]}"/>')
        if hi > lo:
            cx = x + bw / 2
            y0, y1 = T + ph - ph * lo / top, T + ph - ph * hi / top
            out.append(f'<line x1="{cx:.1f}" y1="{y0:.1f}" x2="{cx:.1f}" y2="{y1:.1f}" stroke="black"/>')
        out.append(f'<text x="{x + bw / 2:.1f}" y="{y - 4:.1f}" text-anchor="middle">{_fmt(mean)}</text>')
        lx, ly = x + bw / 2, T + ph + 12
        out.append(f'<text x="{lx:.1f}" y="{ly:.1f}" text-anchor="end" transform="rotate(-35 {lx:.1f} {ly:.1f})">{_esc(label)}</text>')
    out.append(f'<line x1="{L}" y1="{T + ph}" x2="{L + pw}" y2="{T + ph}" stroke="black"/>')
    out.append("</svg>")
    return "\n".join(out)


def load(history: str) -> "OrderedDict[tuple[str, str], OrderedDict[str, list[dict]]]":
    groups: OrderedDict = OrderedDict()
    with open(history) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            r = json.loads(line)
            key = (str(r.get("suite", "suite")), str(r.get("model", "model")))
            groups.setdefault(key, OrderedDict()).setdefault(str(r.get("suite_label", "run")), []).append(r)
    return groups


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--history", default=os.path.join(ROOT, "bench", "results", "history.jsonl"))
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    out_dir = a.out or os.path.dirname(os.path.abspath(a.history))
    os.makedirs(out_dir, exist_ok=True)
    groups = load(a.history)
    written = []
    md = ["# Benchmark plots", ""]
    for (suite, model), runs in groups.items():
        md += [f"## {suite} — {model}", ""]
        for key, ylabel in METRICS:
            bars = []
            for label, recs in runs.items():
                vals = [float(r[key]) for r in recs if r.get(key) is not None]
                if vals:
                    bars.append((label, sum(vals) / len(vals), min(vals), max(vals)))
            if not bars:
                continue
            name = f"{suite}_{model}_{key}.svg"
            with open(os.path.join(out_dir, name), "w") as f:
                f.write(bar_chart(f"{suite} / {model}: {ylabel}", ylabel, bars))
            written.append(name)
            md.append(f"![{ylabel}]({name})")
        md.append("")
    with open(os.path.join(out_dir, "plots.md"), "w") as f:
        f.write("\n".join(md))
    print(json.dumps({"plots": len(written), "out": out_dir}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
