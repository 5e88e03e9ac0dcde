"""Draws the per-weight size tables of :class:`keys_values_b200.tools.size_log.PerWeightSizeLog` as an SVG file
(``keys_values/scripts/plot_size_log.py``, ``plot_size_log_stored_values.py``).

    python -m keys_values_b200.tools.plot_size_log DIR [--table gradients] [--qs 0.5 0.99 max] [--q_max max]
        [--top_n 10] [--step_limit N] [--log] [--out sizes.svg]

The ``top_n`` rows with the largest value of quantile ``q_max`` over all steps are drawn, one panel per quantile in
``qs`` (shared step axis, one colour per row in all panels, legend with the names of ``weight_names.csv``). The SVG is
written by this module itself: no plotting library is needed.
"""
from __future__ import annotations

import argparse
import csv
import math
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

COLOURS = ("#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#bcbd22", "#17becf")


def load_tables(directory: Path, table: str = "weights"):
    """``{(weight_idx, q): [(step, value), …]}`` and ``{weight_idx: name}``."""
    series: Dict[Tuple[int, str], List[Tuple[int, float]]] = defaultdict(list)
    with open(Path(directory) / f"size_{table}.csv") as fp:
        for row in csv.DictReader(fp):
            series[(int(row["weight_idx"]), row["q"])].append((int(row["step"]), float(row["value"])))
    names = {}
    names_file = Path(directory) / "weight_names.csv"
    if names_file.is_file():
        with open(names_file) as fp:
            names = {int(r["weight_idx"]): r["name"] for r in csv.DictReader(fp)}
    for pts in series.values():
        pts.sort()
    return series, names


def select_top(series, q_max: str, top_n: int, step_limit: Optional[int] = None) -> List[int]:
    best: Dict[int, float] = {}
    for (idx, q), pts in series.items():
        if q != q_max:
            continue
        vals = [v for s, v in pts if step_limit is None or s < step_limit]
        if vals:
            best[idx] = max(vals)
    return [i for i, _ in sorted(best.items(), key=lambda kv: -kv[1])[:top_n]]


def _ticks(lo: float, hi: float, n: int = 5) -> List[float]:
    if hi <= lo:
        return [lo]
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m * mag for m in (1, 2, 5, 10) if m * mag >= raw), default=raw)
    first = math.ceil(lo / step) * step
    out, t = [], first
    while t <= hi + 1e-12 * abs(hi):
        out.append(t)
        t += step
    return out


def render_svg(series, names, rows: Sequence[int], qs: Sequence[str], step_limit: Optional[int] = None, log_scale: bool = False,
               title: str = "") -> str:
    width, panel_h, left, right, top, gap = 900, 220, 70, 260, 40, 30
    plot_w = width - left - right
    height = top + len(qs) * (panel_h + gap) + 20
    steps = sorted({s for (i, q), pts in series.items() if i in rows and q in qs for s, _ in pts if step_limit is None or s < step_limit})
    if not steps:
        return f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="80"><text x="10" y="40">no data</text></svg>'
    s_lo, s_hi = steps[0], max(steps[-1], steps[0] + 1)
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="11">',
           f'<rect width="{width}" height="{height}" fill="white"/>', f'<text x="{left}" y="20" font-size="14">{title}</text>']
    tr = (lambda v: math.log10(max(v, 1e-30))) if log_scale else (lambda v: v)
    for k, q in enumerate(qs):
        y0 = top + k * (panel_h + gap)
        vals = [tr(v) for i in rows for s, v in series.get((i, q), []) if step_limit is None or s < step_limit]
        v_lo, v_hi = (min(vals), max(vals)) if vals else (0.0, 1.0)
        if v_hi <= v_lo:
            v_hi = v_lo + 1.0
        sx = lambda s: left + (s - s_lo) / (s_hi - s_lo) * plot_w  # noqa: E731
        sy = lambda v: y0 + panel_h - (tr(v) - v_lo) / (v_hi - v_lo) * panel_h  # noqa: E731
        out.append(f'<rect x="{left}" y="{y0}" width="{plot_w}" height="{panel_h}" fill="none" stroke="#444"/>')
        out.append(f'<text x="{left + 4}" y="{y0 + 14}">quantile {q}{" (log10)" if log_scale else ""}</text>')
        for t in _ticks(v_lo, v_hi):
            y = y0 + panel_h - (t - v_lo) / (v_hi - v_lo) * panel_h
            out.append(f'<line x1="{left}" y1="{y:.1f}" x2="{left + plot_w}" y2="{y:.1f}" stroke="#ddd"/>')
            out.append(f'<text x="{left - 6}" y="{y + 4:.1f}" text-anchor="end">{t:.3g}</text>')
        if k == len(qs) - 1:
            for t in _ticks(s_lo, s_hi, 8):
                out.append(f'<text x="{sx(t):.1f}" y="{y0 + panel_h + 14}" text-anchor="middle">{t:g}</text>')
            out.append(f'<text x="{left + plot_w / 2}" y="{y0 + panel_h + 28}" text-anchor="middle">step</text>')
        for c, i in enumerate(rows):
            pts = [(s, v) for s, v in series.get((i, q), []) if step_limit is None or s < step_limit]
            if pts:
                path = " ".join(f"{sx(s):.1f},{sy(v):.1f}" for s, v in pts)
                out.append(f'<polyline points="{path}" fill="none" stroke="{COLOURS[c % len(COLOURS)]}" stroke-width="1.5"/>')
    for c, i in enumerate(rows):
        y = top + 14 + 16 * c
        out.append(f'<line x1="{left + plot_w + 10}" y1="{y - 4}" x2="{left + plot_w + 34}" y2="{y - 4}" stroke="{COLOURS[c % len(COLOURS)]}" stroke-width="2"/>')
        out.append(f'<text x="{left + plot_w + 40}" y="{y}">{names.get(i, f"weight {i}")[:36]}</text>')
    out.append("</svg>")
    return "\n".join(out)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("directory")
    ap.add_argument("--table", default="weights", choices=["weights", "gradients"])
    ap.add_argument("--qs", nargs="+", default=["0.5", "0.99", "max"])
    ap.add_argument("--q_max", default="max")
    ap.add_argument("--top_n", type=int, default=10)
    ap.add_argument("--step_limit", type=int, default=None)
    ap.add_argument("--log", action="store_true")
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    series, names = load_tables(Path(args.directory), args.table)
    rows = select_top(series, args.q_max, args.top_n, args.step_limit)
    svg = render_svg(series, names, rows, args.qs, args.step_limit, args.log, title=f"sizes of {args.table}: top {len(rows)} by quantile {args.q_max}")
    out = Path(args.out) if args.out else Path(args.directory) / f"size_{args.table}.svg"
    out.write_text(svg)
    print(f"wrote {out} ({len(rows)} rows, {len(args.qs)} panels)")


if __name__ == "__main__":
    main()
