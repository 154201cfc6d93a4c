"""Plot median peer-initialisation latency per rank count with min/max error bars.

    python -m mnnvl_sharp_b200.cli.plot_init_latency init_latency.csv --output init_latency.png

Same figure as the reference project's scripts/plot_init_latency.py (7.5 x 4.5 in, 160 dpi,
axes "rank count" / "peer access initialization latency (ms)"), drawn with matplotlib's
headless Agg raster when matplotlib is installed. Without matplotlib the same chart is written
as a hand-made SVG next to the requested path (same stem, .svg), so the sweep never fails for
want of a plotting library.
"""
from __future__ import annotations

import argparse
import csv
import statistics
from pathlib import Path


def load(csv_path: Path) -> dict[int, list[float]]:
    grouped: dict[int, list[float]] = {}
    with csv_path.open(newline="") as f:
        for row in csv.DictReader(f):
            grouped.setdefault(int(row["rank_count"]), []).append(float(row["peer_init_ms"]))
    return grouped


def svg_chart(grouped: dict[int, list[float]]) -> str:
    width, height, left, right, top, bottom = 720, 432, 70, 20, 20, 50
    counts = sorted(grouped)
    med = [statistics.median(grouped[c]) for c in counts]
    lo = [min(grouped[c]) for c in counts]
    hi = [max(grouped[c]) for c in counts]
    y_max = max(hi) * 1.1 or 1.0
    x_min, x_max = min(counts), max(counts)
    span = (x_max - x_min) or 1

    def x(c):
        return left + (c - x_min) / span * (width - left - right) if len(counts) > 1 else (left + width - right) / 2

    def y(v):
        return height - bottom - v / y_max * (height - top - bottom)

    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="12">',
             f'<rect width="{width}" height="{height}" fill="white"/>']
    for k in range(6):
        v = y_max * k / 5
        parts.append(f'<line x1="{left}" x2="{width - right}" y1="{y(v):.1f}" y2="{y(v):.1f}" stroke="#ddd"/>')
        parts.append(f'<text x="{left - 8}" y="{y(v) + 4:.1f}" text-anchor="end">{v:.2f}</text>')
    parts.append(f'<line x1="{left}" x2="{left}" y1="{top}" y2="{height - bottom}" stroke="black"/>')
    parts.append(f'<line x1="{left}" x2="{width - right}" y1="{height - bottom}" y2="{height - bottom}" stroke="black"/>')
    points = " ".join(f"{x(c):.1f},{y(m):.1f}" for c, m in zip(counts, med))
    parts.append(f'<polyline points="{points}" fill="none" stroke="#1f77b4" stroke-width="1.8"/>')
    for c, m, a, b in zip(counts, med, lo, hi):
        parts.append(f'<line x1="{x(c):.1f}" x2="{x(c):.1f}" y1="{y(a):.1f}" y2="{y(b):.1f}" stroke="#1f77b4"/>')
        for v in (a, b):
            parts.append(f'<line x1="{x(c) - 4:.1f}" x2="{x(c) + 4:.1f}" y1="{y(v):.1f}" y2="{y(v):.1f}" stroke="#1f77b4"/>')
        parts.append(f'<circle cx="{x(c):.1f}" cy="{y(m):.1f}" r="3.5" fill="#1f77b4"/>')
        parts.append(f'<text x="{x(c):.1f}" y="{height - bottom + 16}" text-anchor="middle">{c}</text>')
    parts.append(f'<text x="{(left + width - right) / 2}" y="{height - 10}" text-anchor="middle">rank count</text>')
    parts.append(f'<text transform="translate(16 {(top + height - bottom) / 2}) rotate(-90)" text-anchor="middle">'
                 'peer access initialization latency (ms)</text>')
    parts.append("</svg>")
    return "\n".join(parts)


def plot(csv_path: Path, output: Path) -> Path | None:
    grouped = load(csv_path)
    if not grouped:
        return None
    output.parent.mkdir(parents=True, exist_ok=True)
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        svg_path = output.with_suffix(".svg")
        svg_path.write_text(svg_chart(grouped))
        return svg_path
    counts = sorted(grouped)
    med = [statistics.median(grouped[c]) for c in counts]
    lows = [m - min(grouped[c]) for m, c in zip(med, counts)]
    highs = [max(grouped[c]) - m for m, c in zip(med, counts)]
    fig, ax = plt.subplots(figsize=(7.5, 4.5))
    ax.errorbar(counts, med, yerr=[lows, highs], marker="o", capsize=4, linewidth=1.8)
    ax.set_xlabel("rank count")
    ax.set_ylabel("peer access initialization latency (ms)")
    ax.grid(True, axis="y", alpha=0.35)
    ax.set_xticks(counts)
    fig.tight_layout()
    fig.savefig(output, dpi=160)
    return output


def main(argv: list[str] | None = None) -> int:
    p = argparse.ArgumentParser(description="Plot peer initialisation latency.")
    p.add_argument("csv_path", type=Path)
    p.add_argument("--output", type=Path, required=True)
    args = p.parse_args(argv)
    written = plot(args.csv_path, args.output)
    if written is None:
        raise SystemExit("CSV did not contain any rows")
    print(f"wrote {written}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
