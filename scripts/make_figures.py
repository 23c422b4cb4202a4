#!/usr/bin/env python
"""Regenerate tables and figures from results/ only — nothing is re-measured.

    python scripts/make_figures.py [--results results] [--out figures] [--readme README.md]

Tables: the optimisation ladder (results/ladder/<gpu>/*.json), the multi-GPU table (results/dist/<gpu>-xN/*.json),
kernel micro-benchmarks (results/kernels/*.json). Figures (plain SVG written by this script, no plotting library needed):
tokens/s bar charts of the ladder and of the multi-GPU table and, if a run's metrics.jsonl is given with --metrics, its
loss curve (the reference draws the same two with matplotlib, scripts/make_figures.py:60-150). With --readme the tables also replace whatever stands between the
``<!-- results:begin -->`` and ``<!-- results:end -->`` markers of that file (the reference regenerates the numbers block
of its README the same way, scripts/make_figures.py:207-235), so the README never carries a hand-copied number.
"""

import argparse
import json
import math
from pathlib import Path


def load(folder: Path):
    return {p.stem: json.loads(p.read_text()) for p in sorted(folder.glob("*.json"))}


def ladder_rows(results: Path):
    for gpu in sorted((results / "ladder").glob("*")):
        for name, r in load(gpu).items():
            yield gpu.name, name, r["tokens_per_s"]["median"], r["step_ms"]["median"]


def dist_rows(results: Path):
    for folder in sorted((results / "dist").glob("*-x*")):
        for name, r in load(folder).items():
            yield folder.name, name, r["tokens_per_s"]["median"], r["bench"]["world"]


BEGIN, END = "<!-- results:begin -->", "<!-- results:end -->"


def update_block(readme: Path, lines: list[str]) -> None:
    """Replace the text between the two markers of `readme` with `lines` (the markers are appended if the file has none)."""
    text = readme.read_text() if readme.exists() else ""
    block = BEGIN + "\n" + "\n".join(lines) + "\n" + END
    if BEGIN in text and END in text:
        head, rest = text.split(BEGIN, 1)
        text = head + block + rest.split(END, 1)[1]
    else:
        text = text.rstrip("\n") + "\n\n" + block + "\n"
    readme.write_text(text)
    print(f"rewrote the results block of {readme}")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--results", type=Path, default=Path("results"))
    ap.add_argument("--out", type=Path, default=Path("figures"))
    ap.add_argument("--metrics", type=Path, default=None, help="a run's metrics.jsonl for the loss curve")
    ap.add_argument("--readme", type=Path, default=None, help="file whose results block (between the markers) is rewritten")
    a = ap.parse_args(argv)
    a.out.mkdir(parents=True, exist_ok=True)
    lines = ["## Optimisation ladder", "| gpu | stage | tok/s | step ms |", "|---|---|---|---|"]
    ladder = list(ladder_rows(a.results)) if (a.results / "ladder").exists() else []
    lines += [f"| {g} | {n} | {t:,.0f} | {ms:.2f} |" for g, n, t, ms in ladder]
    lines += ["", "## Multi-GPU", "| folder | config | tok/s | GPUs |", "|---|---|---|---|"]
    if (a.results / "dist").exists():
        lines += [f"| {f} | {n} | {t:,.0f} | {w} |" for f, n, t, w in dist_rows(a.results)]
    if (a.results / "kernels").exists():
        for name, r in load(a.results / "kernels").items():
            lines += ["", f"## Kernel benchmark: {name} ({r['device']})"]
            if r["rows"]:
                keys = list(r["rows"][0])
                lines += ["| " + " | ".join(keys) + " |", "|" + "---|" * len(keys)]
                lines += ["| " + " | ".join(f"{row[k]:.4g}" if isinstance(row[k], float) else str(row[k]) for k in keys) + " |" for row in r["rows"]]
    (a.out / "tables.md").write_text("\n".join(lines) + "\n")
    print(f"wrote {a.out / 'tables.md'}")
    if a.readme is not None:
        update_block(a.readme, lines)
    if ladder:
        svg_bars(a.out / "ladder_tokens_per_s.svg", [f"{g}/{n}" if len({g for g, *_ in ladder}) > 1 else n for g, n, _, _ in ladder],
                 [t for _, _, t, _ in ladder], "tokens / s")
    dist = list(dist_rows(a.results)) if (a.results / "dist").exists() else []
    if dist:
        svg_bars(a.out / "dist_tokens_per_s.svg", [f"{n} x{w}" for _, n, _, w in dist], [t for _, _, t, _ in dist], "tokens / s")
    if a.metrics and a.metrics.exists():
        recs = [json.loads(line) for line in a.metrics.read_text().splitlines() if line.strip()]
        train = [(r["tokens"], r["loss"]) for r in recs if "loss" in r and "tokens" in r]
        series = {"train": train}
        val = [(r["step"], r["val_loss"]) for r in recs if "val_loss" in r]
        if val and train:
            first = next(r for r in recs if "loss" in r and "tokens" in r)
            per = first["tokens"] / (first["step"] + 1)
            series["val"] = [((s + 1) * per, v) for s, v in val]
        if train:
            svg_lines(a.out / "loss.svg", series, "tokens", "loss")


# ----------------------------------------------------------------------------- figures, written as plain SVG (no plotting library)
W, H, LEFT, RIGHT, TOP, BOTTOM = 760, 360, 70, 20, 20, 110
COLORS = ("#2f6fb7", "#d9662b", "#2a9d6f", "#8a5fbf")


def nice_ticks(lo: float, hi: float, n: int = 5) -> list[float]:
    """About n round tick values covering [lo, hi] (steps of 1, 2 or 5 times a power of ten)."""
    if hi <= lo:
        hi = lo + 1.0
    raw = (hi - lo) / n
    mag = 10.0 ** math.floor(math.log10(raw))
    step = next(m * mag for m in (1, 2, 5, 10) if m * mag >= raw)
    first = math.floor(lo / step) * step
    ticks, t = [], first
    while t <= hi + 1e-9 * step:
        ticks.append(round(t, 10))
        t += step
    if ticks[-1] < hi:
        ticks.append(round(ticks[-1] + step, 10))
    return ticks


def human(v: float) -> str:
    for unit, div in (("G", 1e9), ("M", 1e6), ("k", 1e3)):
        if abs(v) >= div:
            return f"{v / div:.3g}{unit}"
    return f"{v:.3g}"


def _frame(ticks, y_of, ylabel):
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" viewBox="0 0 {W} {H}" font-family="sans-serif" font-size="11">',
           f'<rect width="{W}" height="{H}" fill="white"/>']
    for t in ticks:
        y = y_of(t)
        out.append(f'<line x1="{LEFT}" y1="{y:.1f}" x2="{W - RIGHT}" y2="{y:.1f}" stroke="#e3e3e3"/>')
        out.append(f'<text x="{LEFT - 6}" y="{y + 4:.1f}" text-anchor="end" fill="#444">{human(t)}</text>')
    out.append(f'<text x="14" y="{TOP + (H - TOP - BOTTOM) / 2:.1f}" transform="rotate(-90 14 {TOP + (H - TOP - BOTTOM) / 2:.1f})" text-anchor="middle" fill="#222">{ylabel}</text>')
    return out


def svg_bars(path: Path, labels: list[str], values: list[float], ylabel: str) -> None:
    ticks = nice_ticks(0.0, max(values))
    top = ticks[-1]
    y_of = lambda v: TOP + (H - TOP - BOTTOM) * (1.0 - v / top)
    out = _frame(ticks, y_of, ylabel)
    slot = (W - LEFT - RIGHT) / len(values)
    for i, (name, v) in enumerate(zip(labels, values)):
        x, y = LEFT + i * slot + 0.15 * slot, y_of(v)
        out.append(f'<rect x="{x:.1f}" y="{y:.1f}" width="{0.7 * slot:.1f}" height="{H - BOTTOM - y:.1f}" fill="{COLORS[0]}"/>')
        out.append(f'<text x="{x + 0.35 * slot:.1f}" y="{y - 4:.1f}" text-anchor="middle" fill="#222">{human(v)}</text>')
        cx = x + 0.35 * slot
        out.append(f'<text x="{cx:.1f}" y="{H - BOTTOM + 12}" transform="rotate(35 {cx:.1f} {H - BOTTOM + 12})" fill="#222">{name}</text>')
    path.write_text("\n".join(out + ["</svg>"]) + "\n")
    print(f"wrote {path}")


def svg_lines(path: Path, series: dict, xlabel: str, ylabel: str) -> None:
    xs = [x for pts in series.values() for x, _ in pts]
    ys = [y for pts in series.values() for _, y in pts]
    yt, xt = nice_ticks(min(ys), max(ys)), nice_ticks(min(xs), max(xs))
    y_of = lambda v: TOP + (H - TOP - BOTTOM) * (1.0 - (v - yt[0]) / (yt[-1] - yt[0]))
    x_of = lambda v: LEFT + (W - LEFT - RIGHT) * (v - xt[0]) / (xt[-1] - xt[0])
    out = _frame(yt, y_of, ylabel)
    for t in xt:
        out.append(f'<text x="{x_of(t):.1f}" y="{H - BOTTOM + 16}" text-anchor="middle" fill="#444">{human(t)}</text>')
    out.append(f'<text x="{LEFT + (W - LEFT - RIGHT) / 2:.1f}" y="{H - BOTTOM + 38}" text-anchor="middle" fill="#222">{xlabel}</text>')
    for k, (name, pts) in enumerate(series.items()):
        color = COLORS[k % len(COLORS)]
        path_d = " ".join(f"{'M' if i == 0 else 'L'}{x_of(x):.1f},{y_of(y):.1f}" for i, (x, y) in enumerate(pts))
        out.append(f'<path d="{path_d}" fill="none" stroke="{color}" stroke-width="1.5"/>')
        if len(pts) <= 40:
            out += [f'<circle cx="{x_of(x):.1f}" cy="{y_of(y):.1f}" r="2.5" fill="{color}"/>' for x, y in pts]
        out.append(f'<text x="{W - RIGHT - 60}" y="{TOP + 14 + 14 * k}" fill="{color}">{name}</text>')
    path.write_text("\n".join(out + ["</svg>"]) + "\n")
    print(f"wrote {path}")


if __name__ == "__main__":
    main()
