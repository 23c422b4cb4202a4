#!/usr/bin/env python
"""Regenerate tables (and, when matplotlib is installed, figures) from results/ only — nothing is re-measured.

    python scripts/make_figures.py [--results results] [--out figures] [--readme README.md]

Tables: the optimisation ladder (results/ladder/<gpu>/*.json), the multi-GPU table (results/dist/<gpu>-xN/*.json),
kernel micro-benchmarks (results/kernels/*.json). Figures: ladder tokens/s bar chart and, if a run's
metrics.jsonl is given with --metrics, its loss curve. With --readme the tables also replace whatever stands between the
``<!-- results:begin -->`` and ``<!-- results:end -->`` markers of that file (the reference regenerates the numbers block
of its README the same way, scripts/make_figures.py:207-235), so the README never carries a hand-copied number.
"""

import argparse
import json
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
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        print("matplotlib is not installed: tables only")
        return
    if ladder:
        fig, ax = plt.subplots(figsize=(8, 3.5))
        ax.bar([n for _, n, _, _ in ladder], [t for _, _, t, _ in ladder])
        ax.set_ylabel("tokens / s")
        ax.tick_params(axis="x", rotation=45)
        fig.tight_layout()
        fig.savefig(a.out / "ladder_tokens_per_s.png", dpi=150)
    if a.metrics and a.metrics.exists():
        recs = [json.loads(l) for l in a.metrics.read_text().splitlines()]
        fig, ax = plt.subplots(figsize=(6, 3.5))
        ax.plot([r["tokens"] for r in recs if "loss" in r], [r["loss"] for r in recs if "loss" in r], label="train")
        val = [(r["step"], r["val_loss"]) for r in recs if "val_loss" in r]
        if val:
            per = next(r["tokens"] / (r["step"] + 1) for r in recs if "loss" in r)
            ax.plot([(s + 1) * per for s, _ in val], [v for _, v in val], "o-", label="val")
        ax.set_xlabel("tokens")
        ax.set_ylabel("loss")
        ax.legend()
        fig.tight_layout()
        fig.savefig(a.out / "loss.png", dpi=150)


if __name__ == "__main__":
    main()
