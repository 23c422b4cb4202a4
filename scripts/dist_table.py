#!/usr/bin/env python
"""Print the multi-GPU table from results/dist/<gpu>-x<N>/*.json: tokens/s, scaling efficiency against the
single-GPU row, memory per GPU.

    python scripts/dist_table.py [results/dist]
"""

import json
import re
import sys
from pathlib import Path


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    root = Path(argv[0]) if argv else Path("results/dist")
    rows = []
    for folder in sorted(root.glob("*-x*")):
        n = int(re.search(r"-x(\d+)$", folder.name).group(1))
        for p in sorted(folder.glob("*.json")):
            r = json.loads(p.read_text())
            rows.append((n, p.stem, r["tokens_per_s"]["median"], r["peak_mem_gb"]["allocated"] if r.get("peak_mem_gb") else None))
    if not rows:
        raise SystemExit(f"no results under {root}")
    base = next((t for n, _, t, _ in rows if n == 1), None)
    print("| GPUs | config | tok/s | scaling efficiency | GB / GPU |\n|---|---|---|---|---|")
    for n, name, tps, mem in rows:
        eff = f"{100 * tps / (base * n):.0f}%" if base else "-"
        print(f"| {n} | {name} | {tps:,.0f} | {eff} | {f'{mem:.2f}' if mem else '-'} |")


if __name__ == "__main__":
    main()
