#!/usr/bin/env python
"""Print the optimisation-ladder table from results/ladder/<gpu>/*.json (written by scripts/bench_train.py).

    python scripts/ladder_table.py [results/ladder/b200]
"""

import json
import sys
from pathlib import Path


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    root = Path(argv[0]) if argv else next(iter(sorted(Path("results/ladder").glob("*"))), None)
    if root is None or not root.exists():
        raise SystemExit("no results under results/ladder: run scripts/bench_train.py on the stage configs first")
    rows = [(json.loads(p.read_text()), p.stem) for p in sorted(root.glob("*.json"))]
    print(f"| stage | tok/s (median) | step ms | vs previous | MFU | peak GB | flags |\n|---|---|---|---|---|---|---|")
    prev = None
    for r, name in rows:
        tps = r["tokens_per_s"]["median"]
        mfu = next(iter(r["mfu"].values()))["median"] if r.get("mfu") else None
        mem = r["peak_mem_gb"]["allocated"] if r.get("peak_mem_gb") else None
        print(f"| {name} | {tps:,.0f} | {r['step_ms']['median']:.2f} | {f'{tps / prev:.2f}x' if prev else '-'} | "
              f"{f'{100 * mfu:.1f}%' if mfu else '-'} | {f'{mem:.2f}' if mem else '-'} | {'; '.join(r.get('throttle_flags', [])) or '-'} |")
        prev = tps


if __name__ == "__main__":
    main()
