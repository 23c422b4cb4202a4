#!/usr/bin/env python
"""Share of GPU kernel time spent in communication kernels, from a kernel-time CSV (the `ncu --csv` launch
list of the profiling recipe, or `nsys stats --report cuda_gpu_kern_sum --format csv`). Communication =
NCCL kernels plus this framework's collective kernels (allreduce_f32 / reduce_scatter_f32 / allgather).

    python scripts/comm_share.py launches.csv
"""

import csv
import sys

COMM = ("nccl", "allreduce_f32_kernel", "reduce_scatter_f32_kernel", "allgather_kernel", "peer_fetch_kernel")


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    rows = list(csv.reader(open(argv[0], errors="ignore")))
    head = next(i for i, r in enumerate(rows) if any("Name" in c for c in r))
    cols = rows[head]
    name_i = next(i for i, c in enumerate(cols) if c in ("Kernel Name", "Name"))
    time_i = next(i for i, c in enumerate(cols) if c in ("Metric Value", "Total Time (ns)"))
    total = comm = 0.0
    for r in rows[head + 1:]:
        if len(r) <= max(name_i, time_i):
            continue
        try:
            t = float(r[time_i].replace(",", ""))
        except ValueError:
            continue
        total += t
        if any(k in r[name_i].lower() for k in COMM):
            comm += t
    print(f"communication kernels: {100 * comm / max(total, 1e-9):.1f}% of {total:.3e} (summed kernel time)")


if __name__ == "__main__":
    main()
