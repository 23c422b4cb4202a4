"""Condense `ncu --page raw --csv` output into the handful of counters the roofline discussion uses.

    python benchmarks/kernels/ncu_table.py capture_raw.csv
"""

import csv
import sys

KEEP = ["gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
        "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "sm__warps_active.avg.pct_of_peak_sustained_active",
        "launch__registers_per_thread", "launch__grid_size", "launch__block_size", "sm__throughput.avg.pct_of_peak_sustained_elapsed",
        "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio", "launch__occupancy_limit_shared_mem"]


def main():
    rows = list(csv.reader(open(sys.argv[1], errors="ignore")))
    head = next(i for i, r in enumerate(rows) if "Kernel Name" in r)
    cols, units = rows[head], rows[head + 1]
    name_i = cols.index("Kernel Name")
    for r in rows[head + 2:]:
        if len(r) != len(cols):
            continue
        print(r[name_i][:90])
        for k in KEEP:
            hits = [i for i, c in enumerate(cols) if c.startswith(k)]
            for i in hits[:1]:
                print(f"    {cols[i]:<75} {r[i]:>16} {units[i]}")


if __name__ == "__main__":
    main()
