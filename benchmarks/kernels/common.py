"""Timing harness for kernel micro-benchmarks on B200.

Each measurement: warm-up calls, then `iters` timed calls; before every timed call a buffer larger
than the L2 cache is overwritten so the kernel starts cold (the size comes from the device's L2
attribute — 126 MB on B200, so the reference's fixed 64 MB flush, benchmarks/kernels/common.py:42,
would not be enough); CUDA events on the launching stream bracket the call; the median is
reported. Clock samples are taken during the run and the result carries the compact clocks record.
Bandwidth figures are computed against the MINIMUM bytes the operator must move.
"""

import json
import sys
from pathlib import Path
from statistics import median

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from nanonemo_b200.utils.env import measured_peaks  # noqa: E402
from nanonemo_b200.utils.gpumon import GpuMonitor, clocks_record  # noqa: E402

_flush = None


def l2_flush():
    global _flush
    if _flush is None:
        l2 = torch.cuda.get_device_properties(0).L2_cache_size
        _flush = torch.empty(max(2 * l2, 256 << 20), dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_ms(fn, iters: int = 30, warmup: int = 5, flush: bool = True) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            l2_flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return median(times)


def peaks() -> dict:
    m = measured_peaks() or {}
    return {"hbm_gbs": m.get("hbm_gbs", 6650.0), "bf16_tflops": m.get("bf16_tflops", 1590.0),
            "source": "measured" if m else "fallback"}


def run(name: str, rows_fn, out_dir: str = "results/kernels"):
    """rows_fn() -> list of dict rows; writes results/kernels/<name>.json and prints a table."""
    with GpuMonitor(200) as mon:
        rows = rows_fn()
    result = {"bench": name, "device": torch.cuda.get_device_name(), "peaks": peaks(), "rows": rows,
              "clocks": clocks_record(mon.samples)}
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / f"{name}.json").write_text(json.dumps(result, indent=1))
    keys = list(rows[0].keys()) if rows else []
    print(" | ".join(keys))
    for r in rows:
        print(" | ".join(f"{r[k]:.4g}" if isinstance(r[k], float) else str(r[k]) for k in keys))
    print("clocks:", result["clocks"])
    return result
