"""Timing harness for kernel micro-benchmarks on B200.

Each measurement: warm-up calls, the call captured into a CUDA graph, then `iters` timed replays; before
every replay a buffer larger than the L2 cache is overwritten so the kernel starts cold (the size comes
from the device's L2 attribute — 126 MB on B200, so the reference's fixed 64 MB flush,
benchmarks/kernels/common.py:42, would not be enough); CUDA events on the launching stream bracket the
replay, the host synchronises once at the end, and the median is reported (the reference harness times
graph replays for the same reason, benchmarks/kernels/common.py:30-64). Clock samples are taken during the run and the result carries the compact clocks record.
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


def _captured(fn, warmup: int):
    """`fn` recorded into a CUDA graph (after warm-up on a side stream, as capture requires), or None when the call cannot
    be captured (it synchronises, or allocates outside the graph's pool)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(graph):
            fn()
    except Exception as e:  # noqa: BLE001 - fall back to timing plain launches
        print(f"[time_ms] not capturable, timing plain launches instead: {type(e).__name__}: {str(e)[:200]}", file=sys.stderr)
        torch.cuda.synchronize()
        return None
    return graph


def time_ms(fn, iters: int = 30, warmup: int = 5, flush: bool = True, graph: bool = True, spread: bool = False):
    """Median device time of one call of `fn` in ms. By default the call is captured into a CUDA graph once and every timed
    repetition is flush -> event -> graph replay -> event with a single synchronize at the end, so neither the host's launch
    overhead nor its jitter lands between the two events (a 40 us kernel timed around a Python-level launch carries a few
    us of noise). `graph=False` times plain launches. `spread=True` returns {"median", "p20", "p80"} instead."""
    replay = _captured(fn, warmup) if graph else None
    call = replay.replay if replay is not None else fn
    if replay is None:
        for _ in range(warmup):
            fn()
    for _ in range(3):
        call()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for first, second in pairs:
        if flush:
            l2_flush()
        first.record()
        call()
        second.record()
    torch.cuda.synchronize()
    times = sorted(a.elapsed_time(b) for a, b in pairs)
    if spread:
        pick = lambda q: times[min(len(times) - 1, int(q * len(times)))]
        return {"median": median(times), "p20": pick(0.2), "p80": pick(0.8)}
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
