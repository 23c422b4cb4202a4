#!/usr/bin/env python
"""Where a training step spends its GPU time: kernel time per group from the PyTorch profiler (CUDA activity only).

    python scripts/step_breakdown.py --config configs/b200/single.yaml [--steps 3] [--set train.micro_batch=32] [--timeline]
    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node=2 scripts/step_breakdown.py \
        --config configs/b200/ddp.yaml --timeline

Prints one row per kernel group (GEMMs, attention forward / backward, norms, SwiGLU, RoPE, cross-entropy, optimizer,
collectives, everything else) with milliseconds per step and the share of the total. Times come from the profiler's kernel
records, so they add up to busy GPU time, not to wall-clock step time.

With --timeline the kernel records are also laid out in time (from the profiler's trace): wall time per step, busy time of the
compute stream, its largest idle gaps with the kernels on either side, and for the collective kernels how much of their run
time fell into such gaps, i.e. was EXPOSED rather than hidden under compute (the reference's scripts/nsys_comm.py reports only
the share of kernel time that is communication, not whether it overlapped).
"""

import argparse
import json
import sys
import tempfile
from collections import defaultdict
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

GROUPS = [  # first match wins
    ("tcgen05 GEMM (CTA pair)", ("gemm2_tcgen05",)),
    ("tcgen05 GEMM (single CTA)", ("gemm_tcgen05",)),
    ("flash attention backward", ("flash_bwd", "flash_delta", "flash_dq_convert")),
    ("flash attention forward", ("flash_fwd",)),
    ("add + RMSNorm", ("rmsnorm", "dw_reduce")),
    ("SwiGLU", ("swiglu",)),
    ("RoPE", ("rope",)),
    ("cross-entropy", ("ce_inplace", "ce_stats", "ce_grad")),
    ("embedding", ("embedding",)),
    ("AdamW / grad norm", ("adamw", "sumsq")),
    ("collectives", ("allreduce", "reduce_scatter", "allgather", "all_gather", "nccl")),
    ("MXFP8 quantise", ("mxfp8",)),
    ("library GEMM", ("cutlass", "cublas", "nvjet", "gemm")),
]


def group_of(name: str) -> str:
    low = name.lower()
    for label, keys in GROUPS:
        if any(k in low for k in keys):
            return label
    return "other"


COLLECTIVE_KEYS = ("allreduce", "reduce_scatter", "allgather", "all_gather", "nccl", "vp_embed", "peer_fetch", "sumsq_combine")


def timeline_report(trace_events: list, steps: int, top: int = 8) -> list[str]:
    """Lines describing how one rank's kernels were laid out in time. `trace_events`: the chrome-trace records of the
    profiler (dicts with ph == "X", cat == "kernel", ts / dur in microseconds and args.stream)."""
    kernels = sorted(({"name": e["name"], "t0": float(e["ts"]), "t1": float(e["ts"]) + float(e["dur"]), "stream": e.get("args", {}).get("stream", 0)}
                      for e in trace_events if e.get("ph") == "X" and e.get("cat") == "kernel"), key=lambda k: k["t0"])
    if not kernels:
        return ["no kernel records in the trace"]
    busy_by_stream = defaultdict(float)
    for k in kernels:
        busy_by_stream[k["stream"]] += k["t1"] - k["t0"]
    main_stream = max(busy_by_stream, key=busy_by_stream.get)
    comp = [k for k in kernels if k["stream"] == main_stream]
    wall = kernels[-1]["t1"] - kernels[0]["t0"]
    # idle intervals of the compute stream (merged coverage, then the holes)
    gaps, edge = [], comp[0]["t1"]
    prev = comp[0]
    for k in comp[1:]:
        if k["t0"] > edge:
            gaps.append((edge, k["t0"], prev["name"], k["name"]))
        if k["t1"] > edge:
            edge, prev = k["t1"], k
    idle = sum(b - a for a, b, _, _ in gaps)
    coll = [k for k in kernels if any(key in k["name"].lower() for key in COLLECTIVE_KEYS)]
    coll_busy = sum(k["t1"] - k["t0"] for k in coll)
    exposed = 0.0
    for k in coll:
        for a, b, _, _ in gaps:
            lo, hi = max(a, k["t0"]), min(b, k["t1"])
            if hi > lo:
                exposed += hi - lo
    ms = lambda us: us / 1e3 / steps
    out = [f"timeline ({steps} steps, this rank): wall {ms(wall):.2f} ms / step | compute stream busy {ms(busy_by_stream[main_stream]):.2f} | "
           f"compute stream idle {ms(idle):.2f} | collective kernels {ms(coll_busy):.2f} of which exposed (compute stream idle) {ms(exposed):.2f}",
           f"largest idle gaps of the compute stream (us, whole window):"]
    for a, b, before, after in sorted(gaps, key=lambda g: g[0] - g[1])[:top]:
        during = sorted({k["name"][:40] for k in kernels if k["stream"] != main_stream and k["t0"] < b and k["t1"] > a})
        out.append(f"  {b - a:8.1f}  after {before[:48]} | before {after[:48]} | other streams: {', '.join(during) or '-'}")
    return out


def main(argv=None):
    import torch
    from torch.profiler import ProfilerActivity, profile

    from nanonemo_b200 import parallel
    from nanonemo_b200.data.loader import DeviceBatches, TokenLoader
    from nanonemo_b200.train.config import apply_overrides, load_config
    from nanonemo_b200.train.optim import build_optimizer
    from nanonemo_b200.train.trainer import AMP_DTYPES, build_parallel, build_scaler, train_step

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--set", nargs="*", default=[], metavar="section.key=value")
    ap.add_argument("--timeline", action="store_true", help="also report idle gaps of the compute stream and exposed collective time")
    a = ap.parse_args(argv)
    model_cfg, cfg = apply_overrides(*load_config(a.config), a.set)
    d = parallel.init()
    if not d.device.startswith("cuda"):
        raise SystemExit("step_breakdown.py needs a CUDA device")
    strategy = build_parallel(model_cfg, cfg, d)
    opt = build_optimizer(strategy.model, cfg.peak_lr, cfg.weight_decay, store=strategy.store)
    amp, scaler = AMP_DTYPES[cfg.precision], build_scaler(cfg, d.device, strategy.sharded_grads)
    loader = TokenLoader(cfg.data_dir, "train", cfg.seq_len, cfg.micro_batch, seed=cfg.seed, rank=strategy.dp_rank,
                         world_size=strategy.dp_world, device=d.device)
    src, accum = DeviceBatches(loader, 4), cfg.grad_accum(strategy.dp_world)
    for _ in range(3):
        train_step(strategy, opt, src, accum, cfg.grad_clip, amp, scaler, host_sync=False)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(a.steps):
            train_step(strategy, opt, src, accum, cfg.grad_clip, amp, scaler, host_sync=False)
        torch.cuda.synchronize()
    per_group, per_kernel = defaultdict(float), defaultdict(float)
    for ev in prof.key_averages():
        us = getattr(ev, "device_time_total", None) or getattr(ev, "cuda_time_total", 0.0)
        if us:
            per_group[group_of(ev.key)] += us / 1e3 / a.steps
            per_kernel[ev.key] += us / 1e3 / a.steps
    if d.main:
        total = sum(per_group.values())
        print(f"GPU kernel time per step: {total:.2f} ms over {a.steps} steps ({cfg.parallel}, world {d.world})")
        print("| group | ms / step | share |\n|---|---|---|")
        for label, ms in sorted(per_group.items(), key=lambda kv: -kv[1]):
            print(f"| {label} | {ms:.2f} | {100 * ms / total:.1f} % |")
        print("\ntop kernels:")
        for name, ms in sorted(per_kernel.items(), key=lambda kv: -kv[1])[:12]:
            print(f"  {ms:7.3f} ms  {name[:110]}")
        if a.timeline:
            with tempfile.TemporaryDirectory() as tmp:
                path = Path(tmp) / "trace.json"
                prof.export_chrome_trace(str(path))
                events = json.loads(path.read_text()).get("traceEvents", [])
            print()
            print("\n".join(timeline_report(events, a.steps)))
    parallel.destroy()


if __name__ == "__main__":
    main()
