#!/usr/bin/env python
"""Headline benchmark: training tokens/s of NanoNemo-114M, DDP, bf16 with fp32 master weights.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W [--impl reference]

Config (weak scaling): 12 layers, d_model 768, 12 query / 4 KV heads, SwiGLU 2048, vocab 50,304,
seq 1024, micro-batch 32 per GPU, one micro-batch per optimizer step, AdamW + global-norm clip,
uniform-random token ids in [0, 50257), random-init weights. Prints ONE JSON line on rank 0.

Two numbers are measured on the same objects:
* ``value``: K steps timed on the device (CUDA events on the launching stream, barrier +
  synchronize on both sides, max over ranks) with the step's inputs already resident on the GPU and
  no host read inside the loop — forward, backward, gradient all-reduce, clip and AdamW all included;
* ``e2e``: the same K steps through the public ``train_step`` API with, every step, the H2D copy of
  that step's token ids from pinned host memory and the D2H read of the loss and gradient norm.
``--impl reference`` runs the unmodified reference package from baseline/_ref through its own
``benchmark()`` entry point on the same shapes (see baseline/run_reference.py).
"""

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BASELINE_TOKENS_PER_S = None  # the reference publishes no B200 number (BASELINE.json "published": {})
MICRO_BATCH, SEQ_LEN = 32, 1024


def headline_config(micro_batch: int, seq_len: int, world: int, parallel: str) -> dict:
    """The `config` entry of the JSON line: the same keys and values for both arms (what differs between the arms is the
    implementation, printed under `stack`)."""
    dp = 1 if parallel == "tp" else world
    return {"model": "NanoNemo-114M (12L, d768, 12Q/4KV, ff2048, vocab 50304)", "global_batch": micro_batch * dp,
            "seq_len": seq_len, "micro_batch_per_gpu": micro_batch,
            "parallelism": {"ddp": f"dp{world}", "none": "dp1", "fsdp": f"fsdp{world}", "tp": f"tp{world}+sp"}[parallel],
            "optimizer": "AdamW + clip 1.0, fp32 master weights",
            "l2": "no flush: per-step working set (0.46 GB weights + ~10 GB activations) is far larger than the 126 MB L2"}


def measured_peaks() -> dict:
    """bf16 GEMM throughput measured on this pool's B200 by the driver (burst and sustained TFLOP/s), if the file is there."""
    try:
        return json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except (OSError, ValueError):
        return {}


def parse():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--micro-batch", type=int, default=MICRO_BATCH)
    ap.add_argument("--kernels", default="sm100", choices=["sm100", "torch"],
                    help="operator implementation of this framework's arm (torch = the oracle path)")
    ap.add_argument("--parallel", default="ddp", choices=["ddp", "fsdp", "tp"],
                    help="layout for N > 1 (the headline number is ddp; fsdp / tp give the other BASELINE configs)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel from the host instead of replaying the micro-batch from a CUDA graph (ddp / single GPU)")
    ap.add_argument("--bucket-mb", type=float, default=100.0, help="gradient bucket size of the data-parallel all-reduce (MiB)")
    ap.add_argument("--set", nargs="*", default=[], metavar="section.key=value")
    return ap.parse_args()


def run_ours(a):
    import torch
    import torch.distributed as dist

    from nanonemo_b200 import parallel
    from nanonemo_b200.data.loader import DeviceBatches, TokenLoader
    from nanonemo_b200.models.config import ModelConfig
    from nanonemo_b200.ops import _lib
    from nanonemo_b200.train.config import TrainConfig, apply_overrides
    from nanonemo_b200.train.optim import build_optimizer, lr_at
    from nanonemo_b200.train.trainer import AMP_DTYPES, build_parallel, build_scaler, train_step
    from nanonemo_b200.utils.gpumon import GpuMonitor, clocks_record
    from nanonemo_b200.utils.mfu import flops_per_token

    d = parallel.init()
    world = d.world
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")
    if not d.device.startswith("cuda"):
        raise SystemExit("bench.py needs CUDA GPUs")
    if a.kernels == "sm100" and not _lib.available():
        raise SystemExit("the kernel library is not built: python -c 'import __graft_entry__ as g; g.build()'")
    model_cfg = ModelConfig.sm100() if a.kernels == "sm100" else ModelConfig(attn_backend="mem_efficient")
    par = a.parallel if world > 1 else "none"
    dp = 1 if par == "tp" else world  # tensor parallel: one replica = the whole group
    cfg = TrainConfig(data_dir="synthetic", out_dir="runs/bench", seq_len=SEQ_LEN, micro_batch=a.micro_batch,
                      global_batch_tokens=a.micro_batch * SEQ_LEN * dp, total_tokens=10**12, precision="bf16",
                      parallel=par, ddp_bucket_mb=a.bucket_mb, fsdp_prefetch=True, eval_every=10**9,
                      cuda_graph=par in ("none", "ddp") and a.kernels == "sm100" and not a.no_graph)
    model_cfg, cfg = apply_overrides(model_cfg, cfg, a.set)

    # the clock sampler starts first so that it is already delivering samples when the timed region begins
    mon = GpuMonitor(100, gpu_index=d.local_rank)
    mon.__enter__()
    torch.manual_seed(cfg.seed)
    strategy = build_parallel(model_cfg, cfg, d)
    opt = build_optimizer(strategy.model, cfg.peak_lr, cfg.weight_decay, store=strategy.store)
    amp, scaler = AMP_DTYPES[cfg.precision], build_scaler(cfg, d.device, strategy.sharded_grads)
    loader = TokenLoader(cfg.data_dir, "train", cfg.seq_len, cfg.micro_batch, seed=cfg.seed, rank=strategy.dp_rank,
                         world_size=strategy.dp_world, device=d.device)
    accum = cfg.grad_accum(strategy.dp_world)
    staged = DeviceBatches(loader, 8)
    total = 2 * (a.warmup + a.steps)
    n = [0]

    def step(src, host_sync):
        for g in opt.param_groups:
            g["lr"] = lr_at(n[0], cfg.peak_lr, total, max(1, total // 50), cfg.min_lr_ratio)
        n[0] += 1
        return train_step(strategy, opt, src, accum, cfg.grad_clip, amp, scaler, host_sync=host_sync)

    def fence():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    # End-to-end mode reads every step's (loss, grad norm) back to the host, but one step late: the device -> host copy of
    # step i is enqueued behind step i and collected after step i + 1 has been launched, so the GPU never waits for the host
    # (the usual way a training loop logs its loss). Each step still does its own pinned host -> device copy of the batch.
    slots = [(torch.empty(3, dtype=torch.float32).pin_memory(), torch.cuda.Event()) for _ in range(2)]

    def collect(buf):
        vals = buf.tolist()
        if vals[2] != 0:  # a bounded wait inside a kernel ran out: the step's work was skipped, the number would be a lie
            strategy.raise_on_status()
        return vals

    def timed(src, host_sync):
        fence()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.monotonic()
        e0.record()
        last, pending = None, None
        for i in range(a.steps):
            out = step(src, False)
            if not host_sync:
                last = out
                continue
            buf, ev = slots[i & 1]
            buf.copy_(out, non_blocking=True)
            ev.record()
            if pending is not None:
                pending[1].synchronize()
                last = collect(pending[0])
            pending = (buf, ev)
        if pending is not None:
            pending[1].synchronize()
            last = collect(pending[0])
        e1.record()
        fence()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=d.device)
        return parallel.all_max(ms).item(), (t0, time.monotonic()), last

    for _ in range(a.warmup):
        step(staged, False)
    fence()
    try:
        # end-to-end region first, device-only region second: on a power-capped part whichever region runs later sees
        # slightly lower clocks, and the end-to-end figure is the one compared across implementations
        for _ in range(min(2, a.warmup)):
            step(loader, True)  # warm the pinned-host input path
        ms_e2e, win_e2e, last_e2e = timed(loader, True)
        launches0 = _lib.LAUNCHES + strategy.launches
        ms_dev, win_dev, last = timed(staged, False)
        launches = _lib.LAUNCHES + strategy.launches - launches0
        last = last.tolist()
        if len(last) > 2 and last[2] != 0:
            strategy.raise_on_status()
        loss_dev = float(last[0])
        time.sleep(0.25)  # let the sampler flush the last lines of the window
    finally:
        mon.__exit__(None, None, None)
    tokens = a.steps * cfg.global_batch_tokens
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    samples = mon.window(*win_dev) or mon.window(win_e2e[0], win_dev[1])  # a very short device-timed region may fall between two samples
    clocks = clocks_record(samples)
    flops_tok = flops_per_token(model_cfg, cfg.seq_len)
    peaks = measured_peaks()
    if d.main:
        print(json.dumps({
            "metric": "train tokens/s (device-timed, max over ranks)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_dev / a.steps,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
            "dtype": "bf16", "data": "synthetic uniform-random token ids in [0, 50257); random-init weights",
            "impl": "ours", "kernels": a.kernels,
            "config": headline_config(cfg.micro_batch, cfg.seq_len, world, par),
            "stack": "tcgen05 GEMMs with fused RoPE / SwiGLU / softmax-statistics epilogues, tcgen05 FlashAttention, fused norms, "
                     "peer-memory collective kernels on a side stream, one-kernel clip + AdamW"
                     + (", micro-batch replayed from a CUDA graph" if getattr(strategy, "use_cuda_graph", False) else ""),
            "mfu_vs_nominal_2250": value / world * flops_tok / 2250e12,
            "mfu_vs_measured_burst": (value / world * flops_tok / (peaks["bf16_tflops"] * 1e12)) if peaks.get("bf16_tflops") else None,
            "mfu_vs_measured_sustained": (value / world * flops_tok / (peaks["bf16_tflops_sustained"] * 1e12))
            if peaks.get("bf16_tflops_sustained") else None,
            "comparable": "e2e.value (both arms time their public train_step with the host copies inside the region)",
            "loss_last": loss_dev,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                    "h2d_bytes_per_step": loader.h2d_bytes_per_batch * accum, "d2h_bytes_per_step": 12,
                    "loss_last": last_e2e[0], "result_read": "every step, collected one step late (non-blocking copy + event)"},
            "gpu_launches": launches,
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "n_samples": clocks["n_samples"]},
        }), flush=True)
    parallel.destroy()


def main():
    a = parse()
    if a.impl == "reference":
        from baseline.run_reference import main as ref_main

        return ref_main(a, headline_config)
    return run_ours(a)


if __name__ == "__main__":
    main()
