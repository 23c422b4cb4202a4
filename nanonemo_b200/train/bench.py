"""Training-throughput benchmark on the real optimizer step: warm-up excluded, trials x steps timed.

Same protocol as the reference harness (nanonemo/train/bench.py:54-159): the objects are built by
the trainer's own functions, each step is bracketed by CUDA events, clocks are sampled in the
background, ``NANONEMO_PROFILE=1`` opens the ``cudaProfilerStart/Stop`` window around the first
trial. One rule differs: with several ranks the per-step times are reduced with MAX over ranks
before any throughput is computed (the reference reports rank 0's view only, bench.py:63).
"""

import os
import time
from dataclasses import asdict
from statistics import median

import torch

from nanonemo_b200 import parallel
from nanonemo_b200.data.loader import TokenLoader
from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.train.config import TrainConfig
from nanonemo_b200.train.optim import build_optimizer, lr_at
from nanonemo_b200.train.trainer import AMP_DTYPES, build_parallel, build_scaler, static_grads, train_step
from nanonemo_b200.utils.env import capture_env
from nanonemo_b200.utils.gpumon import GpuMonitor, clock_floor, clocks_record, locked_sm_mhz, summarize, throttle_flags
from nanonemo_b200.utils.mfu import flops_per_token, mfu, peak_tflops


def _spread(values) -> dict:
    values = list(values)
    return {"median": median(values), "min": min(values), "max": max(values)}


class StepTimer:
    """Per-step durations in ms: CUDA events on the launching stream, perf_counter on the CPU."""

    def __init__(self, n_steps: int, cuda: bool):
        self.cuda = cuda
        self.marks = ([torch.cuda.Event(enable_timing=True) for _ in range(n_steps + 1)] if cuda
                      else [0.0] * (n_steps + 1))

    def mark(self, i: int):
        if self.cuda:
            self.marks[i].record()
        else:
            self.marks[i] = time.perf_counter()

    def step_ms(self) -> list[float]:
        if self.cuda:
            torch.cuda.synchronize()
            return [a.elapsed_time(b) for a, b in zip(self.marks, self.marks[1:])]
        return [(b - a) * 1e3 for a, b in zip(self.marks, self.marks[1:])]


def max_over_ranks(step_ms: list[float], device: str) -> list[float]:
    t = torch.tensor(step_ms, dtype=torch.float64, device=device if device.startswith("cuda") else "cpu")
    return parallel.all_max(t).tolist()


def benchmark(model_cfg: ModelConfig, cfg: TrainConfig, steps: int = 50, trials: int = 3, warmup_steps: int = 5,
              device: str | None = None, monitor_interval_ms: int = 200) -> dict:
    """Every rank runs this under torchrun; the result is identical on all ranks (times are max over ranks)."""
    d = parallel.init() if device is None else parallel.Dist(device=device)
    device = d.device
    cuda = device.startswith("cuda")
    env = capture_env()

    torch.manual_seed(cfg.seed)
    strategy = build_parallel(model_cfg, cfg, d)
    model = strategy.model
    opt = build_optimizer(model, cfg.peak_lr, cfg.weight_decay, store=strategy.store)
    amp_dtype, scaler = AMP_DTYPES[cfg.precision], build_scaler(cfg, device, strategy.sharded_grads)
    loader = TokenLoader(cfg.data_dir, "train", cfg.seq_len, cfg.micro_batch, seed=cfg.seed,
                         rank=strategy.dp_rank, world_size=strategy.dp_world, device=device)
    accum = cfg.grad_accum(strategy.dp_world)
    total = warmup_steps + steps * trials
    lr_warmup = max(1, round(cfg.warmup_frac * total))
    step = 0

    def run_step():
        nonlocal step
        for group in opt.param_groups:
            group["lr"] = lr_at(step, cfg.peak_lr, total, lr_warmup, cfg.min_lr_ratio)
        step += 1
        return train_step(strategy, opt, loader, accum, cfg.grad_clip, amp_dtype, scaler, static_grads(cfg))

    t0 = time.perf_counter()
    for _ in range(warmup_steps):
        run_step()
    if cuda:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
    warmup_s = time.perf_counter() - t0

    profile = os.environ.get("NANONEMO_PROFILE") == "1" and cuda
    locked = locked_sm_mhz()
    trial_results = []
    with GpuMonitor(monitor_interval_ms, gpu_index=d.local_rank) as mon:
        for trial in range(trials):
            if d.enabled:
                torch.distributed.barrier()
            if profile and trial == 0:
                torch.cuda.profiler.start()
            timer = StepTimer(steps, cuda)
            losses = []
            t_start = time.monotonic()
            timer.mark(0)
            for i in range(steps):
                losses.append(run_step()[0])
                timer.mark(i + 1)
            step_ms = max_over_ranks(timer.step_ms(), device)
            if profile and trial == 0:
                torch.cuda.profiler.stop()
            t_end = time.monotonic()
            window = mon.window(t_start, t_end)
            trial_results.append({
                "tokens_per_s": steps * cfg.global_batch_tokens / (sum(step_ms) / 1e3),
                "step_ms": step_ms, "loss_first": losses[0], "loss_last": losses[-1],
                "loss_scale": scaler.get_scale() if scaler else None,
                "gpu": summarize(window), "clocks": clocks_record(window),
            })

    tps = [t["tokens_per_s"] for t in trial_results]
    flops_tok = flops_per_token(model_cfg, cfg.seq_len)
    peak = peak_tflops(torch.cuda.get_device_name()) if cuda else None
    return {
        "bench": {"steps": steps, "trials": trials, "warmup_steps": warmup_steps, "grad_accum": accum,
                  "tokens_per_step": cfg.global_batch_tokens, "device": device, "world": d.world,
                  "parallel": cfg.parallel, "timing": "cuda events, max over ranks" if cuda else "perf_counter"},
        "tokens_per_s": _spread(tps),
        "step_ms": _spread(median(t["step_ms"]) for t in trial_results),
        "flops_per_token": flops_tok,
        "achieved_tflops": median(tps) * flops_tok / 1e12,
        "peak_tflops": peak,
        "mfu": {k: _spread(mfu(x / d.world, flops_tok, v) for x in tps) for k, v in peak.items() if v} if peak else None,
        "peak_mem_gb": {"allocated": torch.cuda.max_memory_allocated() / 2**30,
                        "reserved": torch.cuda.max_memory_reserved() / 2**30} if cuda else None,
        "warmup_s": warmup_s,
        "locked_sm_mhz": locked,
        "throttle_flags": throttle_flags([t["gpu"] for t in trial_results],
                                         min_mhz=clock_floor(locked, torch.cuda.get_device_name())) if cuda else [],
        "trials": trial_results,
        "params": model.num_params(),
        "config": {"model": asdict(model_cfg), "train": asdict(cfg)},
        "env": env,
    }
