"""Training-throughput benchmark on the real optimizer step.

``benchmark(model_cfg, cfg, steps, trials, warmup_steps)`` builds the run with the trainer's own constructors
(strategy, optimizer, loader), spends ``warmup_steps`` untimed steps, then times ``trials`` groups of ``steps``
optimizer steps. Every step boundary gets a time stamp on the launching stream (a CUDA event; ``perf_counter`` on the
CPU), the per-step durations of all ranks are combined with MAX before any rate is computed, and a background sampler
records the GPU's clocks so that each trial carries its own clock summary. ``NANONEMO_PROFILE=1`` opens the
``cudaProfilerStart/Stop`` window around the first trial for an external profiler's capture range.

The result dictionary has the fields of the reference harness (nanonemo/train/bench.py:54-159: tokens/s spread, step
time, FLOPs per token, achieved TFLOP/s, MFU per peak, peak memory, warm-up seconds, declared clock lock, throttle
flags, per-trial records, parameter count, resolved config, environment); where the reference reports rank 0's own
timings, this one reports the slowest rank's.
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
    ordered = sorted(values)
    return {"median": median(ordered), "min": ordered[0], "max": ordered[-1]}


class StepTimer:
    """Stamps step boundaries and hands back the durations between consecutive stamps in milliseconds. On a GPU a
    stamp is a CUDA event recorded on the current stream, read only after the trial (one synchronize); on the CPU it
    is ``perf_counter``."""

    def __init__(self, n_steps: int, cuda: bool):
        self.cuda = cuda
        self._stamps = []
        self._pool = [torch.cuda.Event(enable_timing=True) for _ in range(n_steps + 1)] if cuda else None

    def mark(self, i: int | None = None) -> None:
        if self.cuda:
            event = self._pool[len(self._stamps)]
            event.record()
            self._stamps.append(event)
        else:
            self._stamps.append(time.perf_counter())

    def step_ms(self) -> list[float]:
        pairs = list(zip(self._stamps, self._stamps[1:]))
        if self.cuda:
            torch.cuda.synchronize()
            return [first.elapsed_time(second) for first, second in pairs]
        return [(second - first) * 1e3 for first, second in pairs]


def max_over_ranks(step_ms: list[float], device: str) -> list[float]:
    """Per-step durations as seen by the slowest rank (identity without a process group)."""
    where = device if device.startswith("cuda") else "cpu"
    return parallel.all_max(torch.tensor(step_ms, dtype=torch.float64, device=where)).tolist()


class _Run:
    """The objects of one benchmarked training run and the step function that drives them."""

    def __init__(self, model_cfg: ModelConfig, cfg: TrainConfig, d: parallel.Dist, planned_steps: int):
        self.cfg, self.d = cfg, d
        torch.manual_seed(cfg.seed)
        self.strategy = build_parallel(model_cfg, cfg, d)
        self.opt = build_optimizer(self.strategy.model, cfg.peak_lr, cfg.weight_decay, store=self.strategy.store)
        self.amp_dtype = AMP_DTYPES[cfg.precision]
        self.scaler = build_scaler(cfg, d.device, self.strategy.sharded_grads)
        self.loader = TokenLoader(cfg.data_dir, "train", cfg.seq_len, cfg.micro_batch, seed=cfg.seed, rank=self.strategy.dp_rank,
                                  world_size=self.strategy.dp_world, device=d.device)
        self.accum = cfg.grad_accum(self.strategy.dp_world)
        # a short schedule of its own over everything this benchmark will run: warm-up fraction as configured
        self.planned = planned_steps
        self.lr_warmup = max(1, round(cfg.warmup_frac * planned_steps))
        self.done = 0

    def step(self) -> tuple[float, float]:
        lr = lr_at(self.done, self.cfg.peak_lr, self.planned, self.lr_warmup, self.cfg.min_lr_ratio)
        for group in self.opt.param_groups:
            group["lr"] = lr
        self.done += 1
        return train_step(self.strategy, self.opt, self.loader, self.accum, self.cfg.grad_clip, self.amp_dtype, self.scaler,
                          static_grads(self.cfg))

    def timed_trial(self, steps: int, cuda: bool, profile: bool) -> tuple[list[float], list[float], tuple[float, float]]:
        """-> (per-step ms of the slowest rank, losses, (t_start, t_end) on the monotonic clock)."""
        if self.d.enabled:
            torch.distributed.barrier()
        if profile:
            torch.cuda.profiler.start()
        timer = StepTimer(steps, cuda)
        began = time.monotonic()
        timer.mark()
        losses = []
        for _ in range(steps):
            losses.append(self.step()[0])
            timer.mark()
        per_step = max_over_ranks(timer.step_ms(), self.d.device)
        if profile:
            torch.cuda.profiler.stop()
        return per_step, losses, (began, time.monotonic())


def benchmark(model_cfg: ModelConfig, cfg: TrainConfig, steps: int = 50, trials: int = 3, warmup_steps: int = 5,
              device: str | None = None, monitor_interval_ms: int = 200) -> dict:
    """Every rank calls this under torchrun; all ranks return the same numbers (times are max over ranks)."""
    d = parallel.init() if device is None else parallel.Dist(device=device)
    cuda = d.device.startswith("cuda")
    env = capture_env()  # before any load: idle clocks
    run = _Run(model_cfg, cfg, d, warmup_steps + steps * trials)

    warm_began = time.perf_counter()
    for _ in range(warmup_steps):
        run.step()
    if cuda:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
    warmup_s = time.perf_counter() - warm_began

    want_profile = cuda and os.environ.get("NANONEMO_PROFILE") == "1"
    records = []
    with GpuMonitor(monitor_interval_ms, gpu_index=d.local_rank) as monitor:
        for index in range(trials):
            per_step, losses, (t0, t1) = run.timed_trial(steps, cuda, want_profile and index == 0)
            seen = monitor.window(t0, t1)
            records.append({
                "tokens_per_s": steps * cfg.global_batch_tokens / (sum(per_step) / 1e3),
                "step_ms": per_step,
                "loss_first": losses[0],
                "loss_last": losses[-1],
                "loss_scale": run.scaler.get_scale() if run.scaler else None,
                "gpu": summarize(seen),
                "clocks": clocks_record(seen),
            })

    rates = [r["tokens_per_s"] for r in records]
    flops_tok = flops_per_token(model_cfg, cfg.seq_len)
    name = torch.cuda.get_device_name() if cuda else None
    peaks = peak_tflops(name) if cuda else None
    lock = locked_sm_mhz()
    result = {
        "bench": {"steps": steps, "trials": trials, "warmup_steps": warmup_steps, "grad_accum": run.accum,
                  "tokens_per_step": cfg.global_batch_tokens, "device": d.device, "world": d.world, "parallel": cfg.parallel,
                  "timing": "cuda events, max over ranks" if cuda else "perf_counter"},
        "tokens_per_s": _spread(rates),
        "step_ms": _spread(median(r["step_ms"]) for r in records),
        "flops_per_token": flops_tok,
        "achieved_tflops": median(rates) * flops_tok / 1e12,
        "peak_tflops": peaks,
        "mfu": None,
        "peak_mem_gb": None,
        "warmup_s": warmup_s,
        "locked_sm_mhz": lock,
        "throttle_flags": [],
        "trials": records,
        "params": run.strategy.model.num_params(),
        "config": {"model": asdict(model_cfg), "train": asdict(cfg)},
        "env": env,
    }
    if peaks:
        result["mfu"] = {key: _spread(mfu(rate / d.world, flops_tok, peak) for rate in rates) for key, peak in peaks.items() if peak}
    if cuda:
        result["peak_mem_gb"] = {"allocated": torch.cuda.max_memory_allocated() / 2**30, "reserved": torch.cuda.max_memory_reserved() / 2**30}
        result["throttle_flags"] = throttle_flags([r["gpu"] for r in records], min_mhz=clock_floor(lock, name))
    return result
