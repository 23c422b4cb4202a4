"""Training loop: gradient accumulation, mixed precision, the parallel layouts, checkpoints, logging.

Public surface and semantics follow the reference trainer (nanonemo/train/trainer.py:24-331):
``train(model_cfg, cfg, device=None, log_fn=None) -> list[dict]`` writes ``config.yaml`` and
``metrics.jsonl`` under ``out_dir``, sets the LR as a pure function of the step, evaluates on fixed
validation batches, checkpoints on a schedule / on a wall-clock or step budget agreed across ranks,
and resumes (weights, moments, LR position, loader position converted through the global sample
count so the data-parallel width may change).

What differs is underneath: the layout is a ``Strategy`` (parallel/strategy.py) that owns gradient
reduction, global-norm clipping and the update; on a GPU with the built library those are fused
kernels over the flat parameter store and the step ends with ONE device->host read that carries both
the loss and the gradient norm.
"""

import json
import time
from pathlib import Path
from typing import Callable

import torch

from nanonemo_b200 import parallel
from nanonemo_b200.data.loader import TokenLoader
from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.models.model import NanoNemo
from nanonemo_b200.parallel.strategy import LocalStrategy
from nanonemo_b200.train import checkpoint
from nanonemo_b200.train.config import TrainConfig, dump_config
from nanonemo_b200.train.optim import build_optimizer, lr_at
from nanonemo_b200.utils import nvtx
from nanonemo_b200.utils.env import git_info
from nanonemo_b200.utils.mfu import flops_per_token, mfu, peak_tflops

AMP_DTYPES = {"fp32": None, "fp16": torch.float16, "bf16": torch.bfloat16, "fp8": torch.bfloat16}


@torch.no_grad()
def evaluate(model, loader: TokenLoader, n_batches: int, loss_ctx=None) -> float:
    """Mean loss over the first `n_batches` validation batches (the same ones every call)."""
    loader.micro_step = 0
    model.eval()
    total = 0.0
    for _ in range(n_batches):
        x, y = loader.next_batch()
        total += float(model(x, y)[1])
    model.train()
    return total / n_batches


def static_grads(cfg: TrainConfig) -> bool:
    return cfg.compile == "reduce-overhead" or cfg.cuda_graph


def _lib_ok(device: str) -> bool:
    if not device.startswith("cuda"):
        return False
    from nanonemo_b200.ops import _lib

    return _lib.available()


def wants_store(model_cfg: ModelConfig, cfg: TrainConfig, device: str) -> bool:
    """The flat parameter store is used for DDP everywhere (its buckets are ranges of the flat
    gradient) and on a GPU whenever the fused update can run (no fp16 loss scaler in the way)."""
    if cfg.parallel == "ddp":
        return True
    return cfg.parallel == "none" and _lib_ok(device) and cfg.precision != "fp16"


def shadow_dtype(model_cfg: ModelConfig, cfg: TrainConfig):
    if not model_cfg.uses_sm100("linear_impl") and not model_cfg.uses_sm100("loss_kernel"):
        return None
    return {"bf16": torch.bfloat16, "fp8": torch.bfloat16, "fp16": torch.float16}.get(cfg.precision)


def build_model(model_cfg: ModelConfig, cfg: TrainConfig, device: str):
    """Returns (model, step_model); step_model is the torch.compile wrapper when `compile` is set and
    the model runs on the plain-PyTorch operators (the hand-written kernels are already fused, so
    `compile` has nothing to do on that path and is skipped)."""
    model = NanoNemo(model_cfg).to(device)
    model.residual_dtype = torch.float32 if cfg.residual_dtype == "fp32" else torch.bfloat16
    any_sm100 = any(model_cfg.uses_sm100(s) for s in ("norm_kernel", "swiglu_kernel", "rope_kernel", "attn_kernel",
                                                        "loss_kernel", "linear_impl", "embed_kernel"))
    if cfg.compile is None or any_sm100:
        return model, model
    # PyTorch-operator path: Inductor, and for reduce-overhead its own CUDA-graph trees (gradients accumulate into
    # the static flat gradient views outside the compiled region)
    return model, torch.compile(model, mode=None if cfg.compile == "default" else cfg.compile)


def build_parallel(model_cfg: ModelConfig, cfg: TrainConfig, d: parallel.Dist) -> LocalStrategy:
    """Lay the model out over the ranks according to cfg.parallel (+ the FP8 forward context)."""
    if cfg.precision == "fp8" and not model_cfg.fp8:
        raise ValueError("precision fp8 needs model.linear_impl: mxfp8 (or te)")
    strategy = _build_parallel(model_cfg, cfg, d)
    if cfg.precision == "fp8":
        from nanonemo_b200.fp8 import fp8_context

        strategy.fwd_ctx = fp8_context(cfg.fp8_recipe)
    return strategy


def _build_parallel(model_cfg: ModelConfig, cfg: TrainConfig, d: parallel.Dist) -> LocalStrategy:
    from nanonemo_b200.parallel.flat import FlatParams

    if cfg.parallel == "none":
        model, step_model = build_model(model_cfg, cfg, d.device)
        store = FlatParams(model, d.device, shadow_dtype(model_cfg, cfg)) if wants_store(model_cfg, cfg, d.device) else None
        strategy = LocalStrategy(model, store, step_model)
        # CUDA graphs: `cuda_graph: true`, or the reference's `compile: reduce-overhead` when the sm100 kernels run
        strategy.use_cuda_graph = d.device.startswith("cuda") and store is not None and step_model is model and (
            cfg.cuda_graph or cfg.compile == "reduce-overhead")
        return strategy
    if cfg.parallel == "ddp":
        from nanonemo_b200.parallel.ddp import DDPStrategy
        from nanonemo_b200.parallel.symm import make_grad_allreduce

        model, step_model = build_model(model_cfg, cfg, d.device)
        grad_alloc, finish = make_grad_allreduce(d, cfg.comm)
        store = FlatParams(model, d.device, shadow_dtype(model_cfg, cfg), grad_alloc=grad_alloc,
                           pad_to=256 * d.world * 8)
        strategy = DDPStrategy(model, d, store, cfg.ddp_bucket_mb, cfg.comm, symm=finish(store), step_model=step_model)
        # the fused all-reduce kernels keep their epochs on the device, so the hooks' launches can be captured
        strategy.use_cuda_graph = cfg.cuda_graph and strategy.fused and step_model is model
        return strategy
    if cfg.parallel == "fsdp":
        from nanonemo_b200.parallel.fsdp import build_fsdp

        return build_fsdp(model_cfg, cfg, d)
    from nanonemo_b200.parallel.tp import build_tp

    return build_tp(model_cfg, cfg, d)  # tp and the 2-D fsdp_tp mesh


def build_scaler(cfg: TrainConfig, device: str, sharded: bool = False):
    """fp16 only: loss scaling against gradient underflow; the sharded variant agrees on inf/nan across ranks."""
    if cfg.precision != "fp16":
        return None
    kind = device.split(":")[0]
    if sharded:
        from torch.distributed.fsdp.sharded_grad_scaler import ShardedGradScaler

        return ShardedGradScaler(kind)
    return torch.amp.GradScaler(kind)


def train_step(strategy: LocalStrategy, opt, loader: TokenLoader, accum: int, grad_clip: float,
               amp_dtype=None, scaler=None, keep_grads: bool = False, host_sync: bool = True):
    """One optimizer step over `accum` micro-batches -> (mean loss over ranks, pre-clip grad norm),
    both floats, fetched with a single device->host copy. The same copy carries the kernels' status
    flag (non-zero once a bounded wait inside a tensor-core pipeline or a collective ran out): the
    step raises on every rank that sees it instead of training on with a skipped collective.
    With host_sync=False the result is returned as one device tensor (loss, norm, status flag) and
    nothing waits for the GPU; the caller checks element 2 when it reads the tensor."""
    model = strategy.step_model
    loss_sum = None
    strategy.begin_step(opt, grad_clip)
    for i in range(accum):
        x, y = loader.next_batch()
        torch.compiler.cudagraph_mark_step_begin()  # no-op unless a compiled model replays CUDA graphs
        if getattr(strategy, "use_cuda_graph", False):
            loss = strategy.full_loss(strategy.graphed_micro_step(x, y, amp_dtype, accum, last=i == accum - 1))
            loss_sum = loss.clone() if loss_sum is None else loss_sum + loss
            continue
        with strategy.sync_ctx(i == accum - 1), strategy.loss_ctx():
            with nvtx.span("forward"), torch.autocast(x.device.type, dtype=amp_dtype, enabled=amp_dtype is not None), strategy.fwd_ctx():
                _, loss = model(x, y)
            loss = loss / accum  # the summed .grad is then the gradient of the mean loss
            with nvtx.span("backward"):
                (scaler.scale(loss) if scaler else loss).backward()
        loss = strategy.full_loss(loss.detach())
        loss_sum = loss if loss_sum is None else loss_sum + loss
    with nvtx.span("optimizer"):
        grad_norm = strategy.step(opt, grad_clip, scaler, keep_grads)
    flag = strategy.status_flag()
    parts = [parallel.all_mean(loss_sum.float()).reshape(()), grad_norm.float().reshape(())]
    both = torch.stack(parts + [flag.to(parts[0].device)] if flag is not None else parts)
    if not host_sync:
        return both
    values = both.tolist()  # the only host sync of the step
    if len(values) > 2 and values[2] != 0:
        strategy.raise_on_status()
    return values[0], values[1]


def train(model_cfg: ModelConfig, cfg: TrainConfig, device: str | None = None,
          log_fn: Callable[[dict], None] | None = None) -> list[dict]:
    """Train until cfg.total_steps optimizer steps or a session limit; returns rank 0's records."""
    d = parallel.init()
    if cfg.parallel != "none" and not d.enabled:
        raise ValueError(f"parallel={cfg.parallel!r} needs several processes: launch with torchrun")
    if cfg.parallel == "none" and d.world > 1:
        raise ValueError(f"{d.world} processes but parallel='none': set ddp, fsdp, tp or fsdp_tp")
    if device is not None and not d.enabled:
        d = parallel.Dist(device=device)
    device = d.device
    out_dir = Path(cfg.out_dir)
    if d.main:
        out_dir.mkdir(parents=True, exist_ok=True)
        (out_dir / "config.yaml").write_text(dump_config(model_cfg, cfg))

    torch.manual_seed(cfg.seed)
    strategy = build_parallel(model_cfg, cfg, d)
    model = strategy.model
    opt = build_optimizer(model, cfg.peak_lr, cfg.weight_decay, store=strategy.store)
    amp_dtype, scaler = AMP_DTYPES[cfg.precision], build_scaler(cfg, device, strategy.sharded_grads)
    train_loader = TokenLoader(cfg.data_dir, "train", cfg.seq_len, cfg.micro_batch, seed=cfg.seed,
                               rank=strategy.dp_rank, world_size=strategy.dp_world, device=device)
    val_loader = TokenLoader(cfg.data_dir, "val", cfg.seq_len, cfg.micro_batch, seed=cfg.seed, device=device)
    accum, total_steps = cfg.grad_accum(strategy.dp_world), cfg.total_steps
    on_cuda = device.startswith("cuda")
    peak = peak_tflops(torch.cuda.get_device_name()) if on_cuda else None
    flops_tok = flops_per_token(model_cfg, cfg.seq_len)

    ckpt = None
    if cfg.checkpointing:
        ckpt = checkpoint.Checkpointer(cfg.ckpt_dir or out_dir / "ckpt", d.main, use_async=cfg.ckpt_async)
    start_step, resumed_from = 0, None
    if cfg.resume_from:
        path = checkpoint.find_latest(cfg.resume_from)
        if path is None:
            raise FileNotFoundError(f"no checkpoint under {cfg.resume_from}")
        state = checkpoint.load(path, strategy, opt)
        consumed = state["micro_step"] * state.get("dp_world", 1)  # global count of micro-batches read
        if consumed % strategy.dp_world:
            raise ValueError(f"cannot split {consumed} consumed micro-batches over {strategy.dp_world} ranks")
        start_step, train_loader.micro_step = state["step"] + 1, consumed // strategy.dp_world
        if scaler and state.get("scaler"):
            scaler.load_state_dict(state["scaler"])
        resumed_from = str(path)

    def trainer_state(step: int) -> dict:
        return {"step": step, "micro_step": train_loader.micro_step,
                "scaler": scaler.state_dict() if scaler else None, "world": d.world,
                "dp_world": strategy.dp_world, "parallel": cfg.parallel}

    history: list[dict] = []
    metrics_file = (out_dir / "metrics.jsonl").open("a" if resumed_from else "w") if d.main else None

    def log(record: dict):
        if not d.main:
            return
        history.append(record)
        metrics_file.write(json.dumps(record) + "\n")
        metrics_file.flush()
        if log_fn:
            log_fn(record)

    log({"event": "start", "git": git_info(), "device": device, "params": model.num_params(),
         "grad_accum": accum, "total_steps": total_steps, "warmup_steps": cfg.warmup_steps,
         "parallel": cfg.parallel, "world": d.world, "start_step": start_step, "resumed_from": resumed_from,
         "kernels": {k: getattr(model_cfg.resolved(), k) for k in
                     ("norm_kernel", "swiglu_kernel", "rope_kernel", "attn_kernel", "loss_kernel", "linear_impl")},
         "inert_settings": cfg.inert_settings(any(model_cfg.uses_sm100(k) for k in ("norm_kernel", "attn_kernel", "linear_impl")))})

    t_session = t_last = time.perf_counter()
    last_logged = start_step - 1
    for step in range(start_step, total_steps):
        lr = lr_at(step, cfg.peak_lr, total_steps, cfg.warmup_steps, cfg.min_lr_ratio)
        for group in opt.param_groups:
            group["lr"] = lr
        loss, grad_norm = train_step(strategy, opt, train_loader, accum, cfg.grad_clip, amp_dtype, scaler,
                                     static_grads(cfg))
        is_last = step == total_steps - 1
        if step % cfg.log_every == 0 or is_last:
            if on_cuda:
                torch.cuda.synchronize()
            now = time.perf_counter()
            record = {"step": step, "loss": loss, "lr": lr, "grad_norm": grad_norm,
                      "tokens": (step + 1) * cfg.global_batch_tokens,
                      "tokens_per_s": (step - last_logged) * cfg.global_batch_tokens / (now - t_last)}
            if on_cuda:
                record["peak_mem_gb"] = torch.cuda.max_memory_allocated() / 2**30
            if scaler:
                record["loss_scale"] = scaler.get_scale()
            if peak:
                key = "bf16_tc" if "bf16_tc" in peak else "fp16_tc"
                record["mfu"] = mfu(record["tokens_per_s"] / d.world, flops_tok, peak[key])
            t_last, last_logged = now, step
            log(record)
        if (step + 1) % cfg.eval_every == 0 or is_last:
            with torch.autocast(device.split(":")[0], dtype=amp_dtype, enabled=amp_dtype is not None), strategy.loss_ctx():
                val_loss = evaluate(strategy.step_model if strategy.sharded_grads else model, val_loader, cfg.eval_batches)
            log({"step": step, "val_loss": val_loss})
            t_last, last_logged = time.perf_counter(), step  # eval time does not count toward tokens/s

        if ckpt:
            out_of_time = cfg.stop_after_min is not None and time.perf_counter() - t_session > 60 * cfg.stop_after_min
            stop = parallel.any_rank(out_of_time, device) or (
                cfg.max_steps is not None and step - start_step + 1 >= cfg.max_steps)
            if stop or is_last or (cfg.ckpt_every and (step + 1) % cfg.ckpt_every == 0):
                ckpt.save(step, strategy, opt, trainer_state(step))
                log({"step": step, "event": "checkpoint"})
                t_last, last_logged = time.perf_counter(), step
            if stop and not is_last:
                log({"step": step, "event": "stopped", "reason": "time limit" if out_of_time else "max_steps"})
                break

    if ckpt:
        ckpt.wait()
    if metrics_file:
        metrics_file.close()
    return history
