"""Run configuration: one YAML file with a ``model:`` and a ``train:`` section defines a run.

Field names, defaults, cross-field validation and typo rejection follow the reference
(nanonemo/train/config.py:11-103) so its YAML files load unchanged. Additions for this framework:
``parallel`` accepts ``fsdp_tp`` (a 2-D mesh: FSDP over ``world / tp_size`` groups of ``tp_size``
tensor-parallel ranks), ``tp_size``, ``comm`` (``fused``: in-kernel NVLink collectives through
symmetric memory; ``nccl``: torch.distributed only, which is also what CPU/gloo runs use),
``residual_dtype`` and ``cuda_graph``. ``data_dir: synthetic`` selects an in-memory uniform-random
token source.
"""

from dataclasses import asdict, dataclass, fields, replace
from pathlib import Path

import yaml

from nanonemo_b200.models.config import ModelConfig

PARALLEL = ("none", "ddp", "fsdp", "tp", "fsdp_tp")


@dataclass
class TrainConfig:
    data_dir: str = "data/nemotron_cc"
    out_dir: str = "runs/default"
    seed: int = 0
    seq_len: int = 1024
    micro_batch: int = 2
    global_batch_tokens: int = 524_288
    total_tokens: int = 2_500_000_000
    peak_lr: float = 6e-4
    min_lr_ratio: float = 0.1
    warmup_frac: float = 0.02
    weight_decay: float = 0.1
    grad_clip: float = 1.0
    eval_every: int = 50
    eval_batches: int = 20
    log_every: int = 1
    precision: str = "fp32"  # fp32 | fp16 (autocast + GradScaler) | bf16 (autocast) | fp8 (bf16 + MXFP8 GEMMs)
    fp8_recipe: str = "delayed"  # accepted for config compatibility; MXFP8 block scales need no history
    compile: str | None = None  # accepted values as in the reference; see `Setup` for what each maps to here
    wandb_project: str | None = None
    wandb_run_name: str | None = None
    parallel: str = "none"
    ddp_bucket_mb: float = 25.0
    ddp_grad_as_bucket_view: bool = False
    fsdp_param_dtype: str = "fp32"  # fp32 | fp16 | bf16: dtype of the gathered parameters
    fsdp_reshard_after_forward: bool = True
    fsdp_prefetch: bool = False
    fsdp_compile_blocks: bool = False
    ckpt_every: int = 0
    ckpt_dir: str | None = None
    ckpt_async: bool = True
    resume_from: str | None = None
    stop_after_min: float | None = None
    max_steps: int | None = None
    # --- additions
    tp_size: int | None = None  # tensor-parallel degree for parallel=tp (default: world) / fsdp_tp
    comm: str = "auto"  # auto | fused | nccl
    residual_dtype: str = "fp32"  # dtype of the residual stream on the sm100 path: fp32 | bf16
    fsdp_gemm_gather: bool = False  # fsdp forward: a block's parameter all-gather runs inside its QKV GEMM kernel (no side-stream gather)
    cuda_graph: bool = False  # replay forward + backward (+ the ddp gradient all-reduce) of a micro-batch from a CUDA graph

    def __post_init__(self):
        if self.fp8_recipe not in ("delayed", "current", "mxfp8"):
            raise ValueError(f"unknown fp8_recipe {self.fp8_recipe!r}")
        if self.precision not in ("fp32", "fp16", "bf16", "fp8"):
            raise ValueError(f"unknown precision {self.precision!r}")
        if self.compile not in (None, "default", "max-autotune", "reduce-overhead"):
            raise ValueError(f"unknown compile mode {self.compile!r}")
        if self.parallel not in PARALLEL:
            raise ValueError(f"unknown parallel {self.parallel!r}")
        if self.parallel != "none" and self.compile == "reduce-overhead":
            raise ValueError("compile=reduce-overhead (CUDA graphs of the compiled module) is single-GPU only")
        if self.cuda_graph and self.parallel not in ("none", "ddp"):
            raise ValueError("cuda_graph replays the micro-batch on one GPU or under ddp (whose gradient all-reduce kernels "
                             "are part of the captured graph); fsdp / tp run eagerly")
        if self.fsdp_param_dtype not in ("fp32", "fp16", "bf16"):
            raise ValueError(f"unknown fsdp_param_dtype {self.fsdp_param_dtype!r}")
        if self.fsdp_compile_blocks and (self.parallel != "fsdp" or self.compile is not None):
            raise ValueError("fsdp_compile_blocks needs parallel=fsdp and compile unset")
        if self.comm not in ("auto", "fused", "nccl"):
            raise ValueError(f"unknown comm {self.comm!r}")
        if self.residual_dtype not in ("fp32", "bf16"):
            raise ValueError(f"unknown residual_dtype {self.residual_dtype!r}")
        if self.parallel == "fsdp_tp" and not self.tp_size:
            raise ValueError("parallel=fsdp_tp needs tp_size")

    def inert_settings(self, model_uses_sm100: bool = True) -> list[str]:
        """Settings of the reference's schema that are accepted (its YAML files load unchanged) but change nothing here, each with
        the reason; the trainer logs them once at start so that a run never silently differs from what its config says."""
        notes = []
        if self.ddp_grad_as_bucket_view:
            notes.append("ddp_grad_as_bucket_view: gradients are ALWAYS views of the flat bucket buffer here (parallel/flat.py)")
        if self.fsdp_compile_blocks:
            notes.append("fsdp_compile_blocks: blocks run hand-written kernels, there is nothing for a per-block compiler to fuse")
        if self.fp8_recipe != "mxfp8" and self.precision == "fp8":
            notes.append(f"fp8_recipe={self.fp8_recipe}: every recipe maps to MXFP8 block scaling (no amax history is kept)")
        if self.compile in ("default", "max-autotune") and model_uses_sm100:
            notes.append(f"compile={self.compile}: skipped on the sm100 kernel path (the step is already a fixed kernel sequence); "
                         "use cuda_graph / compile=reduce-overhead to remove launch gaps")
        return notes

    @property
    def checkpointing(self) -> bool:
        return bool(self.ckpt_every or self.stop_after_min or self.max_steps or self.resume_from)

    def grad_accum(self, world_size: int = 1) -> int:
        per_micro = self.micro_batch * self.seq_len * world_size
        if self.global_batch_tokens % per_micro:
            raise ValueError(f"global_batch_tokens {self.global_batch_tokens} is not a multiple of {per_micro}")
        return self.global_batch_tokens // per_micro

    @property
    def total_steps(self) -> int:
        return self.total_tokens // self.global_batch_tokens

    @property
    def warmup_steps(self) -> int:
        return max(1, round(self.warmup_frac * self.total_steps))


def _build(cls, values: dict):
    known = {f.name for f in fields(cls)}
    bad = set(values) - known
    if bad:
        raise ValueError(f"unknown {cls.__name__} keys: {sorted(bad)}")
    return cls(**values)


def load_config(path: str | Path) -> tuple[ModelConfig, TrainConfig]:
    raw = yaml.safe_load(Path(path).read_text()) or {}
    unknown = set(raw) - {"model", "train"}
    if unknown:
        raise ValueError(f"unknown config sections: {sorted(unknown)}")
    return _build(ModelConfig, raw.get("model") or {}), _build(TrainConfig, raw.get("train") or {})


def dump_config(model_cfg: ModelConfig, train_cfg: TrainConfig) -> str:
    return yaml.safe_dump({"model": asdict(model_cfg), "train": asdict(train_cfg)}, sort_keys=False)


def apply_overrides(model_cfg: ModelConfig, train_cfg: TrainConfig, overrides: list[str]):
    """``section.key=value`` overrides with YAML-parsed values (the CLIs' ``--set``)."""
    updates = {"model": {}, "train": {}}
    for item in overrides:
        target, eq, raw = item.partition("=")
        section, _, key = target.partition(".")
        if section not in updates or not key or not eq:
            raise ValueError(f"bad override {item!r}: expected model.key=value or train.key=value")
        cfg = model_cfg if section == "model" else train_cfg
        if key not in {f.name for f in fields(cfg)}:
            raise ValueError(f"unknown {section} key {key!r}")
        updates[section][key] = yaml.safe_load(raw)
    # one replace per section: keys that are only valid together (parallel=fsdp_tp + tp_size) may come in any order
    if updates["model"]:
        model_cfg = replace(model_cfg, **updates["model"])
    if updates["train"]:
        train_cfg = replace(train_cfg, **updates["train"])
    return model_cfg, train_cfg
