"""Optional Weights & Biases sink for the trainer's records (cf. nanonemo/train/wandb_sink.py:8-47).
wandb is imported only when a project is configured; ``WANDB_MODE=offline`` works without network."""

from dataclasses import asdict

NAMESPACE = {"loss": "train", "lr": "train", "grad_norm": "train", "tokens": "train", "loss_scale": "train",
             "tokens_per_s": "perf", "peak_mem_gb": "perf", "mfu": "perf"}


def to_wandb(record: dict) -> dict:
    """Trainer record -> namespaced metric names; fields W&B has no use for are dropped."""
    out = {f"{NAMESPACE[k]}/{k}": v for k, v in record.items() if k in NAMESPACE}
    if "val_loss" in record:
        out["val/loss"] = record["val_loss"]
    return out


class WandbSink:
    def __init__(self, project, run_name, model_cfg, cfg):
        import wandb

        self.run = wandb.init(project=project, name=run_name, dir=cfg.out_dir,
                              config={"model": asdict(model_cfg), "train": asdict(cfg)})

    def __call__(self, record: dict) -> None:
        if record.get("event") == "start":
            self.run.config.update({k: v for k, v in record.items() if k != "event"}, allow_val_change=True)
        elif (metrics := to_wandb(record)):
            self.run.log(metrics, step=record["step"])

    def close(self) -> None:
        self.run.finish()

    finish = close
