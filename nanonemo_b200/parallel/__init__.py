"""Process-group bootstrap and the cold-path collectives.

One process per GPU, launched by torchrun: ``init()`` reads RANK / WORLD_SIZE / LOCAL_RANK and joins
one group — NCCL for CUDA tensors plus gloo for CPU tensors (the asynchronous checkpoint writer
stages on the CPU), or gloo alone when ``NANONEMO_DEVICE=cpu`` so the multi-rank paths can be tested
on a machine without GPUs (behaviour of nanonemo/distributed/__init__.py:16-70). The hot-path
collectives do not go through here: they are kernels over symmetric memory (parallel/symm.py).
"""

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Dist:
    rank: int = 0
    world: int = 1
    local_rank: int = 0
    device: str = "cuda"

    @property
    def main(self) -> bool:
        return self.rank == 0

    @property
    def enabled(self) -> bool:
        return dist.is_available() and dist.is_initialized()


def init(timeout_s: float | None = None) -> Dist:
    kind = os.environ.get("NANONEMO_DEVICE") or ("cuda" if torch.cuda.is_available() else "cpu")
    if "RANK" not in os.environ:
        return Dist(device=kind)
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    device = f"cuda:{local}" if kind == "cuda" else "cpu"
    if dist.is_initialized():
        return Dist(rank, world, local, device)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    kw = {}
    if timeout_s is None and os.environ.get("NANONEMO_PG_TIMEOUT_S"):
        timeout_s = float(os.environ["NANONEMO_PG_TIMEOUT_S"])
    if timeout_s is not None:
        kw["timeout"] = datetime.timedelta(seconds=timeout_s)
    if kind == "cuda":
        torch.cuda.set_device(local)
        dist.init_process_group("cuda:nccl,cpu:gloo", device_id=torch.device(device), **kw)
    else:
        dist.init_process_group("gloo", **kw)
    return Dist(rank, world, local, device)


def destroy() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def all_mean(x: torch.Tensor, group=None) -> torch.Tensor:
    """Mean over ranks (identity in a single process)."""
    if dist.is_available() and dist.is_initialized():
        x = x.clone()
        dist.all_reduce(x, group=group)
        x /= dist.get_world_size(group)
    return x


def any_rank(flag: bool, device: str) -> bool:
    """True if `flag` is true on any rank, so that every rank takes the same branch."""
    if not (dist.is_available() and dist.is_initialized()):
        return flag
    t = torch.tensor(float(flag), device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return bool(t.item())


def all_max(values: torch.Tensor) -> torch.Tensor:
    """Element-wise max over ranks: benchmark timings are reported as the slowest rank's."""
    if dist.is_available() and dist.is_initialized():
        values = values.clone()
        dist.all_reduce(values, op=dist.ReduceOp.MAX)
    return values
