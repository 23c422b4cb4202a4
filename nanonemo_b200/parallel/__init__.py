"""Process-group bootstrap and the cold-path collectives.

One process per GPU, started by ``torch.distributed.run``. ``init()`` turns the launcher's environment into a
``Dist`` record and joins ONE process group whose backend follows the device: NCCL for CUDA tensors with gloo beside
it for CPU tensors (the asynchronous checkpoint writer stages on the host), or gloo alone when ``NANONEMO_DEVICE=cpu``
so that every multi-rank path can be exercised on a machine without GPUs. A process that was not started by a launcher
gets a single-rank ``Dist`` and no group. The hot-path collectives do not pass through here: they are kernels over
symmetric memory (``parallel/symm.py``). Same surface as the reference module (nanonemo/distributed/__init__.py:16-70)
plus an optional group timeout and ``all_max``.
"""

import datetime
import os

import torch
import torch.distributed as dist

_BACKENDS = {"cuda": "cuda:nccl,cpu:gloo", "cpu": "gloo"}
_LAUNCH_VARS = ("RANK", "WORLD_SIZE", "LOCAL_RANK")


class Dist:
    """Where this process sits in the job: global rank, world size, rank on this node, and its device string."""

    __slots__ = ("rank", "world", "local_rank", "device")

    def __init__(self, rank: int = 0, world: int = 1, local_rank: int = 0, device: str = "cuda"):
        self.rank, self.world, self.local_rank, self.device = rank, world, local_rank, device

    @property
    def main(self) -> bool:
        """The one rank that writes logs, configs and checkpoint pointers."""
        return self.rank == 0

    @property
    def enabled(self) -> bool:
        """True once a process group exists (several ranks, or one rank started by a launcher)."""
        return _group_up()

    def __repr__(self) -> str:
        return f"Dist(rank={self.rank}, world={self.world}, local_rank={self.local_rank}, device={self.device!r})"

    def __eq__(self, other) -> bool:
        return isinstance(other, Dist) and all(getattr(self, k) == getattr(other, k) for k in self.__slots__)


def _group_up() -> bool:
    return dist.is_available() and dist.is_initialized()


def _device_kind() -> str:
    forced = os.environ.get("NANONEMO_DEVICE")
    if forced:
        return forced
    return "cuda" if torch.cuda.is_available() else "cpu"


def _group_timeout(timeout_s: float | None):
    if timeout_s is None:
        env = os.environ.get("NANONEMO_PG_TIMEOUT_S")
        timeout_s = float(env) if env else None
    return None if timeout_s is None else datetime.timedelta(seconds=timeout_s)


def init(timeout_s: float | None = None) -> Dist:
    """Join the job's process group (idempotent). ``timeout_s`` (or NANONEMO_PG_TIMEOUT_S) bounds every collective
    of the group, which is how a rank that never shows up becomes an error on the others instead of a hang."""
    kind = _device_kind()
    if any(v not in os.environ for v in _LAUNCH_VARS):
        return Dist(device=kind)
    rank, world, local = (int(os.environ[v]) for v in _LAUNCH_VARS)
    me = Dist(rank, world, local, f"cuda:{local}" if kind == "cuda" else "cpu")
    if _group_up():
        return me
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    options = {}
    limit = _group_timeout(timeout_s)
    if limit is not None:
        options["timeout"] = limit
    if kind == "cuda":
        torch.cuda.set_device(local)
        options["device_id"] = torch.device(me.device)
    dist.init_process_group(_BACKENDS["cuda" if kind == "cuda" else "cpu"], **options)
    return me


def destroy() -> None:
    if _group_up():
        dist.destroy_process_group()


def _reduced(x: torch.Tensor, op, group=None) -> torch.Tensor:
    """Out-of-place all-reduce; the input itself when there is no group."""
    if not _group_up():
        return x
    out = x.clone()
    dist.all_reduce(out, op=op, group=group)
    return out


def all_mean(x: torch.Tensor, group=None) -> torch.Tensor:
    """Mean over the ranks of `group` (identity in a single process)."""
    if not _group_up():
        return x
    return _reduced(x, dist.ReduceOp.SUM, group) / dist.get_world_size(group)


def all_max(values: torch.Tensor) -> torch.Tensor:
    """Element-wise max over ranks: benchmark timings are reported as the slowest rank's."""
    return _reduced(values, dist.ReduceOp.MAX)


def any_rank(flag: bool, device: str) -> bool:
    """True on every rank as soon as `flag` is true on one of them, so that all ranks take the same branch
    (stop on the time limit, save a checkpoint)."""
    if not _group_up():
        return bool(flag)
    votes = torch.tensor([1.0 if flag else 0.0], device=device)
    return _reduced(votes, dist.ReduceOp.MAX).item() > 0.0
