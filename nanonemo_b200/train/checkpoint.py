"""Checkpoints on torch.distributed.checkpoint (DCP): asynchronous, resumable on another layout.

On-disk layout (same as the reference, nanonemo/train/checkpoint.py:1-80):
    <root>/step_000123/            DCP files holding {"model": ..., "optim": ...}
    <root>/step_000123/trainer.json  step, loader position, loss scale, world sizes (rank 0)
    <root>/latest                  name of the newest COMPLETE checkpoint
``latest`` is written only after every rank's files are on disk (a barrier follows the save), so a
save that was interrupted is never resumed from; the two newest checkpoints are kept.

Every strategy exposes its state through ``strategy.state_for_checkpoint(opt)`` as parameter names
-> FULL tensors (sharded layouts gather their shards for the save; DCP writes a replicated tensor
once), so a checkpoint written under one layout (say FSDP on 8 ranks) loads under any other (DDP on
2, a single process, the HF exporter): each layout slices what it owns on load.
"""

import json
import shutil
from concurrent.futures import Future
from pathlib import Path

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp


def _as_strategy(obj):
    if hasattr(obj, "state_for_checkpoint"):
        return obj
    from nanonemo_b200.parallel.strategy import LocalStrategy

    return LocalStrategy(obj)  # a bare module


def _state(obj, opt) -> dict:
    return _as_strategy(obj).state_for_checkpoint(opt)


def _restore(obj, opt, state) -> None:
    _as_strategy(obj).load_from_checkpoint(opt, state)


class Checkpointer:
    def __init__(self, root, main: bool, keep: int = 2, use_async: bool = True):
        self.root, self.main, self.keep, self.use_async = Path(root), main, keep, use_async
        self._pending: tuple[Future, Path, dict] | None = None

    def save(self, step: int, obj, opt, trainer_state: dict) -> None:
        """`obj` is a Strategy or a bare module. One save in flight at a time."""
        self.wait()
        path = self.root / f"step_{step:06d}"
        state = _state(obj, opt)
        if self.use_async:
            self._pending = (dcp.async_save(state, checkpoint_id=str(path)), path, trainer_state)
        else:
            dcp.save(state, checkpoint_id=str(path))
            self._finish(path, trainer_state)

    def wait(self) -> None:
        if self._pending:
            future, path, trainer_state = self._pending
            future.result()
            self._pending = None
            self._finish(path, trainer_state)

    def _finish(self, path: Path, trainer_state: dict) -> None:
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        if not self.main:
            return
        (path / "trainer.json").write_text(json.dumps(trainer_state))
        tmp = self.root / "latest.tmp"
        tmp.write_text(path.name)
        tmp.replace(self.root / "latest")
        done = sorted(p for p in self.root.glob("step_*") if p.is_dir() and (p / "trainer.json").exists())
        for old in done[:-self.keep]:
            shutil.rmtree(old, ignore_errors=True)


def find_latest(root) -> Path | None:
    """`root` itself if it is a checkpoint, else the one its ``latest`` file names, else None."""
    root = Path(root)
    if (root / "trainer.json").exists():
        return root
    pointer = root / "latest"
    if pointer.exists():
        cand = root / pointer.read_text().strip()
        return cand if (cand / "trainer.json").exists() else None
    return None


def load(path, obj, opt) -> dict:
    """Load model + optimizer in place (resharding to the current layout); returns trainer.json."""
    path = Path(path)
    state = _state(obj, opt)
    dcp.load(state, checkpoint_id=str(path))
    _restore(obj, opt, state)
    return json.loads((path / "trainer.json").read_text())
