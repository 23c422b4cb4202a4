"""Checkpoints on torch.distributed.checkpoint (DCP): asynchronous, sharded, resumable on another layout, and
interchangeable with the reference's.

On-disk layout (nanonemo/train/checkpoint.py:1-80):
    <root>/step_000123/              DCP files holding {"model": ..., "optim": ...}
    <root>/step_000123/trainer.json  step, loader position, loss scale, world sizes (rank 0)
    <root>/latest                    name of the newest COMPLETE checkpoint
``latest`` is written only after every rank's files are on disk (a barrier follows the save), so a save that was
interrupted is never resumed from; the two newest checkpoints are kept.

Keys are the ones ``get_state_dict(model, opt)`` gives the reference: ``model.<fqn>`` with the per-projection names
``attn.wq / wk / wv`` and ``mlp.w_gate / w_up`` (this framework's fused ``wqkv`` and ``w_gu`` are split on save and
joined on load), ``model.lm_head.weight`` beside the tied ``model.tok_emb.weight``, ``optim.state.<fqn>.exp_avg /
exp_avg_sq / step`` and ``optim.param_groups``. A checkpoint of the reference (its released model included) therefore
resumes here and the other way round.

Who writes what: every tensor is cut into ``world`` blocks of rows and rank r keeps block r, wrapped as a DTensor
``Shard(0)`` over a 1-D mesh of all ranks, so DCP writes one chunk per rank in parallel and can reshard on load.
Strategies hand their state over as a STREAM of full tensors (``strategy.checkpoint_tensors``: a sharded layout
all-gathers one unit at a time into a transient buffer), and only the row block is kept: a save costs each rank
``state / world`` of extra memory plus one transient unit, whatever the layout. Loading runs the other way: DCP fills
row-block targets (from any layout, the reference's FSDP2 shards included), each tensor is re-assembled transiently and
passed to ``strategy.restore_tensor``, which keeps what the rank owns.
"""

import json
import shutil
from concurrent.futures import Future
from pathlib import Path

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

KINDS = ("model", "exp_avg", "exp_avg_sq")


def _as_strategy(obj):
    if hasattr(obj, "checkpoint_tensors"):
        return obj
    from nanonemo_b200.parallel.strategy import LocalStrategy

    return LocalStrategy(obj)  # a bare module


# ----------------------------------------------------------------------------- names: fused parameters <-> reference keys
def reference_pieces(name: str, shape: tuple, cfg) -> list[tuple[str, int, int]]:
    """[(reference name, first row, one-past-last row)] of the on-disk tensors that parameter `name` is stored as."""
    rows = shape[0]
    if name.endswith("attn.wqkv.weight"):
        q, kv = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        stem = name[: -len("wqkv.weight")]
        return [(stem + "wq.weight", 0, q), (stem + "wk.weight", q, q + kv), (stem + "wv.weight", q + kv, q + 2 * kv)]
    if name.endswith("mlp.w_gu.weight"):
        stem = name[: -len("w_gu.weight")]
        return [(stem + "w_gate.weight", 0, rows // 2), (stem + "w_up.weight", rows // 2, rows)]
    return [(name, 0, rows)]


def _world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


_MESHES: dict = {}


def _mesh(device_type: str):
    """1-D mesh over every rank of the job (cached): the sharding that the row blocks are declared under."""
    key = (device_type, dist.get_world_size())
    if key not in _MESHES:
        from torch.distributed.device_mesh import init_device_mesh

        _MESHES[key] = init_device_mesh(device_type, (dist.get_world_size(),))
    return _MESHES[key]


def _row_block(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of rank `rank` when `rows` rows are cut the way ``Shard(0)`` cuts them (ceil-sized blocks, last ones short)."""
    per = -(-rows // world)
    return min(rank * per, rows), min((rank + 1) * per, rows)


def _shard0(block: torch.Tensor, full_shape: tuple):
    """This rank's row block of a tensor of `full_shape` as a DTensor (a plain tensor without a process group)."""
    rank, world = _world()
    if world == 1:
        return block
    from torch.distributed.tensor import DTensor, Shard

    stride = [1] * len(full_shape)
    for i in range(len(full_shape) - 2, -1, -1):
        stride[i] = stride[i + 1] * full_shape[i + 1]
    return DTensor.from_local(block, _mesh(block.device.type), [Shard(0)], run_check=False, shape=torch.Size(full_shape),
                              stride=tuple(stride))


def _full(entry) -> torch.Tensor:
    return entry.full_tensor() if hasattr(entry, "full_tensor") else entry


def _param_groups(strategy, opt, cfg) -> list[dict]:
    """``param_groups`` in the form ``get_state_dict`` gives them: hyper-parameters plus the member parameters' names."""
    names = {}
    for n, shape in strategy.checkpoint_names():
        names[n] = [ref for ref, _, _ in reference_pieces(n, shape, cfg)]
    by_param = {id(p): n for n, p in strategy.model.named_parameters()}
    groups = []
    for g in opt.param_groups:
        entry = {k: v for k, v in g.items() if k != "params"}
        entry["params"] = [ref for p in g["params"] if id(p) in by_param for ref in names.get(by_param[id(p)], [])]
        groups.append(entry)
    return groups


# ----------------------------------------------------------------------------- save
def collect_state(obj, opt) -> dict:
    """The DCP state dict of this rank: its row block of every tensor, under the reference's keys."""
    strategy = _as_strategy(obj)
    cfg = strategy.model.cfg
    rank, world = _world()
    shapes = dict(strategy.checkpoint_names())
    model, opt_state = {}, {}
    step = torch.tensor(float(strategy.optimizer_step_count(opt)), dtype=torch.float32)
    for kind in KINDS if opt is not None else KINDS[:1]:
        for name, full in strategy.checkpoint_tensors(opt, kind):
            for ref, r0, r1 in reference_pieces(name, shapes[name], cfg):
                piece_shape = (r1 - r0, *shapes[name][1:])
                b0, b1 = _row_block(r1 - r0, rank, world)
                block = full[r0 + b0:r0 + b1].detach().clone()  # the only part of `full` that outlives this iteration
                entry = _shard0(block, piece_shape)
                if kind == "model":
                    model[ref] = entry
                    if ref == "tok_emb.weight":
                        model["lm_head.weight"] = entry  # the tied head appears under both names, as in the reference
                else:
                    opt_state.setdefault(ref, {"step": step.clone()})[kind] = entry
    state = {"model": model}
    if opt is not None:
        state["optim"] = {"state": opt_state, "param_groups": _param_groups(strategy, opt, cfg)}
    return state


class Checkpointer:
    def __init__(self, root, main: bool, keep: int = 2, use_async: bool = True):
        self.root, self.main, self.keep, self.use_async = Path(root), main, keep, use_async
        self._pending: tuple[Future, Path, dict] | None = None

    def save(self, step: int, obj, opt, trainer_state: dict) -> None:
        """`obj` is a Strategy or a bare module. One save in flight at a time."""
        self.wait()
        path = self.root / f"step_{step:06d}"
        state = collect_state(obj, opt)
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


# ----------------------------------------------------------------------------- load
def restore_state(path, obj, opt, device=None) -> None:
    """Read a checkpoint (this framework's or the reference's, written under any layout) into `obj` / `opt`. One kind
    (weights, first moments, second moments) at a time, so the targets are 1 / world of ONE copy of the model."""
    strategy = _as_strategy(obj)
    cfg = strategy.model.cfg
    rank, world = _world()
    device = torch.device(device) if device is not None else next(strategy.model.parameters()).device
    names = strategy.checkpoint_names()
    step_count = 0
    for kind in KINDS if opt is not None else KINDS[:1]:
        targets, layout = {}, []
        for name, shape in names:
            for ref, r0, r1 in reference_pieces(name, shape, cfg):
                piece_shape = (r1 - r0, *shape[1:])
                b0, b1 = _row_block(r1 - r0, rank, world)
                targets[ref] = _shard0(torch.zeros((b1 - b0, *shape[1:]), dtype=torch.float32, device=device), piece_shape)
                layout.append((name, ref))
        if kind == "model":
            request = {"model": targets}
        else:
            request = {"optim": {"state": {ref: {kind: t} for ref, t in targets.items()}}}
            if kind == KINDS[1]:  # the step counter rides with the first moments (one scalar per parameter, all equal)
                first = layout[0][1]
                request["optim"]["state"][first]["step"] = torch.zeros((), dtype=torch.float32)
        dcp.load(request, checkpoint_id=str(path))
        if kind == KINDS[1]:
            step_count = int(float(request["optim"]["state"][layout[0][1]]["step"]))
        refs_of: dict = {}
        for name, ref in layout:
            refs_of.setdefault(name, []).append(ref)
        for name, _ in names:  # stream order: a sharded layout completes one unit after the other
            parts = [_full(targets.pop(ref)) for ref in refs_of[name]]  # re-assembled transiently, one parameter at a time
            strategy.restore_tensor(opt, kind, name, parts[0] if len(parts) == 1 else torch.cat(parts, dim=0))
    strategy.finish_restore(opt, step_count)


def load(path, obj, opt) -> dict:
    """Load model + optimizer in place (resharding to the current layout); returns trainer.json."""
    path = Path(path)
    restore_state(path, obj, opt)
    return json.loads((path / "trainer.json").read_text())
