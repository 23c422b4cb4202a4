"""Execution strategies: how one model replica is laid out over the ranks and how its gradients
become an optimizer update.

The trainer talks to a ``Strategy`` only: ``sync_ctx(last)`` around each micro-batch, and
``step(opt, grad_clip, scaler)`` which finishes the gradient collectives, clips by the global norm,
applies the update and clears the gradients, returning the pre-clip norm as a device scalar.
``LocalStrategy`` is the single-process case; ddp.py / fsdp.py / tp.py derive from it. This plays
the role of the reference's ``Setup`` record (nanonemo/train/trainer.py:62-75) with the reduction,
clipping and update folded in, because on the flat fused path those are one or two kernels.
"""

from contextlib import nullcontext

import torch
from torch import nn


class LocalStrategy:
    name = "none"
    sharded_grads = False

    def __init__(self, model: nn.Module, store=None, step_model: nn.Module | None = None):
        self.model = model
        self.step_model = step_model if step_model is not None else model  # (a compiled module has no truth value)
        self.store = store
        self.dp_rank, self.dp_world = 0, 1
        self.loss_ctx = nullcontext
        self.fwd_ctx = nullcontext
        self.launches = 0  # kernels of this framework launched by the strategy itself (comm + update)

    # -- per micro-batch
    def sync_ctx(self, last: bool):
        return nullcontext()

    def graphed_micro_step(self, x, y, amp_dtype, accum: int, last: bool = True):
        """Forward + backward of one micro-batch replayed from a CUDA graph: the whole micro-batch becomes one launch,
        which removes the host's enqueue time and most of the gaps between dependent kernels (the reference's
        ``compile: reduce-overhead`` stage). Under data parallelism the gradient all-reduce kernels of the last
        micro-batch, launched on the side stream by the gradient-ready hooks, are captured with it and the side stream
        is joined inside the captured region. The first calls of a (shape, last) pair run eagerly (warm-up), the next
        one is captured, later ones copy the batch into the static input buffers and replay. Gradients accumulate into
        the flat gradient buffer as usual."""
        from nanonemo_b200.ops import _lib

        graphs = self.__dict__.setdefault("_graphs", {})
        st = graphs.setdefault((tuple(x.shape), amp_dtype, accum, bool(last)), {"calls": 0})

        def run(a, b):
            with self.sync_ctx(last), self.loss_ctx():
                with torch.autocast("cuda", dtype=amp_dtype, enabled=amp_dtype is not None), self.fwd_ctx():
                    _, loss = self.step_model(a, b)
                loss = loss / accum
                loss.backward()
            if last:
                self.finish_grads()  # joins the collectives' stream: part of the graph when capturing
            return loss.detach()

        if "graph" in st:
            st["x"].copy_(x)
            st["y"].copy_(y)
            st["graph"].replay()
            _lib.LAUNCHES += st["launches"]  # the captured kernels run again without passing through the launch counter
            self.launches += st["own_launches"]
            if last:
                self.after_graph_replay()
            return st["loss"]
        st["calls"] += 1
        if st["calls"] <= 2:  # eager warm-up: allocator, kernel attributes, status buffers
            return run(x, y)
        st["x"], st["y"] = x.clone(), y.clone()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0, own0 = _lib.LAUNCHES, self.launches
        try:
            with torch.cuda.graph(graph):
                st["loss"] = run(st["x"], st["y"])
        except Exception as e:  # noqa: BLE001 - capture records without executing, so nothing was computed yet: run eagerly from now on
            import warnings

            warnings.warn(f"CUDA-graph capture of the micro-batch failed ({type(e).__name__}: {str(e)[:200]}); continuing without graphs")
            torch.cuda.synchronize()
            self.use_cuda_graph = False
            graphs.clear()
            return run(x, y)
        st["launches"], st["own_launches"] = _lib.LAUNCHES - n0, self.launches - own0
        st["graph"] = graph
        graph.replay()  # capturing records the work without running it: run this micro-batch now
        if last:
            self.after_graph_replay()
        return st["loss"]

    def after_graph_replay(self):
        """Host-side bookkeeping that the hooks would have done had the micro-batch run eagerly."""

    def status_words(self) -> list:
        """Device int32 tensors whose FIRST element turns non-zero when a kernel launched on behalf of this strategy gave
        up on a bounded wait (tensor-core pipelines: ops.gemm.status_tensor; collectives: the communicators' status)."""
        if self.store is None or self.store.device.type != "cuda":
            return []
        from nanonemo_b200.ops import _lib
        from nanonemo_b200.ops.gemm import status_tensor

        return [status_tensor(self.store.device)] if _lib.available() else []

    def status_flag(self):
        """0-dim float tensor, non-zero when any status word is set; None when there is nothing to watch. The trainer
        stacks it with the loss so that it travels in the step's one device -> host copy."""
        words = self.status_words()
        if not words:
            return None
        return torch.stack([w[0] for w in words]).ne(0).sum().float()

    def raise_on_status(self):
        """Called once the host has seen a non-zero status flag: raises with the details the kernels recorded."""
        from nanonemo_b200.ops.gemm import check_status

        for obj in self.status_owners():
            obj.check_status()
        check_status()
        raise RuntimeError("a kernel reported a bounded wait that ran out (status flag set)")

    def status_owners(self) -> list:
        return []

    def full_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss

    # -- per optimizer step
    def begin_step(self, opt, grad_clip) -> None:
        """Called before the first micro-batch of an optimizer step (a layout may plan its collectives around the update)."""

    def finish_grads(self):
        """Block the compute stream until every gradient collective of this step has landed."""

    def global_sumsq(self) -> torch.Tensor:
        return self.store.grad_sumsq()

    def parameters_for_clip(self):
        return self.model.parameters()

    def step(self, opt: torch.optim.Optimizer, grad_clip: float, scaler=None, keep_grads: bool = False):
        self.finish_grads()
        store = self.store
        if store is None:
            if scaler:
                scaler.unscale_(opt)
            norm = torch.nn.utils.clip_grad_norm_(self.parameters_for_clip(), grad_clip if grad_clip and grad_clip > 0 else float("inf"))
            if hasattr(norm, "full_tensor"):
                norm = norm.full_tensor()
            if scaler:
                scaler.step(opt)
                scaler.update()
            else:
                opt.step()
            opt.zero_grad(set_to_none=not keep_grads)
            return norm
        if scaler:
            scaler.unscale_(opt)
        sumsq = self.global_sumsq()
        norm = sumsq.sqrt()
        clip = grad_clip if grad_clip is not None and grad_clip > 0 else None  # <= 0 / None: the norm is only reported
        if store.fused_ok and scaler is None and hasattr(opt, "store"):
            opt.step(grad_norm_sq=sumsq if clip is not None else None, max_norm=clip)  # clips, updates, refreshes the shadow, zeroes grads
            return norm
        if clip is not None:
            self.scale_grads_((clip / (norm + 1e-6)).clamp(max=1.0))
        if scaler:
            scaler.step(opt)
            scaler.update()
        else:
            opt.step()
        store.zero_grad()
        store.refresh_shadow()
        return norm

    def scale_grads_(self, coef: torch.Tensor):
        self.store.grad.mul_(coef.to(self.store.grad.dtype))

    # -- checkpoint state, streamed: one full fp32 tensor at a time under this framework's parameter names.
    # train/checkpoint.py turns the stream into the on-disk key set and keeps only this rank's row block of every tensor, so
    # no rank ever holds more than one full tensor beyond its 1 / world share. Every rank walks the stream in the same
    # order (sharded layouts issue a collective per tensor or per unit).
    STATE_KINDS = ("model", "exp_avg", "exp_avg_sq")

    def checkpoint_names(self) -> list:
        """[(name, full shape)] of every parameter, the tied weight once, in the order the streams use."""
        return [(n, tuple(p.shape)) for n, p in self.model.named_parameters()]

    def checkpoint_tensors(self, opt, kind: str):
        """Yields (name, full tensor) for kind in STATE_KINDS; a moment that does not exist yet is zeros."""
        for n, p in self.model.named_parameters():
            if kind == "model":
                yield n, p.detach()
            else:
                st = opt.state.get(p, {}) if opt is not None else {}
                yield n, st[kind].detach() if kind in st else torch.zeros_like(p)

    def restore_tensor(self, opt, kind: str, name: str, full: torch.Tensor) -> None:
        p = self._params_by_name()[name]
        with torch.no_grad():
            if kind == "model":
                p.copy_(full)
                return
            st = opt.state[p]
            if "exp_avg" not in st:
                st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(p), torch.zeros_like(p)
                st["step"] = torch.tensor(0.0, dtype=torch.float32)
            st[kind].copy_(full)

    def _params_by_name(self) -> dict:
        cache = self.__dict__.get("_by_name")
        if cache is None:
            cache = self.__dict__["_by_name"] = dict(self.model.named_parameters())
        return cache

    def optimizer_step_count(self, opt) -> int:
        for st in (opt.state.values() if opt is not None else ()):
            if "step" in st:
                return int(float(st["step"]))
        return 0

    def finish_restore(self, opt, step_count: int) -> None:
        """After every tensor has been restored: set the optimizer's step counter and refresh whatever is derived from
        the weights (the 16-bit shadow, the views of the flat buffers)."""
        if opt is not None:
            if hasattr(opt, "set_step_count"):
                opt.set_step_count(step_count)
            else:
                for st in opt.state.values():
                    if "step" in st:
                        st["step"] = torch.tensor(float(step_count), dtype=torch.float32)
        if self.store is not None:
            self.store.rebind_grads()
            self.store.refresh_shadow()
