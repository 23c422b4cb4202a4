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
        self.step_model = step_model or model
        self.store = store
        self.dp_rank, self.dp_world = 0, 1
        self.loss_ctx = nullcontext
        self.fwd_ctx = nullcontext
        self.launches = 0  # kernels of this framework launched by the strategy itself (comm + update)

    # -- per micro-batch
    def sync_ctx(self, last: bool):
        return nullcontext()

    def full_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss

    # -- per optimizer step
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
            norm = torch.nn.utils.clip_grad_norm_(self.parameters_for_clip(), grad_clip)
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
        if store.fused_ok and scaler is None and hasattr(opt, "store"):
            opt.step(grad_norm_sq=sumsq, max_norm=grad_clip)  # clips, updates, refreshes the shadow, zeroes grads
            return norm
        self.scale_grads_((grad_clip / (norm + 1e-6)).clamp(max=1.0))
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
