"""AdamW with decay / no-decay parameter groups, the warmup + cosine LR schedule, and the fused
flat-buffer AdamW used on the sm100 path.

Grouping rule and schedule follow the reference (nanonemo/train/optim.py:9-43): weight decay on
tensors with dim >= 2 except the (tied) token embedding; linear warmup from peak/warmup then cosine
to ``min_ratio * peak``, clamped past the end; betas (0.9, 0.95), eps 1e-8.
"""

import math

import torch
from torch import nn


def param_groups(model: nn.Module, weight_decay: float) -> list[dict]:
    decay, no_decay = [], []
    for name, p in model.named_parameters():  # yields the tied embedding/lm_head weight once
        if not p.requires_grad:
            continue
        (decay if p.dim() >= 2 and "tok_emb" not in name else no_decay).append(p)
    return [{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}]


class FusedAdamW(torch.optim.AdamW):
    """torch.optim.AdamW whose ``step`` runs as ONE kernel when the parameters live in a
    ``FlatParams`` store on a CUDA device.

    The fused kernel (csrc/adamw.cu) reads the fp32 gradient, applies the global-norm clip
    coefficient computed on the device (no host sync), updates the fp32 master weight and both
    moments, writes the bf16 compute copy of the weight, and zeroes the gradient — one pass over
    memory instead of the dozen foreach launches of the stock optimizer. The per-parameter state
    tensors (``exp_avg``, ``exp_avg_sq``, ``step``) are views into the flat moment buffers, so
    ``state_dict()`` and torch DCP see an ordinary AdamW. Off the GPU it is the stock optimizer.
    """

    def __init__(self, params, lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, store=None):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, fused=False)
        self.store = store
        self._n_steps = 0
        if store is not None:
            store.attach_optimizer(self)
            if store.fused_ok:
                self.set_step_count(0)

    def set_step_count(self, n: int) -> None:
        """Every parameter's ``step`` entry becomes ONE shared CPU scalar on the fused path (the kernel updates all
        parameters in the same launch, so there is one counter to advance per step, not one per parameter)."""
        self._n_steps = int(n)
        if self.store is not None and self.store.fused_ok:
            shared = torch.tensor(float(n), dtype=torch.float32)
            for st in self.state.values():
                st["step"] = shared
            self._shared_step = shared
        else:
            for st in self.state.values():
                st["step"] = torch.tensor(float(n), dtype=torch.float32)

    @torch.no_grad()
    def step(self, closure=None, grad_norm_sq: torch.Tensor | None = None, max_norm: float | None = None):
        """`grad_norm_sq` (device scalar) and `max_norm` let the fused path clip inside the update."""
        store = self.store
        if store is None or not store.fused_ok:
            assert grad_norm_sq is None, "clip-in-update needs the flat fused path"
            return super().step(closure)
        shared = getattr(self, "_shared_step", None)
        first = next(iter(self.state.values()))["step"] if self.state else None
        if shared is None or first is not shared:  # state was replaced from outside (load_state_dict): re-share it
            self.set_step_count(int(float(first)) if first is not None else 0)
            shared = self._shared_step
        self._n_steps = int(float(shared)) + 1
        store.fused_adamw_step(self, self._n_steps, grad_norm_sq, max_norm)
        shared.fill_(self._n_steps)
        return None


def build_optimizer(model: nn.Module, lr: float, weight_decay: float = 0.1, betas=(0.9, 0.95), eps: float = 1e-8,
                    fused: bool = False, store=None) -> torch.optim.AdamW:
    groups = param_groups(model, weight_decay)
    if store is not None:
        return FusedAdamW(groups, lr=lr, betas=betas, eps=eps, store=store)
    return torch.optim.AdamW(groups, lr=lr, betas=betas, eps=eps, fused=fused)


def lr_at(step: int, peak_lr: float, total_steps: int, warmup_steps: int, min_ratio: float = 0.1) -> float:
    """Linear warmup to peak_lr (step 0 already non-zero), then cosine to min_ratio * peak_lr at the last step."""
    if step < warmup_steps:
        return peak_lr * (step + 1) / warmup_steps
    progress = min((step - warmup_steps) / max(1, total_steps - 1 - warmup_steps), 1.0)
    return peak_lr * (min_ratio + (1.0 - min_ratio) * 0.5 * (1.0 + math.cos(math.pi * progress)))
