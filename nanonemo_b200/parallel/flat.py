"""Flat parameter store: every parameter, gradient and AdamW moment of a model in four contiguous
fp32 buffers (plus an optional bf16 shadow of the weights for the tensor-core GEMMs).

Why: on B200 the optimizer, the gradient norm, zeroing and the gradient collectives are all
HBM-bandwidth or launch bound. With one flat buffer each of them is a single kernel (or a single
collective per bucket range) instead of ~150 small launches, DDP buckets and FSDP shards are plain
index ranges, and the gradient buffer can live in symmetric memory so peer GPUs reduce it in place
over NVLink. Parameters stay ordinary ``nn.Parameter`` objects: ``p.data`` and ``p.grad`` become
views into the flat buffers, so autograd, ``state_dict`` and torch DCP keep working.

The reference has no such structure (it uses torch DDP's reducer buckets, nanonemo/distributed/
ddp.py:14-16, and foreach AdamW, nanonemo/train/optim.py:33); this is the B200-first replacement.
"""

import torch
from torch import nn

ALIGN = 256  # elements; keeps every view 1 KiB aligned in fp32 (16-byte TMA rule holds for bf16 too)


def _shadow_rewritten() -> None:
    """The 16-bit compute copies of the weights have new values: cached quantised copies of them are stale."""
    from nanonemo_b200 import fp8

    fp8.weights_changed()


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class FlatParams:
    def __init__(self, model: nn.Module, device=None, shadow_dtype: torch.dtype | None = None,
                 grad_alloc=None, pad_to: int = ALIGN):
        """`grad_alloc(numel) -> fp32 tensor` lets the caller place the gradient buffer in symmetric
        memory; `pad_to` pads the total size (e.g. to world * ALIGN so reduce-scatter slices are even)."""
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.names = [n for n, _ in named]
        self.params = [p for _, p in named]
        device = torch.device(device) if device is not None else self.params[0].device
        self.device = device
        if device.type == "cuda":
            from nanonemo_b200.ops import direct

            direct.enable()  # a trainer engine owns this model: weightless operators skip the dispatcher (ops/direct.py)
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += _round_up(p.numel(), ALIGN)
        self.numel = _round_up(off, pad_to)
        self.master = torch.zeros(self.numel, dtype=torch.float32, device=device)
        self.grad = grad_alloc(self.numel) if grad_alloc else torch.zeros(self.numel, dtype=torch.float32, device=device)
        self.grad.zero_()
        self.shadow = torch.zeros(self.numel, dtype=shadow_dtype, device=device) if shadow_dtype else None
        self.exp_avg = self.exp_avg_sq = None
        self.decay_flags = torch.zeros(self.numel // ALIGN, dtype=torch.uint8, device=device)
        self.index = {}
        for name, p, o in zip(self.names, self.params, self.offsets):
            n = p.numel()
            self.master[o:o + n].copy_(p.detach().reshape(-1))
            p.data = self.master[o:o + n].view(p.shape)
            p.grad = self.grad[o:o + n].view(p.shape)
            p._main_grad = p.grad  # where the sm100 backward kernels accumulate directly
            p._flat_store, p._flat_offset = self, o
            if self.shadow is not None:
                p._shadow = self.shadow[o:o + n].view(p.shape)
            self.index[id(p)] = (name, o, n)
        self.shadow_fresh = False
        self.refresh_shadow()

    # ------------------------------------------------------------------ helpers
    @property
    def fused_ok(self) -> bool:
        if self.device.type != "cuda":
            return False
        from nanonemo_b200.ops import _lib

        return _lib.available()

    def range_of(self, p) -> tuple[int, int]:
        _, o, n = self.index[id(p)]
        return o, o + _round_up(n, ALIGN)

    def grad_view(self, p) -> torch.Tensor:
        _, o, n = self.index[id(p)]
        return self.grad[o:o + n].view(p.shape)

    def rebind_grads(self):
        """Point every p.grad back at the flat gradient buffer (after something set it to None)."""
        for p in self.params:
            if p.grad is None or p.grad.data_ptr() != self.grad_view(p).data_ptr():
                p.grad = self.grad_view(p)

    def zero_grad(self):
        self.grad.zero_()
        self.rebind_grads()

    def refresh_shadow(self):
        """Re-derive the low-precision compute copy from the fp32 master weights."""
        if self.shadow is not None:
            self.shadow.copy_(self.master)
            _shadow_rewritten()

    def grad_sumsq(self) -> torch.Tensor:
        """Sum of squared gradient entries as a device scalar (fp32), one pass over the flat buffer."""
        if self.fused_ok:
            from nanonemo_b200.ops.adamw import sumsq

            return sumsq(self.grad)
        return self.grad.float().pow(2).sum()

    # ------------------------------------------------------------------ optimizer
    def attach_optimizer(self, opt: torch.optim.Optimizer):
        """Allocate flat moments and install views of them as the optimizer's per-parameter state."""
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.decay_flags.zero_()
        for group in opt.param_groups:
            for p in group["params"]:
                _, o, n = self.index[id(p)]
                if group["weight_decay"] != 0.0:
                    self.decay_flags[o // ALIGN:(o + _round_up(n, ALIGN)) // ALIGN] = 1
                opt.state[p] = {"step": torch.tensor(0.0), "exp_avg": self.exp_avg[o:o + n].view(p.shape),
                                "exp_avg_sq": self.exp_avg_sq[o:o + n].view(p.shape)}
        self._wd = max(g["weight_decay"] for g in opt.param_groups)

    def rebind_optimizer_state(self, opt: torch.optim.Optimizer):
        """After ``opt.load_state_dict`` replaced the state tensors: copy them back into the flat
        buffers and reinstall the views."""
        for p in self.params:
            st = opt.state.get(p)
            if not st:
                continue
            _, o, n = self.index[id(p)]
            for key, flat in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
                view = flat[o:o + n].view(p.shape)
                if st[key].data_ptr() != view.data_ptr():
                    view.copy_(st[key])
                    st[key] = view
            if not torch.is_tensor(st["step"]):
                st["step"] = torch.tensor(float(st["step"]))
            st["step"] = st["step"].detach().to("cpu", torch.float32)

    def fused_adamw_step(self, opt, step: int, grad_norm_sq, max_norm, lo: int = 0, hi: int | None = None):
        from nanonemo_b200.ops.adamw import adamw_flat

        g0 = opt.param_groups[0]
        hi = self.numel if hi is None else hi
        adamw_flat(self.master[lo:hi], self.grad[lo:hi], self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi],
                   None if self.shadow is None else self.shadow[lo:hi], self.decay_flags[lo // ALIGN:hi // ALIGN],
                   lr=g0["lr"], beta1=g0["betas"][0], beta2=g0["betas"][1], eps=g0["eps"], weight_decay=self._wd,
                   step=step, grad_norm_sq=grad_norm_sq, max_norm=max_norm, zero_grad=True)
        _shadow_rewritten()
