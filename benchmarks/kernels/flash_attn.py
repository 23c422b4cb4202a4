"""Causal GQA attention: the tcgen05 kernels vs PyTorch SDPA (mem-efficient = the reference's choice; the default backend
and flash for context) at the training shape B=32, H=12, KVH=4, T=1024, hd=64 and a few others.

    python benchmarks/kernels/flash_attn.py [--quick]

Columns: forward alone, forward + backward through autograd (what a training step pays, repeat_interleave of K / V included
for the SDPA providers, which have no GQA-direct path on every backend), and the BACKWARD alone (the gradient call on a
retained graph: for `sm100` that is the delta pre-pass, the backward kernel and the dQ conversion). All timed as CUDA-graph
replays with the L2 flushed before each.
"""

import argparse

import torch
import torch.nn.functional as F
from common import run, time_ms
from torch.nn.attention import SDPBackend, sdpa_kernel

from nanonemo_b200 import ops
from nanonemo_b200.ops.gemm import check_status

CASES = [(32, 12, 4, 1024, 64), (8, 12, 4, 4096, 64), (128, 12, 4, 256, 64), (8, 16, 4, 2048, 128)]


def flops(B, H, T, hd, bwd):
    f = 4 * B * H * T * T * hd / 2  # causal: half of the square
    return f * (3.5 if bwd else 1.0)


def rows_fn(quick):
    rows = []
    for B, H, KVH, T, hd in (CASES[:1] if quick else CASES):
        # inputs come from the CPU generator: a provider whose capture into a CUDA graph fails can leave the CUDA generator
        # unusable for the rest of the process
        rnd = lambda *shape: torch.randn(*shape).to("cuda", torch.bfloat16)
        q = rnd(B, T, H, hd).transpose(1, 2).requires_grad_()
        k = rnd(B, T, KVH, hd).transpose(1, 2).requires_grad_()
        v = rnd(B, T, KVH, hd).transpose(1, 2).requires_grad_()
        g = rnd(B, H, T, hd)

        def sdpa(backend):
            def f():
                kk, vv = k.repeat_interleave(H // KVH, 1), v.repeat_interleave(H // KVH, 1)
                with sdpa_kernel(backend):
                    return F.scaled_dot_product_attention(q, kk, vv, is_causal=True)
            return f

        def sdpa_default():
            return F.scaled_dot_product_attention(q, k.repeat_interleave(H // KVH, 1), v.repeat_interleave(H // KVH, 1), is_causal=True)

        providers = {"sm100": lambda: ops.flash_attn(q, k, v), "sdpa_mem_efficient": sdpa(SDPBackend.EFFICIENT_ATTENTION),
                     "sdpa_flash": sdpa(SDPBackend.FLASH_ATTENTION), "sdpa_default": sdpa_default}
        for name, fn in providers.items():
            try:
                t_f = time_ms(fn, iters=20)
                t_fb = time_ms(lambda: torch.autograd.grad(fn(), (q, k, v), g), iters=20)
                out = fn()
                t_b = time_ms(lambda: torch.autograd.grad(out, (q, k, v), g, retain_graph=True), iters=20)
            except Exception as e:  # a backend that does not support the shape
                rows.append({"case": f"B{B} H{H}/{KVH} T{T} hd{hd}", "provider": name, "fwd_ms": float("nan"), "fwd_bwd_ms": float("nan"),
                             "bwd_ms": float("nan"), "fwd_tflops": 0.0, "fwd_bwd_tflops": 0.0, "note": type(e).__name__})
                continue
            rows.append({"case": f"B{B} H{H}/{KVH} T{T} hd{hd}", "provider": name, "fwd_ms": t_f, "fwd_bwd_ms": t_fb, "bwd_ms": t_b,
                         "fwd_tflops": flops(B, H, T, hd, False) / t_f / 1e9, "fwd_bwd_tflops": flops(B, H, T, hd, True) / t_fb / 1e9,
                         "note": ""})
        check_status()
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    a = ap.parse_args()
    run("flash_attn", lambda: rows_fn(a.quick))
