"""Causal GQA attention: the tcgen05 kernels vs PyTorch SDPA (mem-efficient = the reference's choice; flash
and cuDNN for context) at the training shape B=32, H=12, KVH=4, T=1024, hd=64 and a few others.

    python benchmarks/kernels/flash_attn.py [--quick]
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
        q = torch.randn(B, T, H, hd, device="cuda", dtype=torch.bfloat16).transpose(1, 2).requires_grad_()
        k = torch.randn(B, T, KVH, hd, device="cuda", dtype=torch.bfloat16).transpose(1, 2).requires_grad_()
        v = torch.randn(B, T, KVH, hd, device="cuda", dtype=torch.bfloat16).transpose(1, 2).requires_grad_()
        g = torch.randn(B, H, T, hd, device="cuda", dtype=torch.bfloat16)

        def sdpa(backend):
            def f():
                kk, vv = k.repeat_interleave(H // KVH, 1), v.repeat_interleave(H // KVH, 1)
                with sdpa_kernel(backend):
                    return F.scaled_dot_product_attention(q, kk, vv, is_causal=True)
            return f

        providers = {"sm100": lambda: ops.flash_attn(q, k, v), "sdpa_mem_efficient": sdpa(SDPBackend.EFFICIENT_ATTENTION),
                     "sdpa_flash": sdpa(SDPBackend.FLASH_ATTENTION)}
        for name, fn in providers.items():
            try:
                t_f = time_ms(fn, iters=20)
                t_fb = time_ms(lambda: torch.autograd.grad(fn(), (q, k, v), g), iters=20)
            except Exception as e:  # a backend that does not support the shape
                rows.append({"case": f"B{B} H{H}/{KVH} T{T} hd{hd}", "provider": name, "fwd_ms": float("nan"), "fwd_bwd_ms": float("nan"),
                             "fwd_tflops": 0.0, "fwd_bwd_tflops": 0.0, "note": type(e).__name__})
                continue
            rows.append({"case": f"B{B} H{H}/{KVH} T{T} hd{hd}", "provider": name, "fwd_ms": t_f, "fwd_bwd_ms": t_fb,
                         "fwd_tflops": flops(B, H, T, hd, False) / t_f / 1e9, "fwd_bwd_tflops": flops(B, H, T, hd, True) / t_fb / 1e9,
                         "note": ""})
        check_status()
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    a = ap.parse_args()
    run("flash_attn", lambda: rows_fn(a.quick))
