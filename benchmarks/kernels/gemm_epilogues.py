"""GEMMs with a fused epilogue against the plain GEMM followed by the stand-alone elementwise kernel, at the 114M shapes:
gate||up projection + SwiGLU, QKV projection + RoPE, head projection + softmax statistics, and the down projection's
input-gradient GEMM + SwiGLU backward. Each row gives both times and the bytes the fused form does not move.

    python benchmarks/kernels/gemm_epilogues.py [--tokens 32768]
"""

import argparse

import torch
from common import run, time_ms

from nanonemo_b200.models.layers import rope_cache
from nanonemo_b200.ops import rope, swiglu_act
from nanonemo_b200.ops.gemm import check_status, gemm, gemm_ce_stats, gemm_rope, gemm_swiglu, gemm_swiglu_bwd


def rows_fn(M: int):
    bf, dev = torch.bfloat16, "cuda"
    d, F, H, KVH, hd, T = 768, 2048, 12, 4, 64, 1024
    rows = []

    def add(name, fused, unfused, saved_bytes, flops):
        tf, tu = time_ms(fused), time_ms(unfused)
        check_status()
        rows.append({"op": name, "fused_ms": tf, "unfused_ms": tu, "speedup": tu / tf, "fused_tflops": flops / tf / 1e9,
                     "hbm_MB_not_moved": saved_bytes / 1e6})

    x = torch.randn(M, d, device=dev, dtype=bf)
    w_gu = torch.randn(2 * F, d, device=dev, dtype=bf) * 0.03
    act = torch.empty(M, F, device=dev, dtype=bf)

    def unfused_swiglu():
        gu = gemm(x, w_gu)
        swiglu_act.fwd_raw(gu[:, :F], gu[:, F:], act)

    add("gate_up fprop + SwiGLU", lambda: gemm_swiglu(x, w_gu), unfused_swiglu, M * 2 * F * 2, 2.0 * M * 2 * F * d)

    w_qkv = torch.randn((H + 2 * KVH) * hd, d, device=dev, dtype=bf) * 0.03
    cos, sin = (t.contiguous() for t in rope_cache(hd, T, device=dev))

    def unfused_rope():
        qkv = gemm(x, w_qkv)
        rope.rope_packed_raw(qkv, qkv, cos, sin, T, H + KVH, hd, 0, 1.0)

    add("qkv fprop + RoPE", lambda: gemm_rope(x, w_qkv, cos, sin, T, (H + KVH) * hd, hd), unfused_rope,
        2 * M * (H + KVH) * hd * 2, 2.0 * M * w_qkv.shape[0] * d)

    rows_ce = 4096
    xh = x[:rows_ce]
    w_head = torch.randn(50304, d, device=dev, dtype=bf) * 0.03
    logits = torch.empty(rows_ce, 50304, device=dev, dtype=bf)
    add("head fprop + softmax statistics (4096 rows)", lambda: gemm_ce_stats(xh, w_head, logits), lambda: gemm(xh, w_head, out=logits),
        rows_ce * 50304 * 2, 2.0 * rows_ce * 50304 * d)  # the statistics replace the first sweep of the two-sweep CE kernel

    dy = torch.randn(M, d, device=dev, dtype=bf)
    w_down = torch.randn(d, F, device=dev, dtype=bf) * 0.03
    gu = torch.randn(M, 2 * F, device=dev, dtype=bf)
    dgu = torch.empty_like(gu)

    def unfused_bwd():
        dact = gemm(dy, w_down, b_mn=True)
        swiglu_act.bwd_raw(dact, gu[:, :F], gu[:, F:], dgu[:, :F], dgu[:, F:])

    add("down dgrad + SwiGLU backward", lambda: gemm_swiglu_bwd(dy, w_down, gu), unfused_bwd, 2 * M * F * 2, 2.0 * M * F * d)
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    a = ap.parse_args()
    run("gemm_epilogues", lambda: rows_fn(a.tokens))
