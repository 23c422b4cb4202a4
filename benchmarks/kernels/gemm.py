"""tcgen05 GEMMs vs torch.matmul (cuBLAS) at the training shapes of the 114M and 1.3B models: the default dispatch (CTA
pairs where they apply), the single-CTA kernel alone (bn=256 / auto), and the MXFP8 block-scaled kernel on pre-quantised
operands for the K-major shapes.

    python benchmarks/kernels/gemm.py [--tokens 32768] [--quick]
"""

import argparse

import torch
from common import peaks, run, time_ms

from nanonemo_b200.ops.gemm import check_status, gemm


def shapes(tokens: int, quick: bool):
    M = tokens
    s = [  # (label, layout, M, N, K)
        ("qkv fprop", "nn", M, 2304, 768), ("o fprop", "nn", M, 768, 768), ("gate_up fprop", "nn", M, 4096, 768),
        ("down fprop", "nn", M, 768, 2048),
        ("qkv dgrad", "dgrad", M, 768, 2304), ("gate_up dgrad", "dgrad", M, 768, 4096), ("down dgrad", "dgrad", M, 2048, 768),
        ("qkv wgrad", "wgrad", 2304, 768, M), ("gate_up wgrad", "wgrad", 4096, 768, M), ("down wgrad", "wgrad", 768, 2048, M),
        ("head fprop", "nn", M, 50304, 768), ("head dgrad", "dgrad", M, 768, 50304), ("head wgrad", "wgrad", 50304, 768, M),
    ]
    if not quick:
        s += [("8192^3", "nn", 8192, 8192, 8192), ("1.3B gate_up fprop", "nn", M, 11264, 2048),
              ("1.3B down fprop", "nn", M, 2048, 5632)]
    return s


def rows_fn(tokens, quick):
    rows = []
    pk = peaks()
    for label, layout, M, N, K in shapes(tokens, quick):
        if layout == "nn":
            a = torch.randn(M, K, device="cuda").bfloat16()
            b = torch.randn(N, K, device="cuda").bfloat16()
            ours = lambda: gemm(a, b)
            ref = lambda: torch.matmul(a, b.t())
        elif layout == "dgrad":
            a = torch.randn(M, K, device="cuda").bfloat16()
            b = torch.randn(K, N, device="cuda").bfloat16()
            ours = lambda: gemm(a, b, b_mn=True)
            ref = lambda: torch.matmul(a, b)
        else:
            a = torch.randn(K, M, device="cuda").bfloat16()
            b = torch.randn(K, N, device="cuda").bfloat16()
            out = torch.zeros(M, N, device="cuda")
            ours = lambda: gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)
            ref = lambda: torch.matmul(a.t(), b)  # bf16 output: cheaper than our fp32 accumulate-in-place
        t_ours, t_ref = time_ms(ours), time_ms(ref)
        single = {"nn": lambda: gemm(a, b, bn=256), "dgrad": lambda: gemm(a, b, b_mn=True, bn=256),
                  "wgrad": lambda: gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True, bn=256)}[layout]
        t_single = time_ms(single)
        t_fp8 = float("nan")
        if layout == "nn" and M % 128 == 0 and N % 128 == 0 and K % 128 == 0:
            from nanonemo_b200 import fp8

            aq, asf, _, _ = fp8.quantize_mx(a)
            bq, bsf, _, _ = fp8.quantize_mx(b)
            t_fp8 = time_ms(lambda: fp8.gemm_mxfp8(aq, asf, bq, bsf))
        check_status()
        flops = 2.0 * M * N * K
        rows.append({"shape": label, "M": M, "N": N, "K": K, "ours_ms": t_ours, "single_cta_ms": t_single, "mxfp8_ms": t_fp8,
                     "cublas_ms": t_ref, "ours_tflops": flops / t_ours / 1e9, "single_cta_tflops": flops / t_single / 1e9,
                     "mxfp8_tflops": flops / t_fp8 / 1e9, "cublas_tflops": flops / t_ref / 1e9,
                     "ours_vs_cublas": t_ref / t_ours, "frac_of_measured_peak": flops / t_ours / 1e9 / pk["bf16_tflops"]})
        del a, b
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--quick", action="store_true")
    a = ap.parse_args()
    run("gemm", lambda: rows_fn(a.tokens, a.quick))
