"""Small profiler target: a few launches of one kernel family at a shape larger than L2 but holding only
a few hundred MB, so an `ncu --set full` capture ends by itself in about a minute.

    python benchmarks/kernels/ncu_target.py {gemm,gemm_single,gemm_mxfp8,gemm_swiglu,gemm_swiglu_bwd,gemm_rope,flash,flash128,rmsnorm,swiglu,rope,
                                             ce,adamw,embedding,quantize}[,more targets] [iters]
"""

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from nanonemo_b200 import ops  # noqa: E402


def build(kind: str):
    """-> a callable that launches the kernels of target `kind` once (inputs are created here, outside the captured launches)."""
    dev, bf = "cuda", torch.bfloat16
    M = 32768
    if kind == "gemm":
        from nanonemo_b200.ops.gemm import gemm

        a, b = torch.randn(M, 768, device=dev, dtype=bf), torch.randn(4096, 768, device=dev, dtype=bf)
        fn = lambda: gemm(a, b)  # default dispatch: the CTA-pair kernel (gemm2_tcgen05_kernel)
    elif kind == "gemm_single":
        from nanonemo_b200.ops.gemm import gemm

        a, b = torch.randn(M, 768, device=dev, dtype=bf), torch.randn(4096, 768, device=dev, dtype=bf)
        fn = lambda: gemm(a, b, bn=256)
    elif kind == "gemm_mxfp8":
        from nanonemo_b200 import fp8

        aq, asf, _, _ = fp8.quantize_mx(torch.randn(M, 768, device=dev, dtype=bf))
        bq, bsf, _, _ = fp8.quantize_mx(torch.randn(4096, 768, device=dev, dtype=bf))
        fn = lambda: fp8.gemm_mxfp8(aq, asf, bq, bsf)
    elif kind == "gemm_swiglu":
        from nanonemo_b200.ops.gemm import gemm_swiglu

        a, b = torch.randn(M, 768, device=dev, dtype=bf), torch.randn(4096, 768, device=dev, dtype=bf)
        fn = lambda: gemm_swiglu(a, b)  # gate||up projection with the SwiGLU epilogue (gemm2_tcgen05_kernel<1>)
    elif kind == "gemm_swiglu_bwd":
        from nanonemo_b200.ops.gemm import gemm_swiglu_bwd

        dy, w_down = torch.randn(M, 768, device=dev, dtype=bf), torch.randn(768, 2048, device=dev, dtype=bf) * 0.03
        gu = torch.randn(M, 4096, device=dev, dtype=bf)
        fn = lambda: gemm_swiglu_bwd(dy, w_down, gu)  # down projection's dgrad with the SwiGLU backward epilogue (gemm2_tcgen05_kernel<4>)
    elif kind == "gemm_rope":
        from nanonemo_b200.models.layers import rope_cache
        from nanonemo_b200.ops.gemm import gemm_rope

        cos, sin = (t.contiguous() for t in rope_cache(64, 1024, device=dev))
        a, b = torch.randn(M, 768, device=dev, dtype=bf), torch.randn(1280, 768, device=dev, dtype=bf)
        fn = lambda: gemm_rope(a, b, cos, sin, 1024, 1024, 64)  # QKV projection with the RoPE epilogue (gemm2_tcgen05_kernel<2>)
    elif kind == "embedding":
        idx = torch.randint(0, 50257, (M,), device=dev)
        w = (torch.randn(50304, 768, device=dev) * 0.02).requires_grad_()
        fn = lambda: ops.embedding(idx, w, impl="sm100").sum().backward()
    elif kind == "quantize":
        from nanonemo_b200 import fp8

        x = torch.randn(M, 2048, device=dev, dtype=bf)
        fn = lambda: fp8.quantize_mx(x, True, True)  # one read -> row-wise e4m3 copy + transposed copy + both scale sets
    elif kind == "flash128":
        qkv = torch.randn(4, 2048, 24 * 128, device=dev, dtype=bf, requires_grad=True)
        fn = lambda: ops.attention_packed(qkv, 16, 4, 128, impl="sm100").sum().backward()
    elif kind == "flash":
        qkv = torch.randn(8, 1024, 1280, device=dev, dtype=bf, requires_grad=True)
        fn = lambda: ops.attention_packed(qkv, 12, 4, 64, impl="sm100").sum().backward()
    elif kind == "rmsnorm":
        x = torch.randn(M, 768, device=dev, requires_grad=True)
        d = torch.randn(M, 768, device=dev, dtype=bf, requires_grad=True)
        w = torch.ones(768, device=dev, requires_grad=True)
        fn = lambda: sum(t.float().sum() for t in ops.add_rms_norm(x, d, w, 1e-5, impl="sm100")).backward()
    elif kind == "swiglu":
        gu = torch.randn(M, 4096, device=dev, dtype=bf, requires_grad=True)
        fn = lambda: ops.swiglu_packed(gu, impl="sm100").sum().backward()
    elif kind == "rope":
        from nanonemo_b200.models.layers import rope_cache

        cos, sin = rope_cache(64, 1024, device=dev)
        qkv = torch.randn(32, 1024, 1280, device=dev, dtype=bf)
        fn = lambda: ops.rope_qkv(qkv, cos, sin, 12, 4, 64, impl="sm100")
    elif kind == "ce":
        x = torch.randn(4096, 768, device=dev, dtype=bf, requires_grad=True)
        w = (torch.randn(50304, 768, device=dev) * 0.02).requires_grad_()
        t = torch.randint(0, 50257, (4096,), device=dev)
        fn = lambda: ops.linear_cross_entropy(x, w, t).backward()
    elif kind == "adamw":
        from nanonemo_b200.ops.adamw import adamw_flat, sumsq

        n = 64 * 1024 * 1024
        p, g, m, v = (torch.randn(n, device=dev) for _ in range(4))
        v.abs_()
        sh = torch.empty(n, device=dev, dtype=bf)
        fl = torch.ones(n // 256, dtype=torch.uint8, device=dev)
        fn = lambda: adamw_flat(p, g, m, v, sh, fl, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=1,
                                grad_norm_sq=sumsq(g), max_norm=1.0)
    else:
        raise SystemExit(f"unknown target {kind}")
    return fn


def main():
    kinds = (sys.argv[1] if len(sys.argv) > 1 else "gemm").split(",")  # several targets: one after the other, inputs freed in between
    iters = int(sys.argv[2]) if len(sys.argv) > 2 else 3
    for kind in kinds:
        fn = build(kind)
        for _ in range(iters):
            fn()
        torch.cuda.synchronize()
        del fn
        torch.cuda.empty_cache()
        print("done", kind, flush=True)


if __name__ == "__main__":
    main()
