"""Bandwidth-bound operators: the sm100 kernels vs PyTorch eager and torch.compile, fwd and fwd+bwd, as a
fraction of the measured HBM copy bandwidth computed on the MINIMUM bytes each operator must move.

    python benchmarks/kernels/elementwise.py [--no-compile]
"""

import argparse

import torch
import torch.nn.functional as F
from common import peaks, run, time_ms

from nanonemo_b200 import ops
from nanonemo_b200.models.layers import rope_cache

M = 32768


def cases(compile_ok):
    bf = torch.bfloat16
    out = []
    # ---- add + RMSNorm: x fp32 residual, delta bf16 -> y bf16, h fp32
    x = torch.randn(M, 768, device="cuda", requires_grad=True)
    d = torch.randn(M, 768, device="cuda", dtype=bf, requires_grad=True)
    w = torch.ones(768, device="cuda", requires_grad=True)

    def ref_norm(x, d, w):
        h = x + d
        hf = h.float()
        return (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * w).to(d.dtype), h

    fwd_bytes = M * 768 * (4 + 2 + 2 + 4)
    bwd_bytes = M * 768 * (2 + 4 + 4 + 4 + 2)
    out.append(("add_rms_norm 32768x768", {"sm100": lambda: ops.add_rms_norm(x, d, w, 1e-5, impl="sm100"), "eager": lambda: ref_norm(x, d, w),
                                           "compile": (lambda f: (lambda: f(x, d, w)))(torch.compile(ref_norm)) if compile_ok else None},
                (x, d, w), fwd_bytes, fwd_bytes + bwd_bytes))
    # ---- SwiGLU on the packed projection
    gu = torch.randn(M, 4096, device="cuda", dtype=bf, requires_grad=True)

    def ref_swiglu(gu):
        g, u = gu.chunk(2, -1)
        return F.silu(g) * u

    out.append(("swiglu 32768x2048", {"sm100": lambda: ops.swiglu_packed(gu, impl="sm100"), "eager": lambda: ref_swiglu(gu),
                                      "compile": (lambda f: (lambda: f(gu)))(torch.compile(ref_swiglu)) if compile_ok else None},
                (gu,), M * 2048 * 2 * 3, M * 2048 * 2 * (3 + 5)))
    # ---- RoPE on packed QKV
    cos, sin = rope_cache(64, 1024, device="cuda")
    qkv = torch.randn(32, 1024, 1280, device="cuda", dtype=bf, requires_grad=True)
    ref_rope = lambda t: ops.rope_qkv(t, cos, sin, 12, 4, 64, impl="torch")
    out.append(("rope_qkv B32 T1024 (12+4 heads)", {"sm100": lambda: ops.rope_qkv(qkv, cos, sin, 12, 4, 64, impl="sm100"), "eager": lambda: ref_rope(qkv),
                                                   "compile": (lambda f: (lambda: f(qkv)))(torch.compile(ref_rope)) if compile_ok else None},
                (qkv,), M * 1280 * 2 * 2, M * 1280 * 2 * 4))
    return out


def rows_fn(compile_ok):
    rows, bw = [], peaks()["hbm_gbs"]
    for name, providers, inputs, b_f, b_fb in cases(compile_ok):
        for prov, fn in providers.items():
            if fn is None:
                continue
            try:
                def fb():
                    o = fn()
                    o = o if isinstance(o, tuple) else (o,)
                    torch.autograd.grad([t for t in o], inputs, [torch.ones_like(t) for t in o], allow_unused=True)

                t_f, t_fb = time_ms(fn, iters=20), time_ms(fb, iters=20)
            except Exception as e:  # noqa: BLE001
                rows.append({"op": name, "provider": prov, "fwd_ms": float("nan"), "fwd_bwd_ms": float("nan"), "fwd_frac_hbm": 0.0,
                             "fwd_bwd_frac_hbm": 0.0, "note": type(e).__name__})
                continue
            rows.append({"op": name, "provider": prov, "fwd_ms": t_f, "fwd_bwd_ms": t_fb, "fwd_frac_hbm": b_f / t_f / 1e6 / bw,
                         "fwd_bwd_frac_hbm": b_fb / t_fb / 1e6 / bw, "note": ""})
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--no-compile", action="store_true")
    a = ap.parse_args()
    run("elementwise", lambda: rows_fn(not a.no_compile))
