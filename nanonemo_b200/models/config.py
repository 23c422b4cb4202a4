"""Model hyper-parameters and kernel switches.

Same fields and defaults as the reference ``ModelConfig`` (nanonemo/model/config.py:7-53) so that
every reference YAML loads unchanged. Each kernel switch keeps its reference values and gains the
value ``sm100``: the hand-written Blackwell kernel in ``nanonemo_b200/csrc``. The reference values
``triton`` / ``cuda`` / ``fused`` / ``te`` name kernels this framework does not ship; they resolve
to the single ``sm100`` implementation of that operator (``resolved()``), so a stage config keeps
its meaning ("use the custom kernel here") without a second backend behind it.
"""

from dataclasses import dataclass, replace

_SWITCHES = {
    # switch: (reference values, values that resolve to the sm100 kernel)
    "norm_kernel": (("torch", "triton", "cuda", "sm100"), ("triton", "cuda", "sm100")),
    "swiglu_kernel": (("torch", "triton", "sm100"), ("triton", "sm100")),
    "rope_kernel": (("torch", "triton", "sm100"), ("triton", "sm100")),
    "attn_kernel": (("torch", "cuda", "sm100"), ("cuda", "sm100")),
    "loss_kernel": (("torch", "fused", "sm100"), ("fused", "sm100")),
    "linear_impl": (("torch", "te", "sm100", "mxfp8"), ("sm100",)),
    "embed_kernel": (("torch", "sm100"), ("sm100",)),
}


@dataclass
class ModelConfig:
    n_layers: int = 12
    d_model: int = 768
    n_heads: int = 12
    n_kv_heads: int = 4
    d_ff: int = 2048
    vocab_size: int = 50304
    max_seq_len: int = 1024
    norm_eps: float = 1e-5
    rope_base: float = 10000.0
    init_std: float = 0.02
    attn_backend: str = "math"  # SDPA backend of the torch attention path: math | mem_efficient
    norm_kernel: str = "torch"
    swiglu_kernel: str = "torch"
    rope_kernel: str = "torch"
    attn_kernel: str = "torch"
    loss_kernel: str = "torch"
    linear_impl: str = "torch"  # torch | sm100 (tcgen05 bf16 GEMM) | mxfp8 (block-scaled fp8; "te" resolves here)
    embed_kernel: str = "torch"
    head_dim_override: int | None = None  # head_dim when it is not d_model / n_heads (1.3B: 16 heads x 128)
    fuse_epilogues: bool = True  # sm100 path: RoPE / SwiGLU / softmax statistics inside the producing GEMM's epilogue

    def __post_init__(self):
        assert self.n_heads % self.n_kv_heads == 0, "query heads must group evenly over KV heads"
        if self.head_dim_override is None:
            assert self.d_model % self.n_heads == 0, "d_model must divide evenly into heads"
        assert self.head_dim % 2 == 0, "RoPE rotates pairs of dimensions"
        assert self.attn_backend in ("math", "mem_efficient"), f"unknown attn_backend {self.attn_backend!r}"
        for name, (allowed, _) in _SWITCHES.items():
            assert getattr(self, name) in allowed, f"unknown {name} {getattr(self, name)!r}"

    @property
    def head_dim(self) -> int:
        return self.head_dim_override or self.d_model // self.n_heads

    def uses_sm100(self, switch: str) -> bool:
        """True when `switch` selects this framework's Blackwell kernel."""
        value = getattr(self, switch)
        if switch == "linear_impl":
            return value in ("sm100", "mxfp8", "te")
        return value in _SWITCHES[switch][1]

    @property
    def fp8(self) -> bool:
        return self.linear_impl in ("mxfp8", "te")

    def resolved(self) -> "ModelConfig":
        """Copy with every alias replaced by the kernel that actually runs."""
        out = {}
        for name in _SWITCHES:
            if name == "linear_impl":
                out[name] = {"te": "mxfp8"}.get(self.linear_impl, self.linear_impl)
            else:
                out[name] = "sm100" if self.uses_sm100(name) else "torch"
        return replace(self, **out)

    @classmethod
    def sm100(cls, **kw) -> "ModelConfig":
        """All operators on the hand-written Blackwell kernels."""
        base = dict(norm_kernel="sm100", swiglu_kernel="sm100", rope_kernel="sm100", attn_kernel="sm100",
                    loss_kernel="sm100", linear_impl="sm100", embed_kernel="sm100", attn_backend="mem_efficient")
        base.update(kw)
        return cls(**base)
