"""Raw launcher of the fused rotate-half RoPE on Q and K (csrc/elementwise.cu: rope_packed_kernel).

The kernel works on rows of a packed projection: the first ``n_rot_heads`` heads of every row are rotated, the
remaining ``n_copy_cols`` columns copied through (or left alone when input and output are the same buffer and
``n_copy_cols`` is 0). The inverse (backward) is the same kernel with the sine negated, so only the tables are saved
(as in the reference, nanonemo/kernels/triton/rope.py:44-45,87-90). The differentiable operators built on it are
registered in ``ops/library.py`` (``rope_qkv``, ``rope_rows``).
"""

import torch

from nanonemo_b200.ops import _lib

_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def rope_packed_raw(x2, out2, cos, sin, T, n_rot_heads, hd, n_copy_cols, sign):
    M = x2.shape[0]
    _lib.call("nnb_rope_packed", _lib.ptr(x2), _lib.ptr(out2), _lib.ptr(cos), _lib.ptr(sin), _lib.i64(M), _lib.i32(T),
              _lib.i32(n_rot_heads), _lib.i32(hd), _lib.i32(n_copy_cols), _lib.i64(x2.stride(0)), _lib.i64(out2.stride(0)),
              _lib.f32(sign), _lib.i32(_CODE[x2.dtype]), _lib.vp(_lib.stream_ptr()))


def _tables(cos, sin, T):
    cos, sin = cos[:T], sin[:T]
    if cos.dtype != torch.float32:
        cos, sin = cos.float(), sin.float()
    return cos.contiguous(), sin.contiguous()
