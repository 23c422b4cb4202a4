"""Loader for the ahead-of-time built kernel library ``nanonemo_b200/csrc/libnanonemo_b200.so``.

The kernels are plain ``extern "C"`` launchers taking device pointers, sizes and a stream, compiled
by ``nanonemo_b200/csrc/build.py`` with ``nvcc -gencode arch=compute_100a,code=sm_100a`` and loaded
here with ctypes; they are built before the run (never JIT-compiled per process, unlike the
reference's ``torch.utils.cpp_extension.load`` in nanonemo/kernels/cuda/__init__.py:15-18) and the
library sits in the source tree. Every launcher returns 0 on success or a negative error code
(bad argument, CUDA launch error) that ``check`` turns into an exception.
"""

import ctypes
import os
from functools import lru_cache
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parents[1] / "csrc" / "libnanonemo_b200.so"


@lru_cache(maxsize=1)
def _load():
    if not LIB_PATH.exists():
        return None
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.nnb_last_error.restype = ctypes.c_char_p
    return lib


def available() -> bool:
    """True when the built library exists and a CUDA device is present."""
    return torch.cuda.is_available() and _load() is not None and os.environ.get("NANONEMO_DISABLE_SM100") != "1"


def lib():
    handle = _load()
    if handle is None:
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m nanonemo_b200.csrc.build` "
                           "(the sm100 operators have no fallback)")
    return handle


LAUNCHES = 0  # launchers called through `call` since import (the benchmark reports the delta)


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def call(name: str, *args) -> None:
    """Call launcher `name`; raises with the library's message on a non-zero return."""
    global LAUNCHES
    fn = getattr(lib(), name)
    rc = fn(*args)
    LAUNCHES += 1
    if rc != 0:
        msg = lib().nnb_last_error()
        raise RuntimeError(f"{name} failed (code {rc}): {msg.decode() if msg else 'no message'}")


def call_rc(name: str, *args) -> int:
    """Like `call`, for launchers that answer 1 when they do not serve the problem (nothing was launched): returns 0 or 1."""
    global LAUNCHES
    rc = getattr(lib(), name)(*args)
    if rc == 0:
        LAUNCHES += 1
    elif rc != 1:
        msg = lib().nnb_last_error()
        raise RuntimeError(f"{name} failed (code {rc}): {msg.decode() if msg else 'no message'}")
    return rc


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


i32, i64, f32, vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p
