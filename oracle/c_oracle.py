"""ctypes front end of the plain-C oracle (``gemm_ref.c``).  TEST INFRASTRUCTURE ONLY."""

from __future__ import annotations

import ctypes

import torch

from .build import build

_lib = None


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        _lib.gemm_ref.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i32]
        _lib.gemm_ref.restype = None
        _lib.swiglu_ref.argtypes = [vp, vp, vp, vp, i64, i64, i64, i32]
        _lib.swiglu_ref.restype = None
    return _lib


def gemm_c(operation: str, *tensors: torch.Tensor) -> torch.Tensor:
    """``mm``/``addmm``/``bmm``/``swiglu`` on CPU tensors through the C oracle."""
    lib = _load()
    tensors = tuple(t.contiguous() for t in tensors)
    dtype = tensors[-1].dtype
    is_bf16 = 1 if dtype == torch.bfloat16 else 0
    if operation == "swiglu":
        x, wg, wu = tensors
        m, k = x.shape
        n = wg.shape[0]
        out = torch.empty((m, n), dtype=dtype)
        lib.swiglu_ref(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), out.data_ptr(), m, n, k, is_bf16)
        return out
    bias = None
    if operation == "addmm":
        bias, a, bt = tensors
    else:
        a, bt = tensors
    batch = a.shape[0] if operation == "bmm" else 1
    m, k = a.shape[-2:]
    n = bt.shape[-2]
    out = torch.empty((*a.shape[:-2], m, n), dtype=dtype)
    lib.gemm_ref(bias.data_ptr() if bias is not None else None, a.data_ptr(), bt.data_ptr(),
                 out.data_ptr(), batch, m, n, k, is_bf16)
    return out
