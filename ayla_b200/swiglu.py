"""Fused SwiGLU op: ``out = silu(x @ w_gate.T) * (x @ w_up.T)`` in one kernel.

The reference has the building blocks (an ``elementwise silu`` and ``mul`` on fp32
accumulators, ayla/passes/lower_to_ptx_template.py:296-315, :62-81, and a fused
matmul+sigmoid op, ayla/gemm_collection/auto_matmul_4096_wgmma256_wg_sigmoid.py:22-142)
but no complete op.  This one follows the calling convention of ``gemm_op``: the
caller allocates ``out`` and the op returns ``None``.
"""

from __future__ import annotations

import os
from functools import cache

import torch

from . import _lib
from .gemm_jit import _SHORT_DTYPES, _TORCH_DTYPES
from .jit_compiler import OpTemplate, ShapeSpecializingJITCompiler
from .torch_custom_call import DEFAULT_NAMESPACE, OperandKind, TensorSpec, make_torch_custom_call


class SwigluLauncher:
    def __init__(self, dtype: str, m: int, n: int, k: int, device: torch.device,
                 config: dict | None = None):
        self.dtype, self.m, self.n, self.k, self.device = dtype, m, n, k, device
        index = device.index if device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(index):
            _lib.init(index)
        self.config = _lib.Config.from_dict(config) if config is not None else None
        self.status = _lib.StatusWord()  # pinned host word: read before every launch without a synchronise
        self._status_ptr = self.status.ptr
        self._device_index = index
        self._debug = bool(os.environ.get("AYLA_B200_DEBUG"))

    def __call__(self, x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                 out: torch.Tensor) -> None:
        if self.status.peek():
            self._report_timeout()
        with torch.cuda.device(self._device_index):
            _lib.swiglu(self.dtype, x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), out.data_ptr(),
                        self.m, self.n, self.k, self.config, self._status_ptr,
                        torch.cuda.current_stream(self._device_index).cuda_stream)
        if self._debug:
            self.check_status()

    def _report_timeout(self) -> None:
        code = self.status.peek()
        self.status.clear()
        raise RuntimeError(f"swiglu: device wait timed out (code {code & 0xFF}, CTA {code >> 8})")

    def check_status(self) -> None:
        """Synchronise and raise if one of the kernel's bounded waits gave up."""
        torch.cuda.synchronize(self._device_index)
        if self.status.peek():
            self._report_timeout()


def swiglu_compiler(dtype: str) -> ShapeSpecializingJITCompiler:
    if dtype not in _SHORT_DTYPES:
        raise ValueError(f"unsupported SwiGLU dtype {dtype}")
    tensor = TensorSpec(_TORCH_DTYPES[dtype], (None, None))
    template = OpTemplate(f"swiglu_{_SHORT_DTYPES[dtype]}", (tensor, tensor, tensor, tensor))

    def compile_specialization(bound: OpTemplate, device: torch.device) -> SwigluLauncher:
        x, w_gate, w_up, out = (spec.sizes for spec in bound.signature)
        m, k = x
        n = w_gate[0]
        if tuple(w_gate) != (n, k) or tuple(w_up) != (n, k):
            raise ValueError(
                f"{bound.name}: w_gate and w_up must both be ({n}, {k}), got {tuple(w_gate)} and {tuple(w_up)}"
            )
        if tuple(out) != (m, n):
            raise ValueError(f"{bound.name}: out must be ({m}, {n}), got {tuple(out)}")
        if n % 8 or k % 8:
            raise ValueError(f"{bound.name}: no schedule for swiglu {m}x{n}x{k} (n and k must be multiples of 8)")
        return SwigluLauncher(dtype, m, n, k, device)

    return ShapeSpecializingJITCompiler(template, compile_specialization)


_COMPILERS: dict[tuple[str, str], ShapeSpecializingJITCompiler] = {}


def swiglu_op(dtype: str = "bfloat16", namespace: str = DEFAULT_NAMESPACE) -> torch._ops.OpOverload:
    """Torch op ``(x, w_gate, w_up, out) -> ()`` (cached per dtype and namespace)."""
    return _swiglu_op(dtype, namespace)


@cache
def _swiglu_op(dtype: str, namespace: str) -> torch._ops.OpOverload:
    compiler = swiglu_compiler(dtype)
    _COMPILERS[(dtype, namespace)] = compiler
    return make_torch_custom_call(compiler, [OperandKind.R] * 3 + [OperandKind.RW], namespace=namespace)


def swiglu_op_compiler(dtype: str = "bfloat16",
                       namespace: str = DEFAULT_NAMESPACE) -> ShapeSpecializingJITCompiler:
    swiglu_op(dtype, namespace)
    return _COMPILERS[(dtype, namespace)]
