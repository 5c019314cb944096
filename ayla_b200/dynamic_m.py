"""Dynamic-M bf16 GEMM as an allocating op: ``op(lhs, rhs) -> out``.

Counterpart of the reference's ``make_dynamic_m_matmul`` (ayla/gemm_collection/dynamic_m.py:90-121):
``rhs`` is a fixed ``[n, k]`` weight, ``lhs`` is ``[m, k]`` with any ``m``, the result ``[m, n]`` is
allocated by the op and its shape inferred from the inputs; one schedule is cached per exact shape.
The reference's three-regime heuristic (:34-66) is replaced by the schedule table / shape-aware
default of this backend, which has dedicated weight-streaming schedules for small ``m``.
"""

from __future__ import annotations

import torch

from .gemm_jit import GemmLauncher, select_gemm_schedule
from .jit_compiler import OpTemplate, ShapeSpecializingJITCompiler
from .torch_custom_call import DEFAULT_NAMESPACE, OperandKind, TensorSpec, make_torch_custom_call


def make_dynamic_m_matmul(n: int, k: int, *, name: str | None = None, namespace: str = DEFAULT_NAMESPACE):
    """Create an exact-shape cached ``op(lhs[m, k], rhs[n, k]) -> out[m, n]`` bf16 GEMM."""
    if n <= 0 or k <= 0:
        raise ValueError("problem dimensions must be positive")
    name = name or f"dynamic_m_matmul_n{n}_k{k}"
    bf16 = torch.bfloat16
    template = OpTemplate(name, (TensorSpec(bf16, (None, k)), TensorSpec(bf16, (n, k)), TensorSpec(bf16, (None, n))))

    def compile_specialization(bound: OpTemplate, device: torch.device) -> GemmLauncher:
        m = bound.signature[0].sizes[0]
        if bound.signature[2].sizes[0] != m:
            raise ValueError(f"{name}: out must have {m} rows")
        schedule = select_gemm_schedule("mm", "bfloat16", m, n, k)
        if schedule is None:
            raise ValueError(f"{name}: no schedule for mm {m}x{n}x{k}")
        return GemmLauncher("mm", "bfloat16", 1, m, n, k, schedule, device)

    compiler = ShapeSpecializingJITCompiler(template, compile_specialization)
    return make_torch_custom_call(
        compiler,
        [OperandKind.R, OperandKind.R, OperandKind.RESULT],
        namespace=namespace,
        infer_result_shapes=lambda lhs, _rhs: [(lhs.shape[0], n)],
    )
