"""B200 (sm_100a) GEMM backend behind the operator surface of frgossen/ayla.

Public surface (same names as the reference, ayla/gemm_jit.py and
ayla/torch_custom_call.py)::

    from ayla_b200 import gemm_op, select_gemm_schedule, measured_gemm_configs, swiglu_op
    gemm_op("mm", "bfloat16")(a, bt, out)          # out = a @ bt.T
    gemm_op("addmm", "float16")(bias, a, bt, out)  # out = bias + a @ bt.T
    gemm_op("bmm", "bfloat16")(a, bt, out)         # batched
    swiglu_op("bfloat16")(x, w_gate, w_up, out)    # out = silu(x@w_gate.T) * (x@w_up.T)
    gemm_act_op("addmm", "gelu", "bfloat16")(bias, a, bt, out)  # out = gelu(bias + a @ bt.T)

The kernels live in ``lib/libayla_b200.so`` (built by ``python -m ayla_b200.build``)
and are reached through the C ABI declared in ``include/ayla_b200.h``.
"""

from .gemm_jit import (
    ACTIVATIONS,
    GemmScheduleSeed,
    gemm_act_mul_op,
    gemm_act_rowmul_op,
    gemm_act_op,
    gemm_jit_compiler,
    gemm_op,
    gemm_op_compiler,
    measured_gemm_configs,
    select_gemm_schedule,
)
from .swiglu import swiglu_op, swiglu_op_compiler
from .torch_custom_call import DEFAULT_NAMESPACE, OperandKind, TensorSpec, make_torch_custom_call

__all__ = [
    "ACTIVATIONS",
    "DEFAULT_NAMESPACE",
    "GemmScheduleSeed",
    "OperandKind",
    "TensorSpec",
    "gemm_act_mul_op",
    "gemm_act_rowmul_op",
    "gemm_act_op",
    "gemm_jit_compiler",
    "gemm_op",
    "gemm_op_compiler",
    "make_torch_custom_call",
    "measured_gemm_configs",
    "select_gemm_schedule",
    "swiglu_op",
    "swiglu_op_compiler",
]
