"""RMSNorm followed by a projection as one row reduction and one GEMM.

``rmsnorm(x) @ W.T`` with ``rmsnorm(x) = x * rsqrt(mean(x^2) + eps) * g`` equals
``r[:, None] * (x @ (W * g).T)`` with ``r = rsqrt(mean(x^2) + eps)``: the norm's weight vector ``g``
moves into the projection weight once (``fold_norm_weight``), and the per-row factor ``r`` is applied
to the fp32 accumulator in the GEMM's epilogue (``gemm_act_rowmul_op``), so the normalised activations
are never written to or read back from memory.  The reference lists epilogue fusion as an aim
(README.md:6-7) and has no kernel of this form.
"""

from __future__ import annotations

import torch

from .gemm_jit import _SHORT_DTYPES, _TORCH_DTYPES, gemm_act_rowmul_op

_DTYPE_NAMES = {torch_dtype: name for name, torch_dtype in _TORCH_DTYPES.items() if name in _SHORT_DTYPES}


def fold_norm_weight(weight: torch.Tensor, norm_weight: torch.Tensor) -> torch.Tensor:
    """``W * g`` along the input features, computed in fp32 and rounded once: ``weight`` is
    ``[out_features, in_features]``, ``norm_weight`` is ``[in_features]``."""
    return (weight.float() * norm_weight.float()).to(weight.dtype)


def rms_norm_linear(x: torch.Tensor, folded_weight: torch.Tensor, eps: float = 1e-5, activation: str = "none",
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """``activation(rmsnorm(x) @ W.T)`` for ``x`` of shape ``[tokens, in_features]`` and
    ``folded_weight = fold_norm_weight(W, g)``.  The row factors are computed in fp32 and handed to
    the kernel in the operands' type; ``activation`` other than ``"none"`` is only equivalent to
    activating the scaled product when it is positively homogeneous (``"relu"``)."""
    if x.dtype not in _DTYPE_NAMES:
        raise ValueError(f"unsupported dtype {x.dtype}")
    if activation not in ("none", "relu"):
        raise ValueError("only 'none' and 'relu' commute with the per-row scale")
    tokens = x.shape[0]
    if out is None:
        out = torch.empty(tokens, folded_weight.shape[0], dtype=x.dtype, device=x.device)
    factors = torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps).to(x.dtype)
    gemm_act_rowmul_op("mm", activation, _DTYPE_NAMES[x.dtype])(x, folded_weight, factors, out)
    return out
