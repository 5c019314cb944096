"""CPU oracle for the GEMM hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (``ayla_b200/``) imports this module; it is used by
``tests/``, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline and
``--impl reference`` legs, always as the checker or the thing timed as a
baseline, never as a fallback.

What it restates.  The reference has no CPU implementation of the contraction;
its kernels are Hopper PTX and its own tests define correctness against PyTorch:
``a @ bt.transpose(-1, -2)`` and ``torch.addmm(bias, a, bt.T)``
(tests/test_gemm_jit.py:59-63), ``torch.mm(a.float(), b.float().t())`` cast to the
output type (tests/gemm_collection/test_correctness.py:419), and
``torch_mm_nt / addmm_nt / bmm_nt`` (benchmarks/common.py:184-198).  The arithmetic
therefore lives in a third-party dependency, PyTorch (pyproject.toml:10-14, unpinned;
torch 2.11.0 here).  The functions below follow the kernel semantics the reference
defines around that call:

* operand convention ``out = [bias +] a @ bt^T``, bias broadcast over rows and added
  to the fp32 accumulator before rounding, bmm per batch (ayla/gemm_jit.py:267-307);
* fp32 accumulation and ONE round-to-nearest-even to the output type
  (ayla/passes/lower_to_ptx_template.py:134-149);
* silu / sigmoid / mul evaluated on the fp32 accumulator before that rounding
  (ayla/passes/lower_to_ptx_template.py:84-113, :296-315, :62-81).

Pinned by ``tests/golden/`` (vectors generated in a container that holds the
reference, script committed beside them) and cross-checked against the plain-C
restatement in ``oracle/gemm_ref.c`` (fp64 accumulation).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

TORCH_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16}

# Tolerances of the project (stated with the benchmark configs): Frobenius
# relative error and max elementwise error relative to rms(ref), both against the
# CPU fp32 result rounded to the output type.
FRO_REL_TOL = 5e-3
MAX_OVER_RMS_TOL = 2e-2


# --------------------------------------------------------------------- reference math

def mm_ref32(a: torch.Tensor, bt: torch.Tensor) -> torch.Tensor:
    """fp32 ``a @ bt^T`` on CPU (tests/gemm_collection/test_correctness.py:419)."""
    return torch.mm(a.float(), bt.float().t())


def addmm_ref32(bias: torch.Tensor, a: torch.Tensor, bt: torch.Tensor) -> torch.Tensor:
    """fp32 ``bias + a @ bt^T``; bias enters before rounding (ayla/gemm_jit.py:280-283)."""
    return torch.addmm(bias.float(), a.float(), bt.float().t())


def bmm_ref32(a: torch.Tensor, bt: torch.Tensor) -> torch.Tensor:
    """fp32 per-batch ``a @ bt^T`` (ayla/gemm_jit.py:284-304)."""
    return torch.bmm(a.float(), bt.float().transpose(1, 2))


def swiglu_ref32(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """fp32 ``silu(x @ w_gate^T) * (x @ w_up^T)`` with no intermediate rounding
    (ayla/passes/lower_to_ptx_template.py:296-315 for silu, :62-81 for mul)."""
    xf = x.float()
    return F.silu(torch.mm(xf, w_gate.float().t())) * torch.mm(xf, w_up.float().t())


def act_ref32(activation: str, x32: torch.Tensor) -> torch.Tensor:
    """The fused-epilogue activations on an fp32 result, before any rounding
    (ayla/passes/lower_to_ptx_template.py:84-113 evaluates its sigmoid the same way)."""
    if activation == "none":
        return x32
    if activation == "relu":
        return torch.relu(x32)
    if activation == "sigmoid":
        return torch.sigmoid(x32)
    if activation == "silu":
        return F.silu(x32)
    if activation == "gelu":
        return F.gelu(x32)
    if activation == "gelu_tanh":
        return F.gelu(x32, approximate="tanh")
    raise ValueError(f"unknown activation {activation}")


def gemm_ref32(operation: str, *tensors: torch.Tensor) -> torch.Tensor:
    if operation == "mm":
        return mm_ref32(*tensors)
    if operation == "addmm":
        return addmm_ref32(*tensors)
    if operation == "bmm":
        return bmm_ref32(*tensors)
    if operation == "swiglu":
        return swiglu_ref32(*tensors)
    raise ValueError(f"unknown operation {operation}")


def gemm_ref(operation: str, dtype: torch.dtype, *tensors: torch.Tensor) -> torch.Tensor:
    """The oracle result: fp32 math, one rounding to ``dtype``."""
    return gemm_ref32(operation, *tensors).to(dtype)


# --------------------------------------------------------------------- seeded inputs

def _normal(gen: torch.Generator, shape, std: float, dtype: torch.dtype) -> torch.Tensor:
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * std).to(dtype)


def make_inputs(config: str, dtype: str = "bfloat16", scale_down: int = 1) -> tuple[str, tuple[torch.Tensor, ...]]:
    """Seeded CPU inputs of a benchmark config, generated in fp32 and cast, so the
    oracle and the GPU kernel see bit-identical operands.

    ``1/K``-style second parameters of the config descriptions are variances
    (std = K**-0.5); bare decimals (0.02, 0.1) are standard deviations.
    ``scale_down`` divides the large extents for quick tests (distributions keep
    the full-size K scaling).
    """
    td = TORCH_DTYPES[dtype]
    s = scale_down

    def gen(seed: int) -> torch.Generator:
        g = torch.Generator(device="cpu")
        g.manual_seed(seed)
        return g

    if config == "C1":  # mm 4096^3, N(0,1)
        g = gen(0)
        n = 4096 // s
        return "mm", (_normal(g, (n, n), 1.0, td), _normal(g, (n, n), 1.0, td))
    if config == "C2a":  # addmm 8192x768x768
        g = gen(1)
        m = 8192 // s
        a = _normal(g, (m, 768), 1.0, td)
        bt = _normal(g, (768, 768), 768 ** -0.5, td)
        bias = _normal(g, (768,), 0.1, td)
        return "addmm", (bias, a, bt)
    if config == "C2b":  # addmm split-K 256x1024x16384
        g = gen(2)
        k = 16384 // s
        a = _normal(g, (256, k), 1.0, td)
        bt = _normal(g, (1024, k), 16384 ** -0.5, td)
        bias = _normal(g, (1024,), 0.1, td)
        return "addmm", (bias, a, bt)
    if config == "C3a":  # bmm 64 x [2048x128]·[2048x128]^T
        g = gen(3)
        b = max(1, 64 // s)
        return "bmm", (_normal(g, (b, 2048, 128), 1.0, td), _normal(g, (b, 2048, 128), 1.0, td))
    if config == "C3b":  # bmm 64 x [2048x2048]·[128x2048]^T, a ~ U(0, 1/2048)
        g = gen(4)
        b = max(1, 64 // s)
        a = (torch.rand((b, 2048, 2048), generator=g, dtype=torch.float32) / 2048.0).to(td)
        return "bmm", (a, _normal(g, (b, 128, 2048), 1.0, td))
    if config == "C4":  # SwiGLU 8192 x 14336 x 4096
        g = gen(5)
        m, n = 8192 // s, 14336 // s
        x = _normal(g, (m, 4096), 1.0, td)
        return "swiglu", (x, _normal(g, (n, 4096), 0.02, td), _normal(g, (n, 4096), 0.02, td))
    raise ValueError(f"unknown config {config}")


SWEEP_M = (1, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384)
SWEEP_NK = ((4096, 4096), (14336, 4096), (4096, 14336))


def make_sweep_inputs(index: int, dtype: str = "bfloat16") -> tuple[tuple[int, int, int], tuple[torch.Tensor, torch.Tensor]]:
    """Point ``index`` of the dynamic-M sweep: seed 100 + index, a and bt ~ N(0, 1/K)."""
    m = SWEEP_M[index % len(SWEEP_M)]
    n, k = SWEEP_NK[index // len(SWEEP_M)]
    g = torch.Generator(device="cpu")
    g.manual_seed(100 + index)
    td = TORCH_DTYPES[dtype]
    return (m, n, k), (_normal(g, (m, k), k ** -0.5, td), _normal(g, (n, k), k ** -0.5, td))


# --------------------------------------------------------------------------- metrics

@dataclass
class Parity:
    fro_rel: float
    max_over_rms: float
    over_bound: int          # elements with |out - ref| > MAX_OVER_RMS_TOL * rms(ref)
    over_bound_one_ulp: int  # ... of which out is within 1 ulp (of the output type) of ref
    max_half_ulps_vs_fp32: float  # max |out - ref32| in units of half an output ulp at ref32
    nonfinite: int
    elements: int

    @property
    def ok(self) -> bool:
        """Within tolerance.  The elementwise bound is tighter than one output ulp
        in the top binade of some configs (an ulp at |v| >= 4*rms is 0.031*rms in
        bf16), so an element that misses it while being the neighbouring
        representable value of a correctly computed fp32 sum is a rounding flip,
        not an error; it is counted and reported, and accepted."""
        return (
            self.nonfinite == 0
            and self.fro_rel <= FRO_REL_TOL
            and (self.max_over_rms <= MAX_OVER_RMS_TOL or self.over_bound == self.over_bound_one_ulp)
        )


def _ulp(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Spacing of ``dtype`` at |x| (x fp32)."""
    mant = 7 if dtype == torch.bfloat16 else 10
    min_exp = -126 if dtype == torch.bfloat16 else -14
    e = torch.floor(torch.log2(x.abs().clamp_min(2.0 ** min_exp)))
    return torch.pow(2.0, e - mant)


def compare(out: torch.Tensor, ref32: torch.Tensor) -> Parity:
    """Compare a kernel result (output dtype, any device) with the fp32 oracle result."""
    dtype = out.dtype
    o = out.detach().to("cpu").float().reshape(-1)
    r32 = ref32.detach().to("cpu").float().reshape(-1)
    r = r32.to(dtype).float()
    nonfinite = int((~torch.isfinite(o)).sum())
    diff = (o - r).abs()
    rms = float(r.double().pow(2).mean().sqrt())
    ref_norm = float(r.double().norm())
    fro = float((o - r).double().norm()) / ref_norm if ref_norm > 0 else float(diff.max())
    bound = MAX_OVER_RMS_TOL * rms
    over = diff > bound
    ulp = _ulp(r, dtype)
    one_ulp = over & (diff <= ulp * 1.0001)
    half_ulps = ((o - r32).abs() / (0.5 * _ulp(r32, dtype))).max()
    return Parity(
        fro_rel=fro,
        max_over_rms=float(diff.max()) / rms if rms > 0 else float(diff.max()),
        over_bound=int(over.sum()),
        over_bound_one_ulp=int(one_ulp.sum()),
        max_half_ulps_vs_fp32=float(half_ulps),
        nonfinite=nonfinite,
        elements=o.numel(),
    )


def flops(operation: str, batch: int, m: int, n: int, k: int) -> float:
    return (4.0 if operation == "swiglu" else 2.0) * batch * m * n * k


def algorithmic_bytes(operation: str, batch: int, m: int, n: int, k: int) -> float:
    """Bytes a launch must move: every operand and the output once, 2 bytes each."""
    if operation == "swiglu":
        return 2.0 * (m * k + 2 * n * k + m * n)
    extra = n if operation == "addmm" else 0
    return 2.0 * (batch * (m * k + n * k + m * n) + extra)
