"""mm, addmm and bmm ops backed by the prebuilt sm_100a kernels.

Drop-in for the reference's JIT GEMM front end (ayla/gemm_jit.py): the same
names, signatures and return types --

    op = gemm_op("mm", "bfloat16")      # op(a, bt, out): out = a @ bt.T
    op(a, bt, out)

``gemm_op(operation, dtype)`` returns the cached ``torch.ops.ayla.jit_{op}_{f16|bf16}``
overload taking ``(a, bt, out)``, ``(bias, a, bt, out)`` or the batched
``(a[B,M,K], bt[B,N,K], out[B,M,N])`` (ayla/gemm_jit.py:396-411);
``measured_gemm_configs`` lists the schedules measured on exactly this shape and
``select_gemm_schedule`` picks the one a launch will use (ayla/gemm_jit.py:168-222).
A schedule here is a tile width / CTA pairing / split-K / raster choice for the
tcgen05 kernel rather than a Hopper pass recipe, and "compiling" a shape only
selects one: the kernels are already built into ``libayla_b200.so``.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass
from functools import cache

import torch

from . import _lib
from .gemm_schedule_table import CONFIGS, SCHEDULES
from .jit_compiler import OpTemplate, ShapeSpecializingJITCompiler
from .torch_custom_call import DEFAULT_NAMESPACE, OperandKind, TensorSpec

_SHORT_DTYPES = {"float16": "f16", "bfloat16": "bf16"}
_TORCH_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16}
_OPERATIONS = ("mm", "addmm", "bmm")
ACTIVATIONS = ("none", "relu", "sigmoid", "silu", "gelu", "gelu_tanh")

# Table entries omit default fields.
_DEFAULTS: dict[str, object] = {
    "tile_n": 256,
    "cta_group": 1,
    "swap_ab": 0,
    "split_k": 1,
    "group_m": 8,
    "grid_ctas": 0,
    "l2_hint_a": 0,
    "l2_hint_b": 0,
    "split_tail": 0,
    "l2_prefetch": 0,
    "cluster_split": 0,
    "stream_k": 0,
    "tile_rows": 0,
    "early_prefetch": 0,
}

# A measured schedule is transferred to another shape only when the shapes are
# this close in summed |log2| of (batch, m, n, k); beyond that the shape-aware
# default of the library is the better guess.
_MAX_TRANSFER_DISTANCE = 2.0


@dataclass(frozen=True)
class GemmScheduleSeed:
    captured_config: dict[str, object]
    builder_config: dict[str, object] | None
    adaptations: tuple[str, ...]
    source_shape: tuple[int, int, int] | None
    source_percentage_of_torch: float | None = None
    post_builder_passes: tuple[str, ...] = ()


def _builder_config(captured: dict[str, object]) -> dict[str, object]:
    """The fields the launcher passes to the library (``struct ayla_b200_config``)."""
    return {key: int(captured[key]) for key in _lib.Config.FIELDS}  # type: ignore[arg-type]


def _shape_supported(m: int, n: int, k: int, batch: int) -> bool:
    # 16-byte row pitch for TMA: n and k in multiples of 8 elements.  (The
    # reference needs k % 64 == 0, ayla/gemm_jit.py:134, :234; K tails are
    # zero-filled by TMA here, so multiples of 8 suffice.)
    return min(batch, m, n, k) > 0 and n % 8 == 0 and k % 8 == 0


def _legal(config: dict[str, object], operation: str, dtype: str, m: int, n: int, k: int,
           batch: int) -> bool:
    cfg = _lib.Config.from_dict(config)
    return _lib.config_valid(cfg, operation, dtype, batch, m, n, k)


def _seed(captured: dict[str, object], operation: str, dtype: str, m: int, n: int, k: int,
          batch: int, source: tuple[int, int, int, int], exact: bool) -> GemmScheduleSeed | None:
    if not _shape_supported(m, n, k, batch):
        return None
    if not _legal(captured, operation, dtype, m, n, k, batch):
        return None
    percentage = captured.get("percentage_of_torch")
    return GemmScheduleSeed(
        captured,
        _builder_config(captured),
        () if exact else (f"nearest measured shape {source}",),
        source[1:],
        float(percentage) if isinstance(percentage, (int, float)) else None,
    )


_SM_COUNT = 148


def _waves(config: dict[str, object], batch: int, m: int, n: int) -> int:
    """Passes of the persistent grid a schedule needs on this shape (whole CTAs or clusters at
    a time).  A schedule measured at one wave is a poor guess for a shape where it needs two."""
    pair = int(config["cta_group"])
    rows, cols = (n, m) if config["swap_ab"] else (m, n)
    tile_rows = int(config["tile_rows"]) or 128
    row_tiles = -(-rows // (tile_rows if config["swap_ab"] else 128 * pair))
    tiles = batch * row_tiles * -(-cols // int(config["tile_n"]))
    split = int(config["split_k"])
    if config["cluster_split"]:
        cluster = split * pair
        return -(-tiles // max(1, _SM_COUNT // cluster))
    units = tiles * (1 if config["split_tail"] else split)
    return -(-units // (_SM_COUNT // pair))


def _column_padding(config: dict[str, object], m: int, n: int) -> float:
    """Share of a schedule's tile columns that lie past the matrix on this shape (the swapped form
    tiles the token dimension): a 128-column tile on 64 output columns computes half of itself for
    nothing, however well it did where it was measured on 128."""
    cols = m if config["swap_ab"] else n
    tile = int(config["tile_n"])
    padded = -(-cols // tile) * tile
    return (padded - cols) / padded


def measured_gemm_configs(operation: str, dtype: str, m: int, n: int, k: int,
                          batch: int = 1) -> tuple[dict[str, object], ...]:
    """All schedules measured on exactly this shape, winner first, as fresh copies."""
    indices = SCHEDULES.get((operation, dtype), {}).get((batch, m, n, k), ())
    return tuple({**_DEFAULTS, **CONFIGS[index]} for index in indices)


def select_gemm_schedule(operation: str, dtype: str, m: int, n: int, k: int,
                         batch: int = 1) -> GemmScheduleSeed | None:
    """The schedule a launch of this shape uses, or ``None`` if the shape is unsupported.

    An exact table hit has empty ``adaptations``; a schedule transferred from a
    nearby measured shape names that shape; otherwise the library's shape-aware
    default is returned with ``source_shape`` ``None``.
    """
    if min(batch, m, n, k) <= 0 or operation not in _OPERATIONS:
        return None
    if dtype not in _SHORT_DTYPES:
        return None
    # fp16 and bf16 run the same kernels at the same speed: a shape measured only in one serves the other
    other = "float16" if dtype == "bfloat16" else "bfloat16"
    table = {**SCHEDULES.get((operation, other), {}), **SCHEDULES.get((operation, dtype), {})}
    if not _shape_supported(m, n, k, batch):
        return None
    query = (batch, m, n, k)

    def distance(shape: tuple[int, int, int, int]) -> float:
        return sum(abs(math.log2(a) - math.log2(b)) for a, b in zip(shape, query, strict=True))

    for shape in sorted(table, key=distance):
        if distance(shape) > _MAX_TRANSFER_DISTANCE:
            break
        for index in table[shape]:
            captured = {**_DEFAULTS, **CONFIGS[index]}
            if shape != query and _waves(captured, batch, m, n) > _waves(captured, shape[0], shape[1], shape[2]):
                continue  # it would no longer fit the number of waves it was measured at
            if shape != query:
                waste = _column_padding(captured, m, n)
                if waste >= 0.34 and waste > _column_padding(captured, shape[1], shape[2]) + 0.2:
                    continue  # its tiles would be a third or more padding here and were not where it was measured
            seed = _seed(captured, operation, dtype, m, n, k, batch, shape, exact=shape == query)
            if seed is not None:
                if shape not in SCHEDULES.get((operation, dtype), {}):
                    seed = GemmScheduleSeed(seed.captured_config, seed.builder_config,
                                            (*seed.adaptations, f"measured in {other}"), seed.source_shape,
                                            seed.source_percentage_of_torch)
                return seed
    return _fallback_schedule(operation, dtype, m, n, k, batch)


def _fallback_schedule(operation: str, dtype: str, m: int, n: int, k: int,
                       batch: int = 1) -> GemmScheduleSeed | None:
    """Unmeasured schedule from the library's heuristic (ayla_b200_default_config)."""
    if not _shape_supported(m, n, k, batch) or dtype not in _SHORT_DTYPES:
        return None
    if operation not in _OPERATIONS or (operation != "bmm" and batch != 1):
        return None
    captured = {**_DEFAULTS, **_lib.default_config(operation, dtype, batch, m, n, k).to_dict()}
    return GemmScheduleSeed(
        captured,
        _builder_config(captured),
        ("unmeasured shape-aware default schedule",),
        None,
        None,
    )


class GemmLauncher:
    """One specialised ``(operation, dtype, shape, device)`` launch.

    Owns the split-K workspaces and the status word of its shape.  The workspace of the
    stream that is current at specialisation time is allocated here, so that a launch
    itself allocates nothing and can be captured in a CUDA graph.  A launch on another
    stream gets a workspace of its own the first time that stream is used (two launches
    of one shape that overlap on different streams would otherwise sum into each other's
    partial tiles); that first use allocates, so it must happen outside graph capture --
    inside capture it raises ``RuntimeError`` as a first call of a new shape does.

    The status word lives in pinned host memory (``_lib.StatusWord``): every call reads it
    before launching, without synchronising, and raises ``RuntimeError`` if an earlier
    launch of this shape ran into one of the kernel's bounded waits; the split-K arrival
    counters that launch may have left dirty are cleared first, so the call after the
    error is correct again.  ``check_status()`` does the same after a synchronise, and
    ``AYLA_B200_DEBUG=1`` calls it after every launch.
    """

    def __init__(self, operation: str, dtype: str, batch: int, m: int, n: int, k: int,
                 seed: GemmScheduleSeed, device: torch.device, activation: str = "none",
                 gated: bool | str = False):
        assert seed.builder_config is not None
        self.operation, self.dtype, self.activation, self.gated = operation, dtype, activation, gated
        self.batch, self.m, self.n, self.k = batch, m, n, k
        self.seed = seed
        self.device = device
        self.config = _lib.Config.from_dict(seed.builder_config)
        index = device.index if device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(index):
            _lib.init(index)
        need = _lib.workspace_bytes(self.config, operation, batch, m, n, k)
        self._ws_bytes = need
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=device) if need else None
        self.status = _lib.StatusWord()
        self._ws_ptr = self.workspace.data_ptr() if self.workspace is not None else 0
        self._status_ptr = self.status.ptr
        # stream handle -> (workspace tensor, argument tail); the first entry serves the stream current now
        with torch.cuda.device(index):
            self._home_stream = torch.cuda.current_stream().cuda_stream if need else None
        self._per_stream: dict[int, tuple[torch.Tensor, tuple]] = {}
        self._debug = bool(os.environ.get("AYLA_B200_DEBUG"))
        # Everything that does not change from call to call, converted for the C call once.
        import ctypes

        lib = _lib.load()
        self._entry = lib.ayla_b200_gemm_act_rowmul if gated == "row" else lib.ayla_b200_gemm_act_mul
        self._head = (_lib.OP_CODES[operation], _lib.DTYPE_CODES[dtype], _lib.ACT_CODES[activation])
        self._tail = (batch, m, n, k, ctypes.byref(self.config), self._ws_ptr or None,
                      self.workspace.numel() if self.workspace is not None else 0, self._status_ptr)
        self._has_bias = operation == "addmm"
        self._device_index = index

    def __call__(self, *tensors: torch.Tensor) -> None:
        bias_ptr = mul_ptr = None
        if self._has_bias:
            bias_ptr = tensors[0].data_ptr()
            tensors = tensors[1:]
        if self.gated:
            a, bt, mul, out = tensors
            mul_ptr = mul.data_ptr()
        else:
            a, bt, out = tensors
        if self.status.peek():
            self._report_timeout()
        stream = torch.cuda.current_stream(self._device_index).cuda_stream
        tail = self._tail
        if self._ws_bytes and stream != self._home_stream:
            tail = self._tail_for_stream(stream)
        # The library launches on the current device (the reference's launcher guards the device
        # the same way, ayla/ptx_runtime.py:268-275).
        if torch.cuda.current_device() != self._device_index:
            with torch.cuda.device(self._device_index):
                code = self._entry(*self._head, bias_ptr, a.data_ptr(), bt.data_ptr(), mul_ptr, out.data_ptr(),
                                   *tail, stream)
        else:
            code = self._entry(*self._head, bias_ptr, a.data_ptr(), bt.data_ptr(), mul_ptr, out.data_ptr(),
                               *tail, stream)
        if code:
            _lib.check(code)
        if self._debug:
            self.check_status()

    def _tail_for_stream(self, stream: int) -> tuple:
        """The call arguments with the workspace that belongs to ``stream`` (allocated on first use)."""
        entry = self._per_stream.get(stream)
        if entry is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(
                    f"jit_{self.operation}: the first launch of this k-split shape on a new stream allocates its "
                    "workspace and cannot happen during CUDA graph capture; run it once on that stream before capturing")
            workspace = torch.zeros(self._ws_bytes, dtype=torch.uint8, device=self.device)
            batch, m, n, k, cfg, _, size, status = self._tail
            entry = (workspace, (batch, m, n, k, cfg, workspace.data_ptr(), size, status))
            self._per_stream[stream] = entry
        return entry[1]

    def _report_timeout(self) -> None:
        code = self.status.peek()
        with torch.cuda.device(self._device_index):
            torch.cuda.current_stream().synchronize()  # nothing of the failed launch is still running
            if self.workspace is not None:
                self.workspace.zero_()  # arrival counters a timed-out k-split leaves behind
            for workspace, _ in self._per_stream.values():
                workspace.zero_()
        self.status.clear()
        raise RuntimeError(
            f"jit_{self.operation}: device wait timed out (code {code & 0xFF}, CTA {code >> 8})"
        )

    def check_status(self) -> None:
        """Synchronise and raise if one of the kernel's bounded waits gave up."""
        torch.cuda.synchronize(self._device_index)
        if self.status.peek():
            self._report_timeout()


def _op_name(operation: str, dtype: str, activation: str = "none", gated: bool | str = False) -> str:
    middle = ("" if activation == "none" else f"_{activation}") + {False: "", True: "_mul", "row": "_rowmul"}[gated]
    return f"jit_{operation}{middle}_{_SHORT_DTYPES[dtype]}"


def _template(operation: str, dtype: str, activation: str = "none", gated: bool | str = False) -> OpTemplate:
    torch_dtype = _TORCH_DTYPES[dtype]
    rank = 3 if operation == "bmm" else 2
    tensor = TensorSpec(torch_dtype, (None,) * rank)
    signature = (tensor,) * (4 if gated else 3)  # a, bt, [mul,] out
    if operation == "addmm":
        signature = (TensorSpec(torch_dtype, (None,)), *signature)
    return OpTemplate(_op_name(operation, dtype, activation, gated), signature)


def gemm_jit_compiler(operation: str, dtype: str, activation: str = "none",
                      gated: bool | str = False) -> ShapeSpecializingJITCompiler:
    """Per-shape dispatcher for one op: validates operands, picks the schedule once
    per ``(device, shapes)`` and launches (ayla/gemm_jit.py:339-393).  ``activation``
    (one of ``ACTIVATIONS``) is fused into the epilogue; with ``gated`` the op takes one more
    operand ``mul`` (shaped like ``out``, before it) and writes ``activation(...) * mul``; with
    ``gated="row"`` that operand is one factor per output row, shaped ``(..., m, 1)``."""
    if gated not in (False, True, "row"):
        raise ValueError(f"unsupported gate {gated!r}")
    if operation not in _OPERATIONS:
        raise ValueError(f"unsupported GEMM operation {operation}")
    if dtype not in _SHORT_DTYPES:
        raise ValueError(f"unsupported GEMM dtype {dtype}")
    if activation not in ACTIVATIONS:
        raise ValueError(f"unsupported GEMM activation {activation}")
    template = _template(operation, dtype, activation, gated)

    def compile_specialization(bound: OpTemplate, device: torch.device) -> GemmLauncher:
        sizes = [spec.sizes for spec in bound.signature]
        mul = sizes.pop(-2) if gated else None
        *bias, a, bt, out = sizes
        *batch, m, k = a
        n = bt[-2]
        lead = tuple(batch)
        if tuple(bt) != (*lead, n, k):
            raise ValueError(
                f"{bound.name}: bt must be {(*lead, n, k)} for a of shape {tuple(a)} "
                f"(out = a @ bt.T), got {tuple(bt)}"
            )
        if tuple(out) != (*lead, m, n):
            raise ValueError(f"{bound.name}: out must be {(*lead, m, n)}, got {tuple(out)}")
        if bias and tuple(bias[0]) != (n,):
            raise ValueError(f"{bound.name}: bias must be ({n},), got {tuple(bias[0])}")
        if gated == "row" and tuple(mul) != (*lead, m, 1):
            raise ValueError(f"{bound.name}: the row factors must be {(*lead, m, 1)}, got {tuple(mul)}")
        if gated is True and tuple(mul) != tuple(out):
            raise ValueError(f"{bound.name}: mul must have the shape of out {tuple(out)}, got {tuple(mul)}")
        schedule = select_gemm_schedule(operation, dtype, m, n, k, *batch)
        if schedule is None:
            raise ValueError(f"{bound.name}: no schedule for {operation} {lead}x{m}x{n}x{k}")
        return GemmLauncher(operation, dtype, batch[0] if batch else 1, m, n, k, schedule, device, activation, gated)

    return ShapeSpecializingJITCompiler(template, compile_specialization)


_COMPILERS: dict[tuple[str, str, str], ShapeSpecializingJITCompiler] = {}


def gemm_op(operation: str, dtype: str, namespace: str = DEFAULT_NAMESPACE) -> torch._ops.OpOverload:
    """Torch op ``(bias?, a, bt, out) -> ()`` writing ``out = [bias +] a @ bt^T``.

    Cached: the same overload object is returned for the same arguments."""
    return _gemm_op(operation, dtype, namespace)


@cache
def _gemm_op(operation: str, dtype: str, namespace: str) -> torch._ops.OpOverload:
    from .torch_custom_call import make_torch_custom_call

    compiler = gemm_jit_compiler(operation, dtype)
    _COMPILERS[(operation, dtype, namespace)] = compiler
    inputs = 3 if operation == "addmm" else 2
    return make_torch_custom_call(compiler, [OperandKind.R] * inputs + [OperandKind.RW],
                                  namespace=namespace)


def gemm_op_compiler(operation: str, dtype: str,
                     namespace: str = DEFAULT_NAMESPACE) -> ShapeSpecializingJITCompiler:
    """The dispatcher behind ``gemm_op(operation, dtype, namespace)`` (for its cache
    size and the launchers' status words)."""
    gemm_op(operation, dtype, namespace)
    return _COMPILERS[(operation, dtype, namespace)]


def gemm_act_mul_op(operation: str, activation: str, dtype: str,
                    namespace: str = DEFAULT_NAMESPACE) -> torch._ops.OpOverload:
    """Torch op ``(bias?, a, bt, mul, out) -> ()`` writing ``out = activation([bias +] a @ bt^T) * mul``
    with ``mul`` shaped like ``out``, named ``jit_{operation}[_{activation}]_mul_{f16|bf16}``: a gated
    projection (``sigmoid(x @ Wg^T) * v``) in one kernel, the product taken in fp32 before the single
    rounding.  The reference recognises this producer region in compiled graphs
    (ayla/torch_compile.py:288-504) but has no kernel for it."""
    return _gemm_act_mul_op(operation, activation, dtype, namespace)


@cache
def _gemm_act_mul_op(operation: str, activation: str, dtype: str, namespace: str) -> torch._ops.OpOverload:
    from .torch_custom_call import make_torch_custom_call

    compiler = gemm_jit_compiler(operation, dtype, activation, gated=True)
    _COMPILERS[(f"{operation}_{activation}_mul", dtype, namespace)] = compiler
    inputs = 4 if operation == "addmm" else 3
    return make_torch_custom_call(compiler, [OperandKind.R] * inputs + [OperandKind.RW],
                                  namespace=namespace)


def gemm_act_rowmul_op(operation: str, activation: str, dtype: str,
                       namespace: str = DEFAULT_NAMESPACE) -> torch._ops.OpOverload:
    """Torch op ``(bias?, a, bt, row_mul, out) -> ()`` writing
    ``out = activation([bias +] a @ bt^T) * row_mul`` with ``row_mul`` shaped ``(..., m, 1)`` (one factor
    per output row, as a ``keepdim`` reduction over the rows of ``a`` leaves it), named
    ``jit_{operation}[_{activation}]_rowmul_{f16|bf16}``.  With no activation and no bias it is a GEMM
    whose left operand carries a per-row scale: an RMSNorm followed by a projection becomes one row
    reduction and this op once the norm's weight vector is folded into ``bt``, because
    ``(x * r[:, None] * g) @ W.T == r[:, None] * (x @ (W * g).T)``.  The reference lists epilogue
    fusion as an aim (README.md:6-7) and has no kernel of this form."""
    return _gemm_act_rowmul_op(operation, activation, dtype, namespace)


@cache
def _gemm_act_rowmul_op(operation: str, activation: str, dtype: str, namespace: str) -> torch._ops.OpOverload:
    from .torch_custom_call import make_torch_custom_call

    compiler = gemm_jit_compiler(operation, dtype, activation, gated="row")
    _COMPILERS[(f"{operation}+{activation}+rowmul", dtype, namespace)] = compiler
    inputs = 4 if operation == "addmm" else 3
    return make_torch_custom_call(compiler, [OperandKind.R] * inputs + [OperandKind.RW], namespace=namespace)


def gemm_act_op(operation: str, activation: str, dtype: str,
                namespace: str = DEFAULT_NAMESPACE) -> torch._ops.OpOverload:
    """Torch op ``(bias?, a, bt, out) -> ()`` writing ``out = activation([bias +] a @ bt^T)``,
    named ``jit_{operation}_{activation}_{f16|bf16}``; the activation is evaluated on the fp32
    accumulator before the single rounding.  The reference has one such kernel, a fixed
    4096-cube matmul + sigmoid (ayla/gemm_collection/auto_matmul_4096_wgmma256_wg_sigmoid.py:22-142);
    this is the same fusion for every shape, operation and activation in ``ACTIVATIONS``.
    ``activation="none"`` returns ``gemm_op(operation, dtype)``."""
    if activation == "none":
        return gemm_op(operation, dtype, namespace)
    return _gemm_act_op(operation, activation, dtype, namespace)


@cache
def _gemm_act_op(operation: str, activation: str, dtype: str, namespace: str) -> torch._ops.OpOverload:
    from .torch_custom_call import make_torch_custom_call

    compiler = gemm_jit_compiler(operation, dtype, activation)
    _COMPILERS[(f"{operation}_{activation}", dtype, namespace)] = compiler
    inputs = 3 if operation == "addmm" else 2
    return make_torch_custom_call(compiler, [OperandKind.R] * inputs + [OperandKind.RW],
                                  namespace=namespace)
