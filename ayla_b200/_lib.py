"""ctypes loader for ``libayla_b200.so`` and typed wrappers of its C ABI.

This is the counterpart of the reference's PTX launcher runtime
(ayla/ptx_runtime.py:26-296, :333-446): where that module JIT-loads PTX through a
``load_inline`` shim, this one ``dlopen``s a prebuilt sm_100a library whose entry
points are declared in ``include/ayla_b200.h``.  There is no fallback: if the
library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

OP_CODES = {"mm": 0, "addmm": 1, "bmm": 2}
DTYPE_CODES = {"float16": 0, "bfloat16": 1}

E_INVALID, E_UNSUPPORTED, E_WORKSPACE, E_CUDA, E_NOT_INIT = 1, 2, 3, 4, 5

EXPORTS = (
    "ayla_b200_init",
    "ayla_b200_gemm",
    "ayla_b200_gemm_act",
    "ayla_b200_gemm_act_mul",
    "ayla_b200_gemm_act_rowmul",
    "ayla_b200_gemm_static_scratch",
    "ayla_b200_swiglu",
    "ayla_b200_default_config",
    "ayla_b200_config_valid",
    "ayla_b200_workspace_bytes",
    "ayla_b200_workspace_counter_bytes",
    "ayla_b200_copy_2d",
    "ayla_b200_kernel_count",
    "ayla_b200_kernel_info",
    "ayla_b200_set_wait_timeout_ms",
    "ayla_b200_debug_set_flags",
    "ayla_b200_set_launch_overlap",
    "ayla_b200_last_error",
    "ayla_b200_version",
)


class Config(ctypes.Structure):
    """Mirror of ``struct ayla_b200_config``."""

    _fields_ = [
        ("tile_n", ctypes.c_int32),
        ("cta_group", ctypes.c_int32),
        ("swap_ab", ctypes.c_int32),
        ("split_k", ctypes.c_int32),
        ("group_m", ctypes.c_int32),
        ("grid_ctas", ctypes.c_int32),
        ("l2_hint_a", ctypes.c_int32),
        ("l2_hint_b", ctypes.c_int32),
        ("split_tail", ctypes.c_int32),
        ("l2_prefetch", ctypes.c_int32),
        ("cluster_split", ctypes.c_int32),
        ("stream_k", ctypes.c_int32),
        ("tile_rows", ctypes.c_int32),
        ("early_prefetch", ctypes.c_int32),
    ]

    FIELDS = tuple(name for name, _ in _fields_)

    @classmethod
    def from_dict(cls, values: dict) -> "Config":
        cfg = cls(tile_n=256, cta_group=1, swap_ab=0, split_k=1, group_m=8, grid_ctas=0,
                  l2_hint_a=0, l2_hint_b=0, split_tail=0, l2_prefetch=0, cluster_split=0, stream_k=0, tile_rows=0,
                  early_prefetch=0)
        for key in cls.FIELDS:
            if key in values and values[key] is not None:
                setattr(cfg, key, int(values[key]))
        return cfg

    def to_dict(self) -> dict:
        return {key: int(getattr(self, key)) for key in self.FIELDS}


class AylaB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


_lock = threading.Lock()
_lib: ctypes.CDLL | None = None
_initialised_devices: set[int] = set()


def library_path() -> Path:
    override = os.environ.get("AYLA_B200_LIB")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / "lib" / "libayla_b200.so"


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if not path.exists():
            raise ImportError(
                f"{path} not found: build it with `python -m ayla_b200.build` "
                "(there is no non-CUDA fallback)"
            )
        lib = ctypes.CDLL(str(path))
        i32, i64, vp, sz = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t
        cfgp = ctypes.POINTER(Config)
        lib.ayla_b200_init.argtypes = [i32]
        lib.ayla_b200_init.restype = i32
        lib.ayla_b200_gemm.argtypes = [i32, i32, vp, vp, vp, vp, i64, i64, i64, i64, cfgp, vp, sz, vp, vp]
        lib.ayla_b200_gemm.restype = i32
        lib.ayla_b200_gemm_act.argtypes = [i32, i32, i32, vp, vp, vp, vp, i64, i64, i64, i64, cfgp, vp, sz, vp, vp]
        lib.ayla_b200_gemm_act.restype = i32
        lib.ayla_b200_gemm_act_mul.argtypes = [i32, i32, i32, vp, vp, vp, vp, vp, i64, i64, i64, i64, cfgp, vp, sz, vp, vp]
        lib.ayla_b200_gemm_act_mul.restype = i32
        lib.ayla_b200_gemm_act_rowmul.argtypes = lib.ayla_b200_gemm_act_mul.argtypes
        lib.ayla_b200_gemm_act_rowmul.restype = i32
        lib.ayla_b200_gemm_static_scratch.argtypes = [i32, i32, vp, vp, vp, vp, i64, i64, i64, i64, cfgp, vp, vp]
        lib.ayla_b200_gemm_static_scratch.restype = i32
        lib.ayla_b200_swiglu.argtypes = [i32, vp, vp, vp, vp, i64, i64, i64, cfgp, vp, vp]
        lib.ayla_b200_swiglu.restype = i32
        lib.ayla_b200_default_config.argtypes = [i32, i32, i64, i64, i64, i64, cfgp]
        lib.ayla_b200_default_config.restype = i32
        lib.ayla_b200_config_valid.argtypes = [cfgp, i32, i32, i64, i64, i64, i64]
        lib.ayla_b200_config_valid.restype = i32
        lib.ayla_b200_workspace_bytes.argtypes = [cfgp, i32, i64, i64, i64, i64]
        lib.ayla_b200_workspace_bytes.restype = sz
        lib.ayla_b200_workspace_counter_bytes.argtypes = [cfgp, i32, i64, i64, i64, i64]
        lib.ayla_b200_workspace_counter_bytes.restype = sz
        lib.ayla_b200_copy_2d.argtypes = [vp, sz, vp, sz, sz, sz, vp]
        lib.ayla_b200_copy_2d.restype = i32
        lib.ayla_b200_kernel_count.argtypes = []
        lib.ayla_b200_kernel_count.restype = i32
        i32p = ctypes.POINTER(ctypes.c_int32)
        lib.ayla_b200_kernel_info.argtypes = [i32, i32p, i32p, i32p, i32p, i32p, i32p]
        lib.ayla_b200_kernel_info.restype = i32
        lib.ayla_b200_set_wait_timeout_ms.argtypes = [i64]
        lib.ayla_b200_set_wait_timeout_ms.restype = None
        lib.ayla_b200_debug_set_flags.argtypes = [i32]
        lib.ayla_b200_debug_set_flags.restype = None
        lib.ayla_b200_set_launch_overlap.argtypes = [i32]
        lib.ayla_b200_set_launch_overlap.restype = None
        lib.ayla_b200_last_error.argtypes = []
        lib.ayla_b200_last_error.restype = ctypes.c_char_p
        lib.ayla_b200_version.argtypes = []
        lib.ayla_b200_version.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def last_error() -> str:
    return (load().ayla_b200_last_error() or b"").decode()


def check(code: int) -> None:
    """Map a C status code to the exception types the reference raises:
    ``ValueError`` for argument/shape problems (ayla/jit_compiler.py:76-93,
    ayla/gemm_jit.py:378-381) and ``RuntimeError`` for CUDA failures
    (ayla/ptx_runtime.py:41-49)."""
    if code == 0:
        return
    message = last_error()
    if code in (E_INVALID, E_UNSUPPORTED, E_WORKSPACE):
        raise ValueError(message)
    raise AylaB200Error(code, message)


class StatusWord:
    """The status word of a launcher: a uint32 in pinned host memory that the kernels write
    through its device mapping (under unified addressing pinned host memory has the same
    address on the device) and the host reads without synchronising.  A kernel whose bounded
    wait gave up leaves a non-zero code there; the launcher looks at the word before its next
    launch, so a timed-out launch is reported at the next call of that shape instead of
    silently poisoning later ones."""

    def __init__(self):
        import torch

        self.tensor = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.ptr = self.tensor.data_ptr()
        self._word = ctypes.c_uint32.from_address(self.ptr)

    def peek(self) -> int:
        """The current value, read from host memory: no device synchronisation."""
        return self._word.value

    def clear(self) -> None:
        self._word.value = 0


def init(device: int) -> None:
    """Per-device set-up; must first happen outside CUDA-graph capture."""
    if device in _initialised_devices:
        return
    check(load().ayla_b200_init(int(device)))
    _initialised_devices.add(device)


def version() -> str:
    return load().ayla_b200_version().decode()


def kernel_variants() -> list[dict]:
    lib = load()
    out = []
    for i in range(lib.ayla_b200_kernel_count()):
        vals = [ctypes.c_int32() for _ in range(6)]
        check(lib.ayla_b200_kernel_info(i, *[ctypes.byref(v) for v in vals]))
        keys = ("tile_n", "cta_group", "epilogue", "transposed_out", "stages", "smem_bytes")
        out.append({k: v.value for k, v in zip(keys, vals)})
    return out


def default_config(op: str, dtype: str, batch: int, m: int, n: int, k: int) -> Config:
    cfg = Config()
    check(load().ayla_b200_default_config(OP_CODES[op], DTYPE_CODES[dtype], batch, m, n, k,
                                          ctypes.byref(cfg)))
    return cfg


def config_valid(cfg: Config, op: str, dtype: str, batch: int, m: int, n: int, k: int) -> bool:
    return load().ayla_b200_config_valid(ctypes.byref(cfg), OP_CODES[op], DTYPE_CODES[dtype],
                                         batch, m, n, k) == 0


def workspace_bytes(cfg: Config, op: str, batch: int, m: int, n: int, k: int) -> int:
    return int(load().ayla_b200_workspace_bytes(ctypes.byref(cfg), OP_CODES[op], batch, m, n, k))


def workspace_counter_bytes(cfg: Config, op: str, batch: int, m: int, n: int, k: int) -> int:
    return int(load().ayla_b200_workspace_counter_bytes(ctypes.byref(cfg), OP_CODES[op], batch, m, n, k))


def gemm(op: str, dtype: str, bias_ptr: int, a_ptr: int, bt_ptr: int, out_ptr: int, batch: int,
         m: int, n: int, k: int, cfg: Config | None, workspace_ptr: int, workspace_size: int,
         status_ptr: int, stream: int) -> None:
    check(load().ayla_b200_gemm(
        OP_CODES[op], DTYPE_CODES[dtype], bias_ptr or None, a_ptr, bt_ptr, out_ptr, batch, m, n, k,
        ctypes.byref(cfg) if cfg is not None else None, workspace_ptr or None, workspace_size,
        status_ptr or None, stream or None))


ACT_CODES = {"none": 0, "relu": 1, "sigmoid": 2, "silu": 3, "gelu": 4, "gelu_tanh": 5}


def gemm_act(op: str, dtype: str, activation: str, bias_ptr: int, a_ptr: int, bt_ptr: int, out_ptr: int,
             batch: int, m: int, n: int, k: int, cfg: Config | None, workspace_ptr: int, workspace_size: int,
             status_ptr: int, stream: int) -> None:
    """``gemm`` with ``activation`` applied to the fp32 result before it is rounded."""
    check(load().ayla_b200_gemm_act(
        OP_CODES[op], DTYPE_CODES[dtype], ACT_CODES[activation], bias_ptr or None, a_ptr, bt_ptr, out_ptr,
        batch, m, n, k, ctypes.byref(cfg) if cfg is not None else None, workspace_ptr or None, workspace_size,
        status_ptr or None, stream or None))


def gemm_act_mul(op: str, dtype: str, activation: str, bias_ptr: int, a_ptr: int, bt_ptr: int, mul_ptr: int,
                 out_ptr: int, batch: int, m: int, n: int, k: int, cfg: Config | None, workspace_ptr: int,
                 workspace_size: int, status_ptr: int, stream: int) -> None:
    """``gemm_act`` followed by an elementwise product with ``mul`` (shaped like ``out``), still before
    the one rounding."""
    check(load().ayla_b200_gemm_act_mul(
        OP_CODES[op], DTYPE_CODES[dtype], ACT_CODES[activation], bias_ptr or None, a_ptr, bt_ptr, mul_ptr or None,
        out_ptr, batch, m, n, k, ctypes.byref(cfg) if cfg is not None else None, workspace_ptr or None,
        workspace_size, status_ptr or None, stream or None))


def gemm_act_rowmul(op: str, dtype: str, activation: str, bias_ptr: int, a_ptr: int, bt_ptr: int, row_mul_ptr: int,
                    out_ptr: int, batch: int, m: int, n: int, k: int, cfg: Config | None, workspace_ptr: int,
                    workspace_size: int, status_ptr: int, stream: int) -> None:
    """``gemm_act`` followed by a product with one factor per output row (``batch * m`` elements of the
    operands' type), still before the one rounding."""
    check(load().ayla_b200_gemm_act_rowmul(
        OP_CODES[op], DTYPE_CODES[dtype], ACT_CODES[activation], bias_ptr or None, a_ptr, bt_ptr, row_mul_ptr or None,
        out_ptr, batch, m, n, k, ctypes.byref(cfg) if cfg is not None else None, workspace_ptr or None,
        workspace_size, status_ptr or None, stream or None))


STATIC_SCRATCH_BYTES = 8 << 20


def gemm_static_scratch(op: str, dtype: str, bias_ptr: int, a_ptr: int, bt_ptr: int, out_ptr: int,
                        batch: int, m: int, n: int, k: int, cfg: Config | None, status_ptr: int,
                        stream: int) -> None:
    """``gemm`` for callers that cannot provide or allocate a workspace: split-K scratch
    comes from the 8 MiB array built into the library (see ``include/ayla_b200.h``)."""
    check(load().ayla_b200_gemm_static_scratch(
        OP_CODES[op], DTYPE_CODES[dtype], bias_ptr or None, a_ptr, bt_ptr, out_ptr, batch, m, n, k,
        ctypes.byref(cfg) if cfg is not None else None, status_ptr or None, stream or None))


def copy_2d(dst_ptr: int, dst_pitch: int, src_ptr: int, src_pitch: int, width_bytes: int, rows: int,
            stream: int) -> None:
    """Strided device-to-device copy on the copy engines."""
    check(load().ayla_b200_copy_2d(dst_ptr, dst_pitch, src_ptr, src_pitch, width_bytes, rows, stream or None))


def swiglu(dtype: str, x_ptr: int, wg_ptr: int, wu_ptr: int, out_ptr: int, m: int, n: int, k: int,
           cfg: Config | None, status_ptr: int, stream: int) -> None:
    check(load().ayla_b200_swiglu(
        DTYPE_CODES[dtype], x_ptr, wg_ptr, wu_ptr, out_ptr, m, n, k,
        ctypes.byref(cfg) if cfg is not None else None, status_ptr or None, stream or None))


def set_launch_overlap(enabled: bool) -> None:
    """Allow (default) or forbid a launch to run its set-up under the previous kernel's tail."""
    load().ayla_b200_set_launch_overlap(1 if enabled else 0)
