"""Expose a launcher as a ``torch.ops.<namespace>.<name>`` custom op.

Same surface as the reference's glue (ayla/torch_custom_call.py:40-43, :64-80,
:83-155): ``OperandKind`` marks each launcher operand as read-only input (R),
caller-allocated in/out tensor (RW, rendered ``Tensor(aN!)`` in the schema) or
op-allocated result (RESULT); the op gets a CUDA implementation that calls the
launcher and a Meta implementation that only allocates, so tracing never
launches a kernel.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass
from enum import Enum
from typing import Protocol

import torch

DEFAULT_NAMESPACE = "ayla"

_LIBRARIES: dict[str, torch.library.Library] = {}


class OperandKind(Enum):
    R = "r"
    RW = "rw"
    RESULT = "result"


@dataclass(frozen=True)
class TensorSpec:
    """Dtype and (possibly dynamic, ``None``) sizes of one launcher operand.

    Stands in for the reference's ``GmemTensorType`` (ayla/gpu_dialect.py) as far
    as the op glue needs it."""

    dtype: torch.dtype
    sizes: tuple[int | None, ...]

    @classmethod
    def build(cls, sizes: Sequence[int | None], dtype: torch.dtype) -> "TensorSpec":
        return cls(dtype, tuple(sizes))

    @property
    def is_static(self) -> bool:
        return all(size is not None for size in self.sizes)


class Launcher(Protocol):
    @property
    def name(self) -> str: ...

    @property
    def signature(self) -> Sequence[TensorSpec]: ...

    def __call__(self, *tensors: torch.Tensor) -> None: ...


def _library(namespace: str) -> torch.library.Library:
    if namespace not in _LIBRARIES:
        _LIBRARIES[namespace] = torch.library.Library(namespace, "FRAGMENT")
    return _LIBRARIES[namespace]


def make_schema(op_name: str, kinds: Sequence[OperandKind]) -> str:
    """``name(Tensor arg0, Tensor(a2!) arg2, ...) -> ...`` for the given operand kinds."""
    params: list[str] = []
    results = 0
    for position, kind in enumerate(kinds):
        if kind is OperandKind.RESULT:
            results += 1
        elif kind is OperandKind.RW:
            params.append(f"Tensor(a{position}!) arg{len(params)}")
        else:
            params.append(f"Tensor arg{len(params)}")
    returns = "Tensor" if results == 1 else "(" + ", ".join(["Tensor"] * results) + ")"
    return f"{op_name}({', '.join(params)}) -> {returns}"


def make_torch_custom_call(
    launcher: Launcher,
    signature_mapping: Sequence[OperandKind],
    *,
    namespace: str = DEFAULT_NAMESPACE,
    name: str | None = None,
    infer_result_shapes: Callable[..., list[tuple[int, ...]]] | None = None,
) -> torch._ops.OpOverload:
    kinds = list(signature_mapping)
    op_name = name or launcher.name
    lib = _library(namespace)
    lib.define(make_schema(op_name, kinds))
    result_positions = [i for i, kind in enumerate(kinds) if kind is OperandKind.RESULT]

    def new_results(inputs: tuple[torch.Tensor, ...]) -> list[torch.Tensor]:
        if not result_positions:
            return []
        specs = [launcher.signature[i] for i in result_positions]
        if infer_result_shapes is not None:
            shapes = [tuple(shape) for shape in infer_result_shapes(*inputs)]
        else:
            shapes = [tuple(spec.sizes) for spec in specs]
        if len(shapes) != len(specs):
            raise ValueError(f"{op_name}: expected {len(specs)} result shapes, got {len(shapes)}")
        device = inputs[0].device if inputs else torch.device("cuda")
        return [torch.empty(shape, dtype=spec.dtype, device=device) for spec, shape in zip(specs, shapes)]

    def pack(results: list[torch.Tensor]):
        if not results:
            return None
        return results[0] if len(results) == 1 else tuple(results)

    def cuda_impl(*inputs: torch.Tensor):
        results = new_results(inputs)
        given, made = iter(inputs), iter(results)
        operands = [next(made) if kind is OperandKind.RESULT else next(given) for kind in kinds]
        launcher(*operands)
        return pack(results)

    def meta_impl(*inputs: torch.Tensor):
        return pack(new_results(inputs))

    lib.impl(op_name, cuda_impl, "CUDA")
    lib.impl(op_name, meta_impl, "Meta")
    return getattr(getattr(torch.ops, namespace), op_name).default
