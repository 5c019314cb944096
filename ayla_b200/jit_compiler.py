"""Per-shape dispatch cache in front of the prebuilt kernels.

Keeps the contract of the reference's ``ShapeSpecializingJITCompiler``
(ayla/jit_compiler.py:17-120): one launcher per ``(device, shapes)`` key, the same
argument validation and ``ValueError`` messages (:76-93), and a ``RuntimeError``
when a new shape first shows up during CUDA-graph capture (:106-110).  What
"compiling" means is different: the kernels are already compiled, so a cache miss
only picks a schedule, sizes the split-K workspace and runs the per-device
set-up -- host work that must not happen inside a captured region because it
allocates.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass

import torch

from .torch_custom_call import TensorSpec


@dataclass(frozen=True)
class OpTemplate:
    """Name and operand signature of one op; ``None`` sizes are bound per call."""

    name: str
    signature: tuple[TensorSpec, ...]

    def specialize(self, shapes: Sequence[tuple[int, ...]]) -> "OpTemplate":
        if len(shapes) != len(self.signature):
            raise ValueError(f"{self.name}: expected {len(self.signature)} shapes, got {len(shapes)}")
        bound = []
        for spec, shape in zip(self.signature, shapes):
            if len(shape) != len(spec.sizes):
                raise ValueError(
                    f"{self.name}: expected a rank-{len(spec.sizes)} tensor, got shape {tuple(shape)}"
                )
            for want, got in zip(spec.sizes, shape):
                if want is not None and want != got:
                    raise ValueError(f"{self.name}: expected size {want}, got {got} in {tuple(shape)}")
            bound.append(TensorSpec(spec.dtype, tuple(int(s) for s in shape)))
        return OpTemplate(self.name, tuple(bound))


class ShapeSpecializingJITCompiler:
    """Cache one launcher per concrete tensor signature."""

    def __init__(self, template: OpTemplate, compile_fn: Callable[[OpTemplate, torch.device], Callable]):
        if not template.signature:
            raise ValueError("ShapeSpecializingJITCompiler requires at least one operand")
        self._template = template
        self._compile_fn = compile_fn
        self._cache: dict[tuple[object, ...], Callable] = {}

    @property
    def name(self) -> str:
        return self._template.name

    @property
    def signature(self) -> tuple[TensorSpec, ...]:
        return self._template.signature

    @property
    def cache_size(self) -> int:
        return len(self._cache)

    def _metadata(self, tensors: tuple[torch.Tensor, ...]):
        if len(tensors) != len(self.signature):
            raise ValueError(f"{self.name}: expected {len(self.signature)} tensors, got {len(tensors)}")
        if any(not t.is_cuda for t in tensors):
            raise ValueError(f"{self.name}: all tensors must be CUDA tensors")
        if any(not t.is_contiguous() for t in tensors):
            raise ValueError(f"{self.name}: all tensors must be contiguous")
        device = tensors[0].device
        if any(t.device != device for t in tensors[1:]):
            raise ValueError(f"{self.name}: all tensors must be on one CUDA device")
        for tensor, spec in zip(tensors, self.signature):
            if tensor.dtype != spec.dtype:
                raise ValueError(f"{self.name}: expected dtype {spec.dtype}, got {tensor.dtype}")
        shapes = [tuple(t.shape) for t in tensors]
        return (device, tuple(shapes)), shapes

    def _launcher(self, tensors: tuple[torch.Tensor, ...]):
        key, shapes = self._metadata(tensors)
        launcher = self._cache.get(key)
        if launcher is not None:
            return launcher
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                f"{self.name}: specialization cache miss during CUDA graph capture; "
                "invoke the kernel once before capture"
            )
        launcher = self._compile_fn(self._template.specialize(shapes), key[0])
        self._cache[key] = launcher
        return launcher

    def __call__(self, *tensors: torch.Tensor) -> None:
        self._launcher(tuple(tensors))(*tensors)
