"""Dispatch cache, with fakes -- mirrors the reference's tests/test_jit_compiler.py:44-93."""

import pytest
import torch

from ayla_b200.jit_compiler import OpTemplate, ShapeSpecializingJITCompiler
from ayla_b200.torch_custom_call import TensorSpec


def _template(name="dispatch_test") -> OpTemplate:
    bf16 = torch.bfloat16
    return OpTemplate(name, (TensorSpec(bf16, (None, 8)), TensorSpec(bf16, (16, 8)), TensorSpec(bf16, (None, 16))))


def _shapes(m=4):
    return [(m, 8), (16, 8), (m, 16)]


class _Launcher:
    def __init__(self):
        self.launches = 0

    def __call__(self, *args):
        self.launches += 1


class _Tensor:
    device = torch.device("cuda")


def _patch_metadata(monkeypatch, compiler, m=4):
    monkeypatch.setattr(compiler, "_metadata", lambda tensors: (("test", m), _shapes(m)))
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)


def test_jit_compiler_caches_by_shape(monkeypatch):
    compiled = []

    def compile_fn(bound, device):
        compiled.append(bound)
        return _Launcher()

    compiler = ShapeSpecializingJITCompiler(_template(), compile_fn)
    _patch_metadata(monkeypatch, compiler)
    tensors = (_Tensor(), _Tensor(), _Tensor())
    compiler(*tensors)
    compiler(*tensors)
    assert len(compiled) == 1 and compiler.cache_size == 1
    assert compiler._launcher(tensors).launches == 2
    assert all(spec.is_static for spec in compiled[0].signature)
    assert not all(spec.is_static for spec in compiler.signature)


def test_jit_compiler_rejects_capture_time_cache_miss(monkeypatch):
    compiler = ShapeSpecializingJITCompiler(_template("dispatch_capture_miss"), lambda bound, device: _Launcher())
    _patch_metadata(monkeypatch, compiler)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: True)
    with pytest.raises(RuntimeError, match="before capture"):
        compiler(_Tensor(), _Tensor(), _Tensor())


def test_jit_compiler_rejects_noncontiguous_tensors():
    class Tensor:
        is_cuda = True
        device = torch.device("cuda")

        def is_contiguous(self):
            return False

    compiler = ShapeSpecializingJITCompiler(_template(), lambda bound, device: _Launcher())
    with pytest.raises(ValueError, match="contiguous"):
        compiler(Tensor(), Tensor(), Tensor())


def test_jit_compiler_rejects_wrong_dtype_and_static_size_mismatch(monkeypatch):
    class Tensor:
        is_cuda = True
        device = torch.device("cuda")
        dtype = torch.float16
        shape = (4, 8)

        def is_contiguous(self):
            return True

    compiler = ShapeSpecializingJITCompiler(_template(), lambda bound, device: _Launcher())
    with pytest.raises(ValueError, match="expected dtype"):
        compiler(Tensor(), Tensor(), Tensor())
    with pytest.raises(ValueError, match="expected size 16"):
        _template().specialize([(4, 8), (32, 8), (4, 16)])
    with pytest.raises(ValueError, match="rank-2"):
        _template().specialize([(4, 8), (16, 8), (2, 4, 16)])
