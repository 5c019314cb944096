"""Custom-op glue on the meta device -- mirrors the reference's
tests/test_torch_custom_call.py:8-53."""

import torch

from ayla_b200.torch_custom_call import OperandKind, TensorSpec, make_schema, make_torch_custom_call


def test_out_only_custom_call_has_meta_kernel():
    class Launcher:
        name = "out_only_meta_test"
        signature = [TensorSpec.build([4, 8], torch.bfloat16), TensorSpec.build([4, 16], torch.bfloat16)]

        def __call__(self, *args):
            raise AssertionError("Meta dispatch must not launch the kernel")

    op = make_torch_custom_call(Launcher(), [OperandKind.R, OperandKind.RW], namespace="ayla_b200_out_only_meta_test")
    src = torch.empty((4, 8), dtype=torch.bfloat16, device="meta")
    out = torch.empty((4, 16), dtype=torch.bfloat16, device="meta")
    assert op(src, out) is None


def test_result_shape_can_be_inferred_from_inputs():
    class Launcher:
        name = "dynamic_result_meta_test"
        signature = [TensorSpec.build([1, 8], torch.bfloat16), TensorSpec.build([1, 16], torch.bfloat16)]

        def __call__(self, *args):
            raise AssertionError("Meta dispatch must not launch the kernel")

    op = make_torch_custom_call(
        Launcher(),
        [OperandKind.R, OperandKind.RESULT],
        namespace="ayla_b200_dynamic_result_meta_test",
        infer_result_shapes=lambda src: [(src.shape[0], 16)],
    )
    src = torch.empty((7, 8), dtype=torch.bfloat16, device="meta")
    result = op(src)
    assert result.shape == (7, 16) and result.dtype == torch.bfloat16 and result.device.type == "meta"


def test_schema_rendering():
    kinds = [OperandKind.R, OperandKind.R, OperandKind.RW]
    assert make_schema("jit_mm_bf16", kinds) == "jit_mm_bf16(Tensor arg0, Tensor arg1, Tensor(a2!) arg2) -> ()"
    assert make_schema("f", [OperandKind.R, OperandKind.RESULT]) == "f(Tensor arg0) -> Tensor"
    assert make_schema("g", [OperandKind.RESULT, OperandKind.RESULT]) == "g() -> (Tensor, Tensor)"


def test_dynamic_m_op_infers_its_result_on_meta():
    from ayla_b200.dynamic_m import make_dynamic_m_matmul

    op = make_dynamic_m_matmul(256, 64, namespace="ayla_b200_dynamic_m_meta_test")
    lhs = torch.empty((3, 64), dtype=torch.bfloat16, device="meta")
    rhs = torch.empty((256, 64), dtype=torch.bfloat16, device="meta")
    out = op(lhs, rhs)
    assert out.shape == (3, 256) and out.dtype == torch.bfloat16 and out.device.type == "meta"
