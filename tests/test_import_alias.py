"""``import ayla`` names the same modules and objects as ``ayla_b200`` (the import paths of the
reference's README.md:37-45)."""


def test_reference_import_paths_resolve_to_this_backend():
    import ayla
    import ayla.gemm_jit
    import ayla.torch_compile
    import ayla.torch_custom_call
    import ayla_b200
    from ayla.gemm_jit import GemmScheduleSeed, gemm_op, measured_gemm_configs, select_gemm_schedule
    from ayla.jit_compiler import ShapeSpecializingJITCompiler
    from ayla.torch_compile import install, uninstall
    from ayla.torch_custom_call import DEFAULT_NAMESPACE, OperandKind, make_torch_custom_call

    assert ayla.gemm_jit is ayla_b200.gemm_jit
    assert gemm_op is ayla_b200.gemm_op and select_gemm_schedule is ayla_b200.select_gemm_schedule
    assert measured_gemm_configs is ayla_b200.measured_gemm_configs and GemmScheduleSeed is ayla_b200.GemmScheduleSeed
    assert install is ayla_b200.torch_compile.install and uninstall is ayla_b200.torch_compile.uninstall
    assert DEFAULT_NAMESPACE == "ayla" and OperandKind is ayla_b200.OperandKind
    assert make_torch_custom_call is ayla_b200.make_torch_custom_call
    assert ShapeSpecializingJITCompiler is ayla_b200.jit_compiler.ShapeSpecializingJITCompiler
    assert ayla.gemm_op("mm", "bfloat16") is ayla_b200.gemm_op("mm", "bfloat16")
