"""Routing decisions of ``ayla_b200.torch_compile`` (mirrors the reference's
tests/test_torch_compile.py:140-157 and tests/test_gemm_jit.py:77-98).  The decision
logic is exercised on CPU with fake CUDA tensors; the end-to-end compile runs on a GPU."""

import pytest
import torch
from torch._inductor import config as inductor_config
from torch._inductor.decomposition import select_decomp_table
from torch._subclasses.fake_tensor import FakeTensorMode
from torch.fx.experimental.proxy_tensor import make_fx

from ayla_b200 import torch_compile as tc

aten = torch.ops.aten


def trace(fn, *specs):
    """FX graph of fn over fake tensors described by (shape, dtype, device) specs."""
    with FakeTensorMode(allow_non_fake_inputs=True):
        args = [torch.empty(shape, dtype=dtype, device=device) for shape, dtype, device in specs]
        return make_fx(fn, decomposition_table=select_decomp_table(), tracing_mode="real")(*args)


def targets(gm):
    return [n.target for n in gm.graph.nodes if n.op == "call_function"]


BF16, F16, F32 = torch.bfloat16, torch.float16, torch.float32


def test_supported_gemms_are_claimed():
    gm = trace(lambda a, bt: torch.mm(a, bt.t()), ((96, 128), BF16, "cuda"), ((128, 128), BF16, "cuda"))
    assert tc.route_gemms(gm.graph) == 1
    assert torch.ops.ayla.jit_mm_bf16_fn.default in targets(gm) and aten.mm.default not in targets(gm)

    gm = trace(lambda bias, a, bt: torch.addmm(bias, a, bt.t()),
               ((128,), F16, "cuda"), ((96, 128), F16, "cuda"), ((128, 128), F16, "cuda"))
    assert tc.route_gemms(gm.graph) == 1
    assert torch.ops.ayla.jit_addmm_f16_fn.default in targets(gm)

    gm = trace(lambda a, bt: torch.bmm(a, bt.transpose(-1, -2)),
               ((2, 96, 128), BF16, "cuda"), ((2, 128, 128), BF16, "cuda"))
    assert tc.route_gemms(gm.graph) == 1
    assert torch.ops.ayla.jit_bmm_bf16_fn.default in targets(gm)
    gm.graph.lint()


@pytest.mark.parametrize(
    "fn, specs",
    [
        # CPU tensors
        (lambda a, bt: torch.mm(a, bt.t()), [((96, 128), BF16, "cpu"), ((128, 128), BF16, "cpu")]),
        # float32
        (lambda a, bt: torch.mm(a, bt.t()), [((96, 128), F32, "cuda"), ((128, 128), F32, "cuda")]),
        # rhs is a plain contiguous [k, n] matrix, not a transposed view of bt
        (lambda a, b: torch.mm(a, b), [((96, 128), BF16, "cuda"), ((128, 64), BF16, "cuda")]),
        # non-contiguous lhs
        (lambda a, bt: torch.mm(a.t(), bt.t()), [((128, 96), BF16, "cuda"), ((128, 128), BF16, "cuda")]),
        # n not a multiple of 8: no schedule
        (lambda a, bt: torch.mm(a, bt.t()), [((96, 128), BF16, "cuda"), ((60, 128), BF16, "cuda")]),
        # scaled addmm
        (lambda bias, a, bt: torch.addmm(bias, a, bt.t(), alpha=2.0),
         [((128,), BF16, "cuda"), ((96, 128), BF16, "cuda"), ((128, 128), BF16, "cuda")]),
        # bias that is not [n]
        (lambda bias, a, bt: torch.addmm(bias, a, bt.t()),
         [((96, 128), BF16, "cuda"), ((96, 128), BF16, "cuda"), ((128, 128), BF16, "cuda")]),
    ],
)
def test_unsupported_gemms_are_declined(fn, specs):
    gm = trace(fn, *specs)
    before = targets(gm)
    assert tc.route_gemms(gm.graph) == 0
    assert targets(gm) == before


def test_swiglu_pattern_is_fused_and_partial_patterns_are_not():
    import torch.nn.functional as F

    specs = (((64, 32), BF16, "cuda"), ((48, 32), BF16, "cuda"), ((48, 32), BF16, "cuda"))
    gm = trace(lambda x, wg, wu: F.silu(torch.mm(x, wg.t())) * torch.mm(x, wu.t()), *specs)
    assert tc.route_swiglu(gm.graph) == 1
    got = targets(gm)
    assert torch.ops.ayla.swiglu_bf16_fn.default in got and aten.mm.default not in got
    gm.graph.lint()
    # operand order of the product does not matter
    gm = trace(lambda x, wg, wu: torch.mm(x, wu.t()) * F.silu(torch.mm(x, wg.t())), *specs)
    assert tc.route_swiglu(gm.graph) == 1
    # the gate product is also returned: fusing would lose it, so the two mm are routed separately
    gm = trace(lambda x, wg, wu: (F.silu(torch.mm(x, wg.t())) * torch.mm(x, wu.t()), torch.mm(x, wg.t())), *specs)
    fused = tc.route_swiglu(gm.graph)
    assert fused == 0 or aten.mm.default in targets(gm) or torch.ops.ayla.jit_mm_bf16_fn.default in targets(gm)
    # different activations of x: not a SwiGLU
    gm = trace(lambda x, y, wg: F.silu(torch.mm(x, wg.t())) * torch.mm(y, wg.t()),
               ((64, 32), BF16, "cuda"), ((64, 32), BF16, "cuda"), ((48, 32), BF16, "cuda"))
    assert tc.route_swiglu(gm.graph) == 0
    # the whole pass: fused op, nothing left for route_gemms
    gm = trace(lambda x, wg, wu: F.silu(torch.mm(x, wg.t())) * torch.mm(x, wu.t()), *specs)
    tc.AylaRoutingPass()(gm.graph)
    assert targets(gm).count(torch.ops.ayla.swiglu_bf16_fn.default) == 1
    assert torch.ops.ayla.jit_mm_bf16_fn.default not in targets(gm)


@pytest.mark.parametrize("activation", ["relu", "sigmoid", "silu", "gelu"])
def test_activation_after_a_gemm_is_fused(activation):
    import torch.nn.functional as F

    act = {"relu": torch.relu, "sigmoid": torch.sigmoid, "silu": F.silu, "gelu": F.gelu}[activation]
    mm_specs = (((64, 32), BF16, "cuda"), ((48, 32), BF16, "cuda"))
    gm = trace(lambda a, bt: act(torch.mm(a, bt.t())), *mm_specs)
    assert tc.route_activations(gm.graph) == 1
    gm.graph.lint()
    assert getattr(torch.ops.ayla, f"jit_mm_{activation}_bf16_fn").default in targets(gm)
    leftovers = {aten.mm.default, aten.relu.default, aten.sigmoid.default, aten.erf.default, aten.exp.default}
    assert not leftovers & set(targets(gm))

    gm = trace(lambda bias, a, bt: act(torch.addmm(bias, a, bt.t())), ((48,), F16, "cuda"),
               ((64, 32), F16, "cuda"), ((48, 32), F16, "cuda"))
    assert tc.route_activations(gm.graph) == 1
    assert getattr(torch.ops.ayla, f"jit_addmm_{activation}_f16_fn").default in targets(gm)

    # the plain product has a second reader: nothing is fused (the GEMM itself is still claimed later)
    gm = trace(lambda a, bt: (lambda prod: act(prod) + prod)(torch.mm(a, bt.t())), *mm_specs)
    assert tc.route_activations(gm.graph) == 0
    assert tc.route_gemms(gm.graph) == 1
    # a GEMM this library would not claim keeps its activation too
    gm = trace(lambda a, b: act(torch.mm(a, b)), ((64, 32), BF16, "cuda"), ((32, 48), BF16, "cuda"))
    assert tc.route_activations(gm.graph) == 0


def test_gated_product_is_fused():
    import torch.nn.functional as F

    specs = (((64, 32), BF16, "cuda"), ((48, 32), BF16, "cuda"), ((64, 48), BF16, "cuda"))
    for name, fn in (("sigmoid_mul", lambda a, bt, v: torch.sigmoid(torch.mm(a, bt.t())) * v),
                     ("silu_mul", lambda a, bt, v: v * F.silu(torch.mm(a, bt.t()))),
                     ("mul", lambda a, bt, v: torch.mm(a, bt.t()) * v)):
        gm = trace(fn, *specs)
        assert tc.route_gated(gm.graph) == 1
        gm.graph.lint()
        assert getattr(torch.ops.ayla, f"jit_mm_{name}_bf16_fn").default in targets(gm)
        assert not {aten.mm.default, aten.mul.Tensor, aten.sigmoid.default} & set(targets(gm))
    # a broadcast gate, a gate of another type, or a product that is read elsewhere: left alone
    gm = trace(lambda a, bt, v: torch.sigmoid(torch.mm(a, bt.t())) * v, specs[0], specs[1], ((48,), BF16, "cuda"))
    assert tc.route_gated(gm.graph) == 0
    gm = trace(lambda a, bt, v: torch.sigmoid(torch.mm(a, bt.t())) * v, specs[0], specs[1], ((64, 48), F32, "cuda"))
    assert tc.route_gated(gm.graph) == 0
    gm = trace(lambda a, bt, v: (lambda prod: (torch.sigmoid(prod) * v, prod))(torch.mm(a, bt.t())), *specs)
    assert tc.route_gated(gm.graph) == 0


def test_swiglu_on_a_concatenated_weight_is_fused():
    import torch.nn.functional as F

    def block(x, w):
        gate, up = torch.mm(x, w.t()).chunk(2, dim=-1)
        return F.silu(gate) * up

    gm = trace(block, ((64, 32), BF16, "cuda"), ((96, 32), BF16, "cuda"))
    assert tc.route_swiglu_concat(gm.graph) == 1
    gm.graph.lint()
    assert torch.ops.ayla.swiglu_bf16_fn.default in targets(gm) and aten.mm.default not in targets(gm)
    # halves that are not a multiple of 8 columns, or a product that is read elsewhere, are left alone
    gm = trace(block, ((64, 32), BF16, "cuda"), ((40, 32), BF16, "cuda"))
    assert tc.route_swiglu_concat(gm.graph) == 0

    def leaky(x, w):
        prod = torch.mm(x, w.t())
        gate, up = prod.chunk(2, dim=-1)
        return F.silu(gate) * up, prod

    gm = trace(leaky, ((64, 32), BF16, "cuda"), ((96, 32), BF16, "cuda"))
    assert tc.route_swiglu_concat(gm.graph) == 0


def test_swiglu_on_a_concatenated_weight_spelled_as_two_slices_is_fused():
    """The form a captured decoder block holds (the reference's
    benchmarks/bench_torch_compile/corpus/muse_glimmer_block.py:42-50): the gate half is
    ``slice(mm, 1, 0, n)``, the up half ``slice(mm, 1, n, INT64_MAX)``, silu decomposed in fp32."""
    big = 9223372036854775807

    def block(x, w_t):
        mm = aten.mm.default(x, w_t)
        gate = aten.slice.Tensor(mm, 1, 0, 48)
        g32 = torch.ops.prims.convert_element_type.default(gate, torch.float32)
        act = torch.ops.prims.convert_element_type.default(
            aten.div.Tensor(g32, aten.add.Tensor(aten.exp.default(aten.neg.default(g32)), 1)), torch.bfloat16)
        up = aten.slice.Tensor(mm, 1, 48, big)
        return aten.mul.Tensor(act, up)

    def traced(x, w):
        return block(x, w.t())

    gm = trace(traced, ((64, 32), BF16, "cuda"), ((96, 32), BF16, "cuda"))
    assert aten.slice.Tensor in targets(gm)
    assert tc.route_swiglu_concat(gm.graph) == 1
    gm.graph.lint()
    assert torch.ops.ayla.swiglu_bf16_fn.default in targets(gm) and aten.mm.default not in targets(gm)

    # slices that are not the two halves are left alone
    def uneven(x, w):
        mm = aten.mm.default(x, w.t())
        return torch.nn.functional.silu(aten.slice.Tensor(mm, 1, 0, 32)) * aten.slice.Tensor(mm, 1, 64, big)

    gm = trace(uneven, ((64, 32), BF16, "cuda"), ((96, 32), BF16, "cuda"))
    assert tc.route_swiglu_concat(gm.graph) == 0


def test_swiglu_fusion_is_declined_where_its_column_tiles_fill_the_sms_badly():
    assert tc._swiglu_pays(8, 14336) and tc._swiglu_pays(4096, 19968) and tc._swiglu_pays(64, 128 * 148)
    assert not tc._swiglu_pays(8, 19968) and not tc._swiglu_pays(64, 128 * 149)

    def block(x, w):
        gate, up = torch.mm(x, w.t()).chunk(2, dim=-1)
        return torch.nn.functional.silu(gate) * up

    gm = trace(block, ((8, 64), BF16, "cuda"), ((2 * 19968, 64), BF16, "cuda"))
    assert tc.route_swiglu_concat(gm.graph) == 0       # left to the plain GEMM route
    assert tc.route_gemms(gm.graph) == 1


def test_gated_decoder_block_body_is_routed_completely():
    """The whole-graph driver's block body (gated attention output projection, SwiGLU on a
    concatenated weight read as two slices, fused QKV): after the pass every GEMM is one of this
    library's ops, the gate is fused into its GEMM and the MLP is the fused SwiGLU op."""
    from ayla_b200.bench_torch_compile import gated_block_fn

    tokens, hidden, attn, ffn, kv = 16, 64, 32, 48, 8
    block = gated_block_fn(attn, ffn, kv)
    cuda = "cuda"
    specs = [((tokens, hidden), BF16, cuda), ((tokens, attn), BF16, cuda), ((tokens, hidden), BF16, cuda),
             ((attn, hidden), BF16, cuda), ((hidden, attn), BF16, cuda), ((2 * ffn, hidden), BF16, cuda),
             ((hidden, ffn), BF16, cuda), ((attn + 2 * kv, hidden), BF16, cuda)] + [((hidden,), BF16, cuda)] * 4
    gm = trace(block, *specs)
    assert targets(gm).count(aten.mm.default) == 5
    tc.AylaRoutingPass()(gm.graph)
    gm.graph.lint()
    found = targets(gm)
    assert aten.mm.default not in found
    assert found.count(torch.ops.ayla.swiglu_bf16_fn.default) == 1
    assert found.count(torch.ops.ayla.jit_mm_sigmoid_mul_bf16_fn.default) == 1
    assert found.count(torch.ops.ayla.jit_mm_bf16_fn.default) == 3


def _freeze(gm, constants):
    """Turn placeholders into attributes of the module, as Inductor's freezing does with parameters."""
    for node in list(gm.graph.nodes):
        if node.op == "placeholder" and node.target in constants:
            gm.register_buffer(f"_frozen_{node.target}", constants[node.target], persistent=False)
            with gm.graph.inserting_before(node):
                attr = gm.graph.get_attr(f"_frozen_{node.target}")
                attr.meta.update(node.meta)
            node.replace_all_uses_with(attr)
            gm.graph.erase_node(node)
    gm.recompile()
    return gm


def rms_then_project(x, g, w):
    return torch.mm(torch.nn.functional.rms_norm(x, (x.shape[-1],), g, 1e-5), w.t())


def test_rmsnorm_before_a_projection_with_constant_weights_becomes_a_row_scaled_gemm():
    m, n, k = 64, 256, 128
    gm = trace(rms_then_project, ((m, k), BF16, "cuda"), ((k,), BF16, "cuda"), ((n, k), BF16, "cuda"))
    names = [node.target for node in gm.graph.nodes if node.op == "placeholder"]
    torch.manual_seed(0)
    g, w = torch.randn(k).to(BF16), torch.randn(n, k).to(BF16)
    _freeze(gm, {names[1]: g, names[2]: w})
    assert tc.route_rmsnorm(gm.graph) == 1
    gm.graph.lint()
    assert torch.ops.ayla.jit_mm_rowmul_bf16_fn.default in targets(gm) and aten.mm.default not in targets(gm)
    call = next(node for node in gm.graph.nodes if node.target is torch.ops.ayla.jit_mm_rowmul_bf16_fn.default)
    x_node, weight_node, factors_node = call.args
    assert x_node.op == "placeholder" and weight_node.op == "get_attr"
    folded = getattr(gm, weight_node.target)
    assert folded.shape == (n, k) and folded.is_contiguous() and folded.dtype == BF16
    assert torch.equal(folded, (w.float() * g.float()).to(BF16))
    assert factors_node.meta["val"].shape == (m, 1) and factors_node.meta["val"].dtype == BF16
    # the normalised activations are no longer computed: only the row reduction is left
    assert sum(1 for t in targets(gm) if t is aten.mul.Tensor) == 0
    # and the rewrite is the same function: r * (x @ (W * g).T) against rms_norm(x, g) @ W.T
    x = torch.randn(m, k).to(BF16)
    want = rms_then_project(x.float(), g.float(), w.float())
    r = torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5).to(BF16).float()
    got = r * (x.float() @ folded.float().t())
    assert (got - want).norm() / want.norm() < 5e-3


def test_rmsnorm_routing_needs_constant_weights_and_the_exact_pattern():
    m, n, k = 64, 256, 128
    specs = (((m, k), BF16, "cuda"), ((k,), BF16, "cuda"), ((n, k), BF16, "cuda"))
    gm = trace(rms_then_project, *specs)  # weights are graph inputs: nothing to fold
    assert tc.route_rmsnorm(gm.graph) == 0
    # a norm over another axis is not RMSNorm over the features
    def other_axis(x, g, w):
        xf = x.float()
        return torch.mm((xf * torch.rsqrt(xf.pow(2).mean(0, keepdim=True) + 1e-5) * g).to(x.dtype), w.t())
    gm = trace(other_axis, *specs)
    names = [node.target for node in gm.graph.nodes if node.op == "placeholder"]
    _freeze(gm, {names[1]: torch.randn(k).to(BF16), names[2]: torch.randn(n, k).to(BF16)})
    assert tc.route_rmsnorm(gm.graph) == 0


def test_every_op_the_pass_can_emit_is_registered_by_install():
    """On a hit in Inductor's code cache the pass never runs in the new process: the cached code
    names torch.ops.ayla.* ops, which must exist after install() alone."""
    from ayla_b200.gemm_jit import ACTIVATIONS, _op_name

    previous = inductor_config.post_grad_custom_post_pass
    try:
        tc.install()
        for dtype, short in (("float16", "f16"), ("bfloat16", "bf16")):
            assert hasattr(torch.ops.ayla, f"swiglu_{short}_fn")
            for operation in ("mm", "addmm", "bmm"):
                for activation in ACTIVATIONS:
                    for gated in (False, True):
                        name = f"{_op_name(operation, dtype, activation, gated)}_fn"
                        assert hasattr(torch.ops.ayla, name), name
            assert hasattr(torch.ops.ayla, f"jit_mm_rowmul_{short}_fn")
        # every activation the matcher can name is one of those
        assert {"relu", "sigmoid", "silu", "gelu", "gelu_tanh"} <= set(ACTIVATIONS)
    finally:
        tc.uninstall()
        inductor_config.post_grad_custom_post_pass = previous


def test_install_is_idempotent_and_uninstall_restores():
    previous = inductor_config.post_grad_custom_post_pass
    try:
        tc.install()
        first = inductor_config.post_grad_custom_post_pass
        assert isinstance(first, tc.AylaRoutingPass) and first.previous is previous
        tc.install()
        assert inductor_config.post_grad_custom_post_pass is first
        assert first.uuid() == first.uuid()
        for operation in ("mm", "addmm", "bmm"):
            for short in ("f16", "bf16"):
                assert hasattr(torch.ops.ayla, f"jit_{operation}_{short}")
                assert hasattr(torch.ops.ayla, f"jit_{operation}_{short}_fn")
        tc.uninstall()
        assert inductor_config.post_grad_custom_post_pass is previous
        # someone else claims the hook after us: stand down without touching it
        tc.install()
        other = lambda graph: None  # noqa: E731
        inductor_config.post_grad_custom_post_pass = other
        tc.uninstall()
        assert inductor_config.post_grad_custom_post_pass is other
    finally:
        inductor_config.post_grad_custom_post_pass = previous
        tc.uninstall()


@pytest.fixture
def ayla_installed():
    tc.install()
    try:
        yield
    finally:
        tc.uninstall()
        torch._dynamo.reset()


@pytest.mark.gpu
@pytest.mark.parametrize("operation", ["mm", "addmm", "bmm"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_torch_compile_routes_supported_gemms_to_jit(operation, dtype, ayla_installed):
    """tests/test_gemm_jit.py:77-98 of the reference."""
    from torch._inductor.utils import run_and_get_code

    lead = (2,) if operation == "bmm" else ()
    a = torch.randn((*lead, 96, 128), device="cuda", dtype=dtype)
    bt = torch.randn((*lead, 128, 128), device="cuda", dtype=dtype)
    bias = torch.randn(128, device="cuda", dtype=dtype)

    def compute(a, bt, bias):
        if operation == "addmm":
            return torch.addmm(bias, a, bt.T)
        if operation == "bmm":
            return torch.bmm(a, bt.transpose(-1, -2))
        return torch.mm(a, bt.T)

    with torch.no_grad(), inductor_config.patch(force_disable_caches=True):
        actual, code = run_and_get_code(torch.compile(compute, fullgraph=True, dynamic=False), a, bt, bias)
        expected = compute(a, bt, bias)
    torch.testing.assert_close(actual, expected, atol=0.125, rtol=0.02)
    assert any(f"jit_{operation}_" in source for source in code)


@pytest.mark.gpu
def test_torch_compile_fuses_swiglu(ayla_installed):
    import torch.nn.functional as F
    from torch._inductor.utils import run_and_get_code

    x = torch.randn(200, 256, device="cuda", dtype=torch.bfloat16)
    wg = (torch.randn(264, 256, device="cuda") * 256 ** -0.5).bfloat16()
    wu = (torch.randn(264, 256, device="cuda") * 256 ** -0.5).bfloat16()

    def mlp(x, wg, wu):
        return F.silu(torch.mm(x, wg.T)) * torch.mm(x, wu.T)

    with torch.no_grad(), inductor_config.patch(force_disable_caches=True):
        actual, code = run_and_get_code(torch.compile(mlp, fullgraph=True, dynamic=False), x, wg, wu)
    expected = (F.silu(x.float() @ wg.float().T) * (x.float() @ wu.float().T)).bfloat16()
    torch.testing.assert_close(actual, expected, atol=0.05, rtol=0.02)
    assert any("swiglu_bf16" in source for source in code)
    assert not any("jit_mm_" in source for source in code)


@pytest.mark.gpu
@pytest.mark.parametrize("activation", ["relu", "sigmoid", "silu", "gelu"])
def test_torch_compile_fuses_activation_into_the_gemm(activation, ayla_installed):
    import torch.nn.functional as F
    from torch._inductor.utils import run_and_get_code

    act = {"relu": torch.relu, "sigmoid": torch.sigmoid, "silu": F.silu, "gelu": F.gelu}[activation]
    a = torch.randn(200, 256, device="cuda", dtype=torch.bfloat16)
    bt = (torch.randn(264, 256, device="cuda") * 256 ** -0.5).bfloat16()
    bias = torch.randn(264, device="cuda", dtype=torch.bfloat16)

    def layer(a, bt, bias):
        return act(torch.addmm(bias, a, bt.T))

    with torch.no_grad(), inductor_config.patch(force_disable_caches=True):
        actual, code = run_and_get_code(torch.compile(layer, fullgraph=True, dynamic=False), a, bt, bias)
    expected = act(torch.addmm(bias.float(), a.float(), bt.float().T)).bfloat16()
    torch.testing.assert_close(actual, expected, atol=0.05, rtol=0.02)
    assert any(f"jit_addmm_{activation}_bf16" in source for source in code)
    assert not any("triton" in source and "sigmoid" in source for source in code)


@pytest.mark.gpu
def test_torch_compile_fuses_a_gated_projection(ayla_installed):
    """sigmoid(x @ Wg.T) * v followed by the output projection: the gate becomes one kernel."""
    from torch._inductor.utils import run_and_get_code

    x = torch.randn(200, 256, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(200, 264, device="cuda", dtype=torch.bfloat16)
    wg = (torch.randn(264, 256, device="cuda") * 256 ** -0.5).bfloat16()
    wo = (torch.randn(256, 264, device="cuda") * 264 ** -0.5).bfloat16()

    def gated(x, v, wg, wo):
        return torch.mm(torch.sigmoid(torch.mm(x, wg.T)) * v, wo.T)

    with torch.no_grad(), inductor_config.patch(force_disable_caches=True):
        actual, code = run_and_get_code(torch.compile(gated, fullgraph=True, dynamic=False), x, v, wg, wo)
    expected = ((torch.sigmoid(x.float() @ wg.float().T) * v.float()).bfloat16().float() @ wo.float().T).bfloat16()
    torch.testing.assert_close(actual, expected, atol=0.06, rtol=0.03)
    assert any("jit_mm_sigmoid_mul_bf16" in source for source in code)
    assert any("jit_mm_bf16" in source for source in code)


@pytest.mark.gpu
def test_torch_compile_routes_rmsnorm_before_a_projection_when_the_weights_are_frozen(ayla_installed):
    """With Inductor's freezing the norm weight and the projection weight are constants: the norm
    weight is folded into the projection, the row factor goes into the GEMM's epilogue."""
    from torch._inductor.utils import run_and_get_code

    class NormThenProject(torch.nn.Module):
        def __init__(self, hidden, out_features):
            super().__init__()
            self.g = torch.nn.Parameter(1.0 + 0.1 * torch.randn(hidden))
            self.w = torch.nn.Parameter(torch.randn(out_features, hidden) * hidden ** -0.5)

        def forward(self, x):
            return torch.nn.functional.linear(torch.nn.functional.rms_norm(x, (x.shape[-1],), self.g, 1e-5), self.w)

    torch.manual_seed(0)
    block = NormThenProject(512, 768).to(device="cuda", dtype=torch.bfloat16).eval()
    x = torch.randn(200, 512, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        expected = block(x)
        with inductor_config.patch(force_disable_caches=True, freezing=True):
            actual, code = run_and_get_code(torch.compile(block, fullgraph=True, dynamic=False), x)
    assert any("jit_mm_rowmul_bf16" in source for source in code)
    error = (actual.float() - expected.float()).norm() / expected.float().norm()
    assert error < 5e-3, error


@pytest.mark.gpu
def test_torch_compile_fuses_swiglu_on_a_concatenated_weight(ayla_installed):
    import torch.nn.functional as F
    from torch._inductor.utils import run_and_get_code

    x = torch.randn(200, 256, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(528, 256, device="cuda") * 256 ** -0.5).bfloat16()

    def mlp(x, w):
        gate, up = torch.mm(x, w.T).chunk(2, dim=-1)
        return F.silu(gate) * up

    with torch.no_grad(), inductor_config.patch(force_disable_caches=True):
        actual, code = run_and_get_code(torch.compile(mlp, fullgraph=True, dynamic=False), x, w)
    both = x.float() @ w.float().T
    expected = (F.silu(both[:, :264]) * both[:, 264:]).bfloat16()
    torch.testing.assert_close(actual, expected, atol=0.05, rtol=0.02)
    assert any("swiglu_bf16" in source for source in code)
    assert not any("jit_mm_" in source for source in code)


@pytest.mark.gpu
def test_torch_compile_declines_cpu_and_plain_layout(ayla_installed):
    from torch._inductor.utils import run_and_get_code

    a = torch.randn(96, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(128, 64, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad(), inductor_config.patch(force_disable_caches=True):
        actual, code = run_and_get_code(torch.compile(lambda x, y: torch.mm(x, y), dynamic=False), a, b)
    torch.testing.assert_close(actual, a @ b, atol=0.125, rtol=0.02)
    assert not any("jit_mm_" in source for source in code)


@pytest.mark.gpu
def test_whole_graph_driver_routes_a_decoder_block():
    from ayla_b200.bench_torch_compile import run

    row = run(tokens=64, layers=1, hidden=256, ffn=512, heads=4, kv_heads=2)
    counts = row["routed_calls_in_generated_code"]
    assert counts["jit_mm_bf16_fn"] >= 3 and counts["swiglu_bf16_fn"] >= 1
    assert row["fro_rel_between_arms"] < 2e-2
    assert row["stock_inductor_ms"] > 0 and row["ayla_b200_ms"] > 0
