"""Route ``aten.mm/addmm/bmm`` in ``torch.compile`` graphs to the sm_100a GEMM ops, with a
following relu / sigmoid / silu / gelu or a SwiGLU gate fused into the GEMM's epilogue.

Same contract as the reference's Inductor integration (ayla/torch_compile.py:652-775):
``install()`` claims contiguous NT-layout fp16/bf16 GEMMs on CUDA -- ``lhs`` contiguous,
``rhs`` a transposed view of a contiguous ``bt`` (strides ``(1, k)``, or ``(n*k, 1, k)`` for
bmm), static sizes, 1-D bias of length n with ``alpha == beta == 1`` -- and leaves
everything else to stock Inductor; ``uninstall()`` hands them back.  ``install()`` is
idempotent and registers all six ``jit_*`` ops up front (ayla/torch_compile.py:743-749).

The mechanism differs because the Inductor of this torch (2.11) has no ``user_lowerings``
hook (the reference's file does not import here): the claim is made by a post-grad FX
pass (``torch._inductor.config.post_grad_custom_post_pass``) that rewrites a claimed node
into a call of the functional form of the op, ``torch.ops.ayla.jit_{op}_{dtype}_fn(a, bt)``,
which Inductor then emits as an extern kernel call.  The pass carries a ``uuid`` so
Inductor's code cache keys on it.
"""

from __future__ import annotations

from functools import cache

import torch
from torch._inductor import config as inductor_config
from torch._inductor.custom_graph_pass import CustomGraphPass, get_hash_for_files

from .gemm_jit import (_SHORT_DTYPES, _TORCH_DTYPES, ACTIVATIONS, _op_name, gemm_jit_compiler, gemm_op,
                       select_gemm_schedule)
from .torch_custom_call import DEFAULT_NAMESPACE, OperandKind, make_torch_custom_call

aten = torch.ops.aten
_DTYPE_NAMES = {torch.float16: "float16", torch.bfloat16: "bfloat16"}


def gemm_fn_op(operation: str, dtype: str, namespace: str = DEFAULT_NAMESPACE,
               activation: str = "none", gated: bool = False) -> torch._ops.OpOverload:
    """Functional form ``(bias?, a, bt[, mul]) -> out`` of ``gemm_op`` / ``gemm_act_op`` /
    ``gemm_act_mul_op`` / (``gated="row"``) ``gemm_act_rowmul_op`` (the result is allocated by the
    op), the form a functional FX graph can hold.  Counterpart of the reference's allocating ops (ayla/gemm_collection/dynamic_m.py:90-121).
    Cached: one op per distinct argument tuple, however the defaults were spelled."""
    return _gemm_fn_op(operation, dtype, namespace, activation, gated if gated == "row" else bool(gated))


@cache
def _gemm_fn_op(operation: str, dtype: str, namespace: str, activation: str,
                gated: bool | str) -> torch._ops.OpOverload:
    compiler = gemm_jit_compiler(operation, dtype, activation, gated)

    def infer(*inputs: torch.Tensor):
        a, bt = (inputs[-3], inputs[-2]) if gated else (inputs[-2], inputs[-1])
        return [(*a.shape[:-1], bt.shape[-2])]

    inputs = (3 if operation == "addmm" else 2) + (1 if gated else 0)
    return make_torch_custom_call(
        compiler,
        [OperandKind.R] * inputs + [OperandKind.RESULT],
        namespace=namespace,
        name=f"{_op_name(operation, dtype, activation, gated)}_fn",
        infer_result_shapes=infer,
    )


@cache
def swiglu_fn_op(dtype: str, namespace: str = DEFAULT_NAMESPACE) -> torch._ops.OpOverload:
    """Functional form ``(x, w_gate, w_up) -> out`` of the fused SwiGLU op."""
    from .swiglu import swiglu_compiler

    return make_torch_custom_call(
        swiglu_compiler(dtype),
        [OperandKind.R] * 3 + [OperandKind.RESULT],
        namespace=namespace,
        name=f"swiglu_{_SHORT_DTYPES[dtype]}_fn",
        infer_result_shapes=lambda x, w_gate, w_up: [(x.shape[0], w_gate.shape[0])],
    )


def _static_ints(values) -> tuple[int, ...] | None:
    out = []
    for v in values:
        if not isinstance(v, int):
            return None
        out.append(v)
    return tuple(out)


def _val(node):
    val = node.meta.get("val") if isinstance(node, torch.fx.Node) else None
    return val if isinstance(val, torch.Tensor) else None


def _claim(operation: str, lhs, rhs, bias=None) -> tuple[str, tuple[int, ...]] | None:
    """Decide whether this GEMM is ours: returns (dtype name, (batch?, m, n, k)) or None."""
    lv, rv = _val(lhs), _val(rhs)
    if lv is None or rv is None:
        return None
    dtype = _DTYPE_NAMES.get(lv.dtype)
    if lv.device.type != "cuda" or dtype is None or rv.dtype != lv.dtype or rv.device != lv.device:
        return None
    rank = 3 if operation == "bmm" else 2
    if lv.dim() != rank or rv.dim() != rank:
        return None
    lsize, rsize = _static_ints(lv.shape), _static_ints(rv.shape)
    lstride, rstride = _static_ints(lv.stride()), _static_ints(rv.stride())
    if None in (lsize, rsize, lstride, rstride):
        return None  # dynamic shapes are left to Inductor
    *batch, m, k = lsize
    n = rsize[-1]
    if rsize[-2] != k or list(rsize[:-2]) != batch:
        return None
    # A row-major a and a column-major b: a @ bt^T with contiguous bt.
    contiguous = (m * k, k, 1)[-rank:]
    if lstride != contiguous:
        return None
    if rstride != (*([n * k] if batch else []), 1, k):
        return None
    if bias is not None:
        bv = _val(bias)
        if bv is None or bv.dtype != lv.dtype or _static_ints(bv.shape) != (n,) or bv.device != lv.device:
            return None
        if _static_ints(bv.stride()) != (1,):
            return None
    if select_gemm_schedule(operation, dtype, m, n, k, *batch) is None:
        return None
    return dtype, (*batch, m, n, k)


prims = torch.ops.prims


def _strip_convert(node, dtype=None):
    """The input of a ``convert_element_type`` node (to ``dtype`` if given), else the node."""
    if (isinstance(node, torch.fx.Node) and node.op == "call_function"
            and node.target is prims.convert_element_type.default
            and (dtype is None or node.args[1] == dtype)):
        return node.args[0]
    return node


def _silu_source(node):
    """If ``node`` computes silu(g), return (g, nodes of the chain); else None.

    Recognises ``aten.silu`` and the two forms Inductor's decompositions leave behind for
    16-bit inputs: ``cvt16(div(cvt32(g), add(exp(neg(cvt32(g))), 1)))`` and
    ``cvt16(mul(cvt32(g), sigmoid(cvt32(g))))``."""
    if not isinstance(node, torch.fx.Node) or node.op != "call_function":
        return None
    if node.target is aten.silu.default:
        return node.args[0], [node]
    chain = [node]
    inner = _strip_convert(node)
    if inner is not node:
        chain.append(inner)
    if not isinstance(inner, torch.fx.Node) or inner.op != "call_function":
        return None
    if inner.target is aten.div.Tensor:
        num, den = inner.args
        if not (isinstance(den, torch.fx.Node) and den.target is aten.add.Tensor):
            return None
        exp, one = den.args[0], den.args[1]
        if one != 1 or not (isinstance(exp, torch.fx.Node) and exp.target is aten.exp.default):
            return None
        neg = exp.args[0]
        if not (isinstance(neg, torch.fx.Node) and neg.target is aten.neg.default):
            return None
        src_a, src_b = _strip_convert(num, torch.float32), _strip_convert(neg.args[0], torch.float32)
        if src_a is not src_b:
            return None
        chain += [den, exp, neg] + [n for n in (num, neg.args[0]) if n is not src_a]
        return src_a, chain
    if inner.target is aten.mul.Tensor:
        a, b = inner.args
        for x, sig in ((a, b), (b, a)):
            if isinstance(sig, torch.fx.Node) and sig.target is aten.sigmoid.default:
                src_a, src_b = _strip_convert(x, torch.float32), _strip_convert(sig.args[0], torch.float32)
                if src_a is src_b:
                    chain += [sig] + [n for n in (x, sig.args[0]) if n is not src_a]
                    return src_a, chain
    return None


def _only_used_by(node, allowed) -> bool:
    return all(user in allowed for user in node.users)


def _swiglu_pays(m: int, n: int, sm_count: int = 148) -> bool:
    """Whether the fused SwiGLU op is the better choice for ``m`` rows and ``n`` output columns.
    With a few rows the op is a weight stream over ``ceil(n / 128)`` column tiles, one per SM and
    no k-split: when those tiles fill the last wave of SMs badly (156 tiles on 148 SMs) the plain
    GEMM on the concatenated weight, which has small-M schedules, plus Inductor's elementwise
    epilogue is faster (measured at 8 rows, n = 19968, k = 6656: 112 us fused, 92 us unfused; at
    n = 14336: 42 us fused, 46 us unfused)."""
    if m > 128:
        return True
    tiles = -(-n // 128)
    waves = -(-tiles // sm_count)
    return waves == 1 or tiles / (waves * sm_count) >= 0.7


def route_swiglu(graph: torch.fx.Graph) -> int:
    """Rewrite ``silu(x @ wg.T) * (x @ wu.T)`` (two claimed mm nodes on the same ``x``) into
    one call of the fused SwiGLU op.  The reference only has the pieces of this fusion
    (ayla/torch_compile.py:532-547 fuses a lone sigmoid; multi-source epilogues are a TODO,
    ayla/passes/promote_buffers.py:626-628)."""
    rewritten = 0
    for node in list(graph.nodes):
        if node.op != "call_function" or node.target is not aten.mul.Tensor or len(node.args) != 2:
            continue
        for act, up in (node.args, node.args[::-1]):
            found = _silu_source(act)
            if found is None or not isinstance(up, torch.fx.Node):
                continue
            gate, chain = found
            if not (isinstance(gate, torch.fx.Node) and gate.target is aten.mm.default
                    and up.target is aten.mm.default and gate is not up):
                continue
            x, wg_t = gate.args
            x2, wu_t = up.args
            if x is not x2:
                continue
            claim_g, claim_u = _claim("mm", x, wg_t), _claim("mm", x, wu_t)
            if claim_g is None or claim_u is None or claim_g != claim_u:
                continue  # same dtype and the same (m, n, k), or it is not one SwiGLU
            if not _swiglu_pays(claim_g[1][0], claim_g[1][1]):
                continue
            members = set(chain) | {node}
            if not (_only_used_by(gate, members) and _only_used_by(up, {node})
                    and all(_only_used_by(n, members) for n in chain)):
                continue  # an intermediate is needed elsewhere: leave the graph alone
            dtype = claim_g[0]
            with graph.inserting_before(node):
                wg = graph.call_function(aten.permute.default, (wg_t, [1, 0]))
                wg.meta["val"] = _val(wg_t).permute(1, 0)
                wu = graph.call_function(aten.permute.default, (wu_t, [1, 0]))
                wu.meta["val"] = _val(wu_t).permute(1, 0)
                new = graph.call_function(swiglu_fn_op(dtype), (x, wg, wu))
                new.meta.update({k: v for k, v in node.meta.items() if k != "original_aten"})
            node.replace_all_uses_with(new)
            graph.erase_node(node)
            rewritten += 1
            break
    if rewritten:
        graph.eliminate_dead_code()
    return rewritten


def _is_call(node, target) -> bool:
    return isinstance(node, torch.fx.Node) and node.op == "call_function" and node.target is target


def _close(value, want: float) -> bool:
    return isinstance(value, (int, float)) and abs(float(value) - want) < 1e-6


def _gelu_source(node):
    """If ``node`` computes the erf form of gelu(x) as Inductor's decompositions leave it for
    16-bit inputs, ``cvt16(mul(mul(x32, 0.5), add(erf(mul(x32, 1/sqrt 2)), 1)))``, return
    (x, chain); else None."""
    chain = [node]
    inner = _strip_convert(node)
    if inner is not node:
        chain.append(inner)
    if not _is_call(inner, aten.mul.Tensor):
        return None
    for half, one_plus in (inner.args, inner.args[::-1]):
        if not (_is_call(half, aten.mul.Tensor) and _is_call(one_plus, aten.add.Tensor)):
            continue
        if not (_close(half.args[1], 0.5) and _close(one_plus.args[1], 1.0)):
            continue
        erf = one_plus.args[0]
        if not (_is_call(erf, aten.erf.default) and _is_call(erf.args[0], aten.mul.Tensor)):
            continue
        scaled = erf.args[0]
        if not _close(scaled.args[1], 0.7071067811865476):
            continue
        x32 = half.args[0]
        if scaled.args[0] is not x32:
            continue
        src = _strip_convert(x32, torch.float32)
        chain += [half, one_plus, erf, scaled] + ([x32] if x32 is not src else [])
        return src, chain
    return None


def _activation_source(node):
    """If ``node`` is an activation this library fuses, return (name, input node, nodes of the
    chain); else None."""
    if not isinstance(node, torch.fx.Node) or node.op != "call_function":
        return None
    if node.target is aten.relu.default:
        return "relu", node.args[0], [node]
    if node.target is aten.gelu.default:
        approximate = node.kwargs.get("approximate", "none")
        return ("gelu_tanh" if approximate == "tanh" else "gelu"), node.args[0], [node]
    inner = _strip_convert(node)
    if _is_call(inner, aten.sigmoid.default):
        src = _strip_convert(inner.args[0], torch.float32)
        chain = [node] + ([inner] if inner is not node else []) + ([inner.args[0]] if inner.args[0] is not src else [])
        return "sigmoid", src, chain
    found = _silu_source(node)
    if found is not None:
        return "silu", found[0], found[1]
    found = _gelu_source(node)
    if found is not None:
        return "gelu", found[0], found[1]
    return None


def _gemm_operands(node):
    """(operation, lhs, rhs, bias) of an aten GEMM node this pass may claim, else None."""
    if _is_call(node, aten.mm.default) and len(node.args) == 2:
        return "mm", node.args[0], node.args[1], None
    if _is_call(node, aten.bmm.default) and len(node.args) == 2:
        return "bmm", node.args[0], node.args[1], None
    if _is_call(node, aten.addmm.default) and len(node.args) == 3:
        if node.kwargs.get("beta", 1) != 1 or node.kwargs.get("alpha", 1) != 1:
            return None
        return "addmm", node.args[1], node.args[2], node.args[0]
    return None


def route_activations(graph: torch.fx.Graph) -> int:
    """Rewrite ``act(gemm)`` -- relu, sigmoid, silu or gelu applied to a claimed mm/addmm/bmm
    that nothing else reads -- into one call of the op with the activation fused into its
    epilogue.  The reference fuses a lone sigmoid onto its fixed 4096-cube matmul under the
    same single-reader condition (ayla/torch_compile.py:532-547)."""
    rewritten = 0
    for node in list(graph.nodes):
        found = _activation_source(node)
        if found is None:
            continue
        activation, src, chain = found
        operands = _gemm_operands(src)
        if operands is None:
            continue
        nv, sv = _val(node), _val(src)
        if nv is None or sv is None or nv.dtype != sv.dtype:
            continue  # an fp32 step inside a chain: the match is made at the chain's last node
        operation, lhs, rhs, bias = operands
        claim = _claim(operation, lhs, rhs, bias)
        if claim is None:
            continue
        members = set(chain)
        if not (_only_used_by(src, members) and all(_only_used_by(n, members) for n in chain if n is not node)):
            continue  # the plain product (or a step of the chain) is needed elsewhere
        dtype = claim[0]
        with graph.inserting_before(node):
            perm = [0, 2, 1] if operation == "bmm" else [1, 0]
            bt = graph.call_function(aten.permute.default, (rhs, perm))
            bt.meta["val"] = _val(rhs).permute(perm)
            args = (lhs, bt) if bias is None else (bias, lhs, bt)
            new = graph.call_function(gemm_fn_op(operation, dtype, DEFAULT_NAMESPACE, activation), args)
            new.meta.update({k: v for k, v in node.meta.items() if k != "original_aten"})
        node.replace_all_uses_with(new)
        graph.erase_node(node)
        rewritten += 1
    if rewritten:
        graph.eliminate_dead_code()
    return rewritten


def route_gated(graph: torch.fx.Graph) -> int:
    """Rewrite ``act(gemm) * other`` (or ``gemm * other``) -- a claimed mm/addmm/bmm that only this
    product reads, times a contiguous tensor of the result's shape and type -- into one call of the
    gated op.  This is the producer half of the gated-attention output projection the reference's
    pass matches without having a kernel for it (ayla/torch_compile.py:288-504)."""
    rewritten = 0
    for node in list(graph.nodes):
        if not _is_call(node, aten.mul.Tensor) or len(node.args) != 2:
            continue
        for lhs_arg, other in (node.args, node.args[::-1]):
            if not isinstance(lhs_arg, torch.fx.Node) or not isinstance(other, torch.fx.Node):
                continue
            found = _activation_source(lhs_arg)
            if found is not None:
                activation, src, chain = found
                fv, sv = _val(lhs_arg), _val(src)
                if fv is None or sv is None or fv.dtype != sv.dtype:
                    continue
            else:
                activation, src, chain = "none", lhs_arg, []
            operands = _gemm_operands(src)
            if operands is None or _gemm_operands(other) is not None:
                continue  # two products: that is SwiGLU's pattern, or not ours at all
            operation, lhs, rhs, bias = operands
            claim = _claim(operation, lhs, rhs, bias)
            ov, nv = _val(other), _val(node)
            if claim is None or ov is None or nv is None:
                continue
            shape, stride = _static_ints(ov.shape), _static_ints(ov.stride())
            if (ov.dtype != nv.dtype or _DTYPE_NAMES.get(ov.dtype) != claim[0] or shape is None
                    or shape != _static_ints(nv.shape) or stride != _static_ints(nv.new_empty(shape).stride())):
                continue  # broadcast, mixed types or a strided gate: leave it to Inductor
            members = set(chain) | {node}
            if not (_only_used_by(src, members) and all(_only_used_by(n, members) for n in chain)):
                continue
            with graph.inserting_before(node):
                perm = [0, 2, 1] if operation == "bmm" else [1, 0]
                bt = graph.call_function(aten.permute.default, (rhs, perm))
                bt.meta["val"] = _val(rhs).permute(perm)
                args = (lhs, bt, other) if bias is None else (bias, lhs, bt, other)
                new = graph.call_function(gemm_fn_op(operation, claim[0], DEFAULT_NAMESPACE, activation, True), args)
                new.meta.update({k: v for k, v in node.meta.items() if k != "original_aten"})
            node.replace_all_uses_with(new)
            graph.erase_node(node)
            rewritten += 1
            break
    if rewritten:
        graph.eliminate_dead_code()
    return rewritten


def _concat_halves(gate, up):
    """If ``gate`` and ``up`` are the two column halves of one 2-D ``aten.mm`` result, return
    (mm node, half width, nodes between the mm and the halves); else None.  Two spellings occur:
    ``chunk``/``split`` (``aten.split.Tensor`` + ``getitem`` 0 and 1) and the pair of slices
    ``aten.slice.Tensor(mm, 1, 0, n)`` / ``aten.slice.Tensor(mm, 1, n, end)`` that a captured
    decoder block holds (benchmarks/bench_torch_compile/corpus/muse_glimmer_block.py:42-50 of the
    reference)."""
    import operator

    if _is_call(gate, operator.getitem) and _is_call(up, operator.getitem):
        split = gate.args[0]
        if not (up.args[0] is split and gate.args[1] == 0 and up.args[1] == 1):
            return None
        if not _is_call(split, aten.split.Tensor) or not _is_call(split.args[0], aten.mm.default):
            return None
        mm = split.args[0]
        mv = _val(mm)
        if mv is None or mv.dim() != 2:
            return None
        n2 = mv.shape[-1]
        dim = split.args[2] if len(split.args) > 2 else 0
        if not isinstance(n2, int) or n2 % 2 or split.args[1] != n2 // 2 or dim not in (-1, 1):
            return None
        if not (_only_used_by(mm, {split}) and _only_used_by(split, {gate, up})):
            return None
        return mm, n2 // 2, [split]
    if _is_call(gate, aten.slice.Tensor) and _is_call(up, aten.slice.Tensor):
        mm = gate.args[0]
        if up.args[0] is not mm or not _is_call(mm, aten.mm.default):
            return None
        mv = _val(mm)
        if mv is None or mv.dim() != 2 or not isinstance(mv.shape[-1], int) or mv.shape[-1] % 2:
            return None
        n2 = mv.shape[-1]
        half = n2 // 2

        def bounds(node):
            dim = node.args[1] if len(node.args) > 1 else 0
            start = node.args[2] if len(node.args) > 2 else None
            end = node.args[3] if len(node.args) > 3 else None
            step = node.args[4] if len(node.args) > 4 else 1
            if dim not in (1, -1) or step != 1:
                return None
            start = 0 if start is None else start
            end = n2 if end is None else end
            if not isinstance(start, int) or not isinstance(end, int):
                return None
            return start, min(end, n2)

        if bounds(gate) != (0, half) or bounds(up) != (half, n2):
            return None
        if not _only_used_by(mm, {gate, up}):
            return None
        return mm, half, []
    return None


def route_swiglu_concat(graph: torch.fx.Graph) -> int:
    """Rewrite SwiGLU on a concatenated weight, ``g, u = (x @ w.T).chunk(2, -1); silu(g) * u``
    with ``w`` of shape ``[2 n, k]`` (the form real decoder blocks use,
    benchmarks/muse_glimmer_block.py:41-50 of the reference), into the fused SwiGLU op on the
    two row halves of ``w``.  The halves may be spelled as ``split`` + ``getitem`` or as two
    ``slice`` nodes of the product."""
    rewritten = 0
    for node in list(graph.nodes):
        if not _is_call(node, aten.mul.Tensor) or len(node.args) != 2:
            continue
        for act, up in (node.args, node.args[::-1]):
            found = _silu_source(act)
            if found is None or not isinstance(up, torch.fx.Node):
                continue
            gate, chain = found
            halves = _concat_halves(gate, up)
            if halves is None:
                continue
            mm, half, between = halves
            n2 = 2 * half
            x, w_t = mm.args
            claim = _claim("mm", x, w_t)
            if claim is None or half % 8 or not _swiglu_pays(claim[1][0], half):
                continue
            members = set(chain) | {node, gate, up, *between}
            if not (_only_used_by(up, {node}) and _only_used_by(gate, members)
                    and all(_only_used_by(n, members) for n in chain)):
                continue
            dtype = claim[0]
            with graph.inserting_before(node):
                w = graph.call_function(aten.permute.default, (w_t, [1, 0]))
                w.meta["val"] = _val(w_t).permute(1, 0)
                wg = graph.call_function(aten.slice.Tensor, (w, 0, 0, half))
                wg.meta["val"] = w.meta["val"][:half]
                wu = graph.call_function(aten.slice.Tensor, (w, 0, half, n2))
                wu.meta["val"] = w.meta["val"][half:]
                new = graph.call_function(swiglu_fn_op(dtype), (x, wg, wu))
                new.meta.update({k: v for k, v in node.meta.items() if k != "original_aten"})
            node.replace_all_uses_with(new)
            graph.erase_node(node)
            rewritten += 1
            break
    if rewritten:
        graph.eliminate_dead_code()
    return rewritten


def _constant_tensor(node, module) -> torch.Tensor | None:
    """The tensor a node denotes when it is a constant of the graph's module (a parameter that
    Inductor's freezing turned into an attribute), seen through ``permute``/``t`` views."""
    if not isinstance(node, torch.fx.Node):
        return None
    if node.op == "get_attr":
        value = module
        for part in str(node.target).split("."):
            value = getattr(value, part, None)
        return value if isinstance(value, torch.Tensor) else None
    if _is_call(node, aten.permute.default):
        inner = _constant_tensor(node.args[0], module)
        return None if inner is None else inner.permute(list(node.args[1]))
    if _is_call(node, aten.t.default):
        inner = _constant_tensor(node.args[0], module)
        return None if inner is None else inner.t()
    return None


def _rms_norm_source(node):
    """If ``node`` is ``x * rsqrt(mean(x^2, -1, keepdim) + eps) * g`` computed in fp32 and rounded to
    the type of ``x`` (the decomposition of ``rms_norm`` with a weight), return ``(x, rsqrt node, g)``."""
    val = _val(node)
    product = _strip_convert(node, val.dtype if val is not None else None)
    if not _is_call(product, aten.mul.Tensor) or len(product.args) != 2:
        return None
    for scaled, g in (product.args, product.args[::-1]):
        if not _is_call(scaled, aten.mul.Tensor) or len(scaled.args) != 2 or not isinstance(g, torch.fx.Node):
            continue
        for xf, r in (scaled.args, scaled.args[::-1]):
            if not _is_call(r, aten.rsqrt.default) or not isinstance(xf, torch.fx.Node):
                continue
            shifted = r.args[0]
            if not ((_is_call(shifted, aten.add.Scalar) or _is_call(shifted, aten.add.Tensor))
                    and isinstance(shifted.args[1], (int, float))):
                continue
            mean = shifted.args[0]
            xv = _val(xf)
            if not _is_call(mean, aten.mean.dim) or xv is None or xv.dtype != torch.float32:
                continue
            dims, keepdim = list(mean.args[1]), (mean.args[2] if len(mean.args) > 2 else False)
            if dims not in ([-1], [xv.dim() - 1]) or not keepdim:
                continue
            square = mean.args[0]
            squared = ((_is_call(square, aten.pow.Tensor_Scalar) and square.args[0] is xf and square.args[1] == 2)
                       or (_is_call(square, aten.mul.Tensor) and square.args[0] is xf and square.args[1] is xf))
            if not squared:
                continue
            x = _strip_convert(xf, torch.float32)
            if x is xf or val is None or _val(x) is None or _val(x).dtype != val.dtype:
                continue
            return x, r, g
    return None


def route_rmsnorm(graph: torch.fx.Graph) -> int:
    """Rewrite ``rms_norm(x, weight=g) @ W.T`` with constant ``g`` and ``W`` (Inductor freezing) into
    ``r * (x @ (W * g).T)``: ``g`` is folded into the projection weight once, here, and the per-row
    factor ``r = rsqrt(mean(x^2) + eps)`` multiplies the fp32 accumulator in the GEMM's epilogue
    (``gemm_act_rowmul_op``), so the normalised activations are neither written nor read back.  With
    weights that are graph inputs (no freezing) nothing is constant and the pattern is left alone."""
    module = graph.owning_module
    if module is None:
        return 0
    from .rmsnorm_linear import fold_norm_weight

    rewritten = 0
    for node in list(graph.nodes):
        if not _is_call(node, aten.mm.default) or len(node.args) != 2:
            continue
        lhs, rhs = node.args
        found = _rms_norm_source(lhs) if isinstance(lhs, torch.fx.Node) else None
        if found is None:
            continue
        x, r, g = found
        claim = _claim("mm", x, rhs)  # x has the shape, type and layout of the normalised activations
        g_const, w_const = _constant_tensor(g, module), _constant_tensor(rhs, module)
        rv = _val(rhs)
        if claim is None or g_const is None or w_const is None or rv is None:
            continue
        dtype, (m, n, k) = claim
        if tuple(w_const.shape) != (k, n) or tuple(g_const.shape) != (k,):
            continue
        name = f"_ayla_b200_folded_weight{rewritten}"
        while hasattr(module, name):
            name += "_"
        module.register_buffer(name, fold_norm_weight(w_const.t(), g_const).contiguous(), persistent=False)
        with graph.inserting_before(node):
            weight = graph.get_attr(name)
            weight.meta["val"] = rv.t().contiguous()
            factors = graph.call_function(prims.convert_element_type.default, (r, _TORCH_DTYPES[dtype]))
            factors.meta["val"] = _val(r).to(_TORCH_DTYPES[dtype])
            new = graph.call_function(gemm_fn_op("mm", dtype, DEFAULT_NAMESPACE, "none", "row"), (x, weight, factors))
            new.meta.update({key: v for key, v in node.meta.items() if key != "original_aten"})
        node.replace_all_uses_with(new)
        graph.erase_node(node)
        rewritten += 1
    if rewritten:
        graph.eliminate_dead_code()
    return rewritten


def route_gemms(graph: torch.fx.Graph) -> int:
    """Rewrite every claimed ``aten.mm/addmm/bmm`` node of ``graph``; returns how many."""
    rewritten = 0
    for node in list(graph.nodes):
        if node.op != "call_function":
            continue
        if node.target is aten.mm.default and len(node.args) == 2:
            operation, (lhs, rhs), bias = "mm", node.args, None
        elif node.target is aten.bmm.default and len(node.args) == 2:
            operation, (lhs, rhs), bias = "bmm", node.args, None
        elif node.target is aten.addmm.default and len(node.args) == 3:
            if node.kwargs.get("beta", 1) != 1 or node.kwargs.get("alpha", 1) != 1:
                continue
            operation, (bias, lhs, rhs) = "addmm", node.args
        else:
            continue
        claim = _claim(operation, lhs, rhs, bias)
        if claim is None:
            continue
        dtype, _ = claim
        op = gemm_fn_op(operation, dtype)
        with graph.inserting_before(node):
            # bt is the transposed view of rhs: contiguous by the stride check above.
            perm = [0, 2, 1] if operation == "bmm" else [1, 0]
            bt = graph.call_function(aten.permute.default, (rhs, perm))
            rv = _val(rhs)
            bt.meta["val"] = rv.permute(perm)
            args = (lhs, bt) if bias is None else (bias, lhs, bt)
            new = graph.call_function(op, args)
            new.meta.update({k: v for k, v in node.meta.items() if k != "original_aten"})
        node.replace_all_uses_with(new)
        graph.erase_node(node)
        rewritten += 1
    if rewritten:
        graph.eliminate_dead_code()
    return rewritten


class AylaRoutingPass(CustomGraphPass):
    """Post-grad pass: ours first, then whatever pass was installed before."""

    def __init__(self, previous=None):
        self.previous = previous

    def __call__(self, graph: torch.fx.Graph) -> None:
        route_swiglu(graph)  # first: it consumes two mm nodes route_gemms would claim
        route_swiglu_concat(graph)
        route_rmsnorm(graph)
        route_gated(graph)
        route_activations(graph)
        route_gemms(graph)
        if self.previous is not None:
            self.previous(graph)

    def uuid(self):
        previous = self.previous.uuid() if isinstance(self.previous, CustomGraphPass) else None
        return ("ayla_b200.routing", get_hash_for_files((__file__,)), previous)


_installed: AylaRoutingPass | None = None


def emittable_ops() -> list[tuple]:
    """Every functional op a rewrite of this pass can put into a graph, as argument tuples of
    ``gemm_fn_op`` (``("swiglu", dtype)`` for the SwiGLU op): each operation and dtype, plain,
    with each activation ``_activation_source`` can name, and each of those with a gate."""
    ops: list[tuple] = []
    for dtype in _TORCH_DTYPES:
        ops.append(("swiglu", dtype))
        for operation in ("mm", "addmm", "bmm"):
            for activation in ACTIVATIONS:
                ops.append((operation, dtype, DEFAULT_NAMESPACE, activation, False))
                ops.append((operation, dtype, DEFAULT_NAMESPACE, activation, True))
        ops.append(("mm", dtype, DEFAULT_NAMESPACE, "none", "row"))
    return ops


def install() -> None:
    """Claim the GEMMs.  Idempotent."""
    global _installed
    # Register every op the pass can emit up front: on a hit in Inductor's code cache the pass does
    # not run in this process, and the cached code calls torch.ops.ayla.* by name.
    for operation in ("mm", "addmm", "bmm"):
        for dtype in _TORCH_DTYPES:
            gemm_op(operation, dtype)
    for spec in emittable_ops():
        if spec[0] == "swiglu":
            swiglu_fn_op(spec[1])
        else:
            gemm_fn_op(*spec)
    current = inductor_config.post_grad_custom_post_pass
    if _installed is not None and current is _installed:
        return
    _installed = AylaRoutingPass(previous=current)
    inductor_config.post_grad_custom_post_pass = _installed


def uninstall() -> None:
    """Hand the GEMMs back.  Stands down if someone else has replaced the pass since."""
    global _installed
    if _installed is None:
        return
    if inductor_config.post_grad_custom_post_pass is _installed:
        inductor_config.post_grad_custom_post_pass = _installed.previous
    _installed = None
