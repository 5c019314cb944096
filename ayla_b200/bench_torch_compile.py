"""Whole-graph comparison: a decoder block compiled by stock Inductor against the same block
compiled with this backend's routing installed.

    python -m ayla_b200.bench_torch_compile [--tokens 8,512,4096] [--layers 4] [--hidden 4096] [--ffn 14336]
    python -m ayla_b200.bench_torch_compile --corpus [--tokens 8,512]

``--corpus`` runs the forms of the reference's own whole-graph corpus
(benchmarks/bench_torch_compile/corpus/): a GEMM with a sigmoid on its output (the epilogue-fusion
case, corpus/gemm_sigmoid.py) and a decoder block body with a gated attention output projection,
RMSNorms with a ``1 + w`` scale, SwiGLU on a concatenated weight spelled as two slices of the
product, and a fused QKV projection (the structure of corpus/muse_glimmer_block.py, restated here as
ordinary PyTorch code with synthetic weights; sizes: hidden 6656, attention 4096, FFN 19968).  Per
entry it prints the three rows the reference's driver prints (benchmarks/bench_torch_compile/
bench_torch_compile.py:44-57): eager, compiled by stock Inductor, and compiled with the routing
installed, each arm with Inductor's caches disabled, plus the geometric mean of stock / routed.

Counterpart of the reference's whole-graph drivers (benchmarks/bench_torch_compile.py and
benchmarks/bench_better_benchmark.py: one arm per backend, a private Inductor cache per arm,
same inputs, speed-up per model).  The model is a synthetic stand-in with the layer shapes of an
8B-class decoder (RMSNorm, fused QKV projection, causal attention, output projection, SwiGLU MLP
on a concatenated gate/up weight, residuals), random weights, bf16, inference only: every GEMM in
it has the NT layout the routing claims, and the MLP is the pattern the SwiGLU fusion targets.
Each arm is compiled in a fresh Dynamo state with Inductor's caches disabled, warmed, captured in
a CUDA graph and timed with CUDA events; one JSON line per token count is printed.
"""

from __future__ import annotations

import argparse
import json
import math
import statistics

import torch
import torch.nn.functional as F
from torch._inductor import config as inductor_config

from . import torch_compile as routing


class DecoderBlock(torch.nn.Module):
    def __init__(self, hidden: int, ffn: int, heads: int, kv_heads: int, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.heads, self.kv_heads, self.head_dim = heads, kv_heads, hidden // heads
        qkv = (heads + 2 * kv_heads) * self.head_dim

        def weight(rows, cols):
            return torch.nn.Parameter((torch.randn(rows, cols, device=device) * cols ** -0.5).to(dtype),
                                      requires_grad=False)

        self.norm1 = torch.nn.Parameter(torch.ones(hidden, device=device, dtype=dtype), requires_grad=False)
        self.norm2 = torch.nn.Parameter(torch.ones(hidden, device=device, dtype=dtype), requires_grad=False)
        self.w_qkv = weight(qkv, hidden)
        self.w_o = weight(hidden, heads * self.head_dim)
        self.w_gate_up = weight(2 * ffn, hidden)
        self.w_down = weight(hidden, ffn)

    @staticmethod
    def rms_norm(x, scale):
        x32 = x.float()
        return (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype) * scale

    def forward(self, x):  # x: [tokens, hidden], one sequence
        tokens = x.shape[0]
        h = self.rms_norm(x, self.norm1)
        qkv = torch.mm(h, self.w_qkv.t())
        q, k, v = qkv.split([self.heads * self.head_dim, self.kv_heads * self.head_dim,
                             self.kv_heads * self.head_dim], dim=-1)
        q = q.view(tokens, self.heads, self.head_dim).transpose(0, 1)
        k = k.view(tokens, self.kv_heads, self.head_dim).transpose(0, 1)
        v = v.view(tokens, self.kv_heads, self.head_dim).transpose(0, 1)
        rep = self.heads // self.kv_heads
        k = k.repeat_interleave(rep, dim=0)
        v = v.repeat_interleave(rep, dim=0)
        attn = F.scaled_dot_product_attention(q[None], k[None], v[None], is_causal=True)[0]
        attn = attn.transpose(0, 1).reshape(tokens, self.heads * self.head_dim)
        x = x + torch.mm(attn, self.w_o.t())
        h = self.rms_norm(x, self.norm2)
        gate, up = torch.mm(h, self.w_gate_up.t()).chunk(2, dim=-1)
        return x + torch.mm(F.silu(gate) * up, self.w_down.t())


class Decoder(torch.nn.Module):
    def __init__(self, layers: int, hidden: int, ffn: int, heads: int, kv_heads: int):
        super().__init__()
        self.blocks = torch.nn.ModuleList(DecoderBlock(hidden, ffn, heads, kv_heads) for _ in range(layers))

    def forward(self, x):
        for block in self.blocks:
            x = block(x)
        return x


def _time_graph(fn, x, rounds: int = 7, launches: int = 4) -> tuple[float, torch.Tensor]:
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream), torch.no_grad():
        for _ in range(3):
            out = fn(x)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(launches):
                out = fn(x)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        samples = []
        for _ in range(rounds):
            start.record(stream)
            graph.replay()
            stop.record(stream)
            stream.synchronize()
            samples.append(start.elapsed_time(stop) / launches)
    return statistics.median(samples), out.clone()


def _compile_arm(model, x, routed: bool):
    from torch._inductor.utils import run_and_get_code

    torch._dynamo.reset()
    if routed:
        routing.install()
    try:
        with torch.no_grad(), inductor_config.patch(force_disable_caches=True):
            compiled = torch.compile(model, fullgraph=True, dynamic=False)
            _, code = run_and_get_code(compiled, x)
            ms, out = _time_graph(compiled, x)
    finally:
        if routed:
            routing.uninstall()
    text = "\n".join(code)
    counts = {name: text.count(f"torch.ops.ayla.{name}") for name in ("jit_mm_bf16_fn", "swiglu_bf16_fn")}
    return ms, out, counts


def run(tokens: int, layers: int, hidden: int, ffn: int, heads: int, kv_heads: int) -> dict:
    torch.manual_seed(0)
    model = Decoder(layers, hidden, ffn, heads, kv_heads)
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    stock_ms, stock_out, _ = _compile_arm(model, x, routed=False)
    ours_ms, ours_out, counts = _compile_arm(model, x, routed=True)
    diff = (ours_out.float() - stock_out.float())
    rel = float(diff.norm() / stock_out.float().norm())
    head_dim = hidden // heads
    gemm_flops = 2.0 * tokens * hidden * ((heads + 2 * kv_heads) * head_dim + heads * head_dim + 3 * ffn) * layers
    return {"model": f"decoder x{layers} hidden={hidden} ffn={ffn} heads={heads}/{kv_heads}", "tokens": tokens,
            "stock_inductor_ms": stock_ms, "ayla_b200_ms": ours_ms, "speedup": stock_ms / ours_ms,
            "routed_calls_in_generated_code": counts, "fro_rel_between_arms": rel,
            "gemm_tflops_ayla_b200": gemm_flops / ours_ms / 1e9, "data": "synthetic, random weights, bf16"}


# ------------------------------------------------------------------ the reference's corpus forms

def gemm_sigmoid_entry(m: int = 4096, k: int = 4096, n: int = 4096):
    """A GEMM with a sigmoid on its output; the weight is ``[n, k]`` as a weight is stored."""
    torch.manual_seed(0)
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    bt = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    return f"gemm_sigmoid {m}x{k}x{n} bf16", (lambda x, w: torch.sigmoid(x @ w.t())), (a, bt)


def gated_pair_entry(tokens: int = 8, hidden: int = 6656, attn: int = 4096):
    """The gated attention output projection alone, at the decode shape the reference's matcher
    names (m = 8, n = 6656, k = 4096, ayla/torch_compile.py:494-504): ``mm -> sigmoid -> mul -> mm``.
    Routed, the first three are one launch (``jit_mm_sigmoid_mul``) and the consumer a second one."""
    torch.manual_seed(2)
    h = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    v = torch.randn(tokens, attn, device="cuda").to(torch.bfloat16)
    w_gate = (torch.randn(attn, hidden, device="cuda") * hidden ** -0.5).to(torch.bfloat16)
    w_o = (torch.randn(hidden, attn, device="cuda") * attn ** -0.5).to(torch.bfloat16)
    return (f"gated attention output projection, {tokens} tokens ({attn} -> {hidden})",
            (lambda h, v, w_gate, w_o: (torch.sigmoid(h @ w_gate.t()) * v) @ w_o.t()), (h, v, w_gate, w_o))


def rmsnorm_projection_entry(tokens: int = 4096, hidden: int = 4096, out_features: int = 6144):
    """An RMSNorm followed by a projection (a decoder block's pre-norm and fused QKV projection) as
    a module whose weights Inductor's freezing turns into constants: routed, the norm weight is
    folded into the projection weight at compile time and the row factors are applied in the GEMM's
    epilogue (``jit_mm_rowmul``), so the normalised activations never exist in memory."""

    class NormThenProject(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.g = torch.nn.Parameter(1.0 + 0.1 * torch.randn(hidden))
            self.w = torch.nn.Parameter(torch.randn(out_features, hidden) * hidden ** -0.5)

        def forward(self, x):
            return F.linear(F.rms_norm(x, (hidden,), self.g, 1e-5), self.w)

    torch.manual_seed(3)
    block = NormThenProject().to(device="cuda", dtype=torch.bfloat16).eval()
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    return (f"RMSNorm + projection, frozen weights, {tokens} tokens ({hidden} -> {out_features})", block, (x,),
            {"freezing": True})


def gated_block_fn(attn: int, ffn: int, kv: int):
    """The block body as a function of its activations and weights (see ``gated_block_entry``)."""

    def norm(x, w, eps):
        x32 = x.float()
        return (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + 1)).to(torch.bfloat16)

    def block(h, attn_out, residual, w_gate, w_o, w_gate_up, w_down, w_qkv, n1, n2, n3, n4):
        gated = torch.sigmoid(h @ w_gate.t()) * attn_out
        x = residual + norm(gated @ w_o.t(), n1, 1e-8)
        both = norm(x, n2, 1e-5) @ w_gate_up.t()
        act = F.silu(both[:, :ffn]) * both[:, ffn:]
        x = x + norm(act @ w_down.t(), n3, 1e-8)
        pre = norm(x, n4, 1e-5)
        q, k, v = (pre @ w_qkv.t()).split([attn, kv, kv], dim=-1)
        return q, k, v, pre, x

    return block


def gated_block_entry(tokens: int, hidden: int = 6656, attn: int = 4096, ffn: int = 19968, kv: int = 256):
    """The body of a decoder block around its two attention halves: gated output projection of the
    previous attention (``sigmoid(h @ Wg.T) * attn_out`` then the output projection), post-norm and
    residual, pre-norm, SwiGLU MLP on a concatenated gate/up weight read as two slices, post-norm and
    residual, pre-norm, and the fused QKV projection of the next attention."""
    torch.manual_seed(1)

    def weight(rows, cols):
        return (torch.randn(rows, cols, device="cuda") * cols ** -0.5).to(torch.bfloat16)

    def vector(size):
        return (torch.randn(size, device="cuda") * 0.02).to(torch.bfloat16)

    params = dict(w_gate=weight(attn, hidden), w_o=weight(hidden, attn), w_gate_up=weight(2 * ffn, hidden),
                  w_down=weight(hidden, ffn), w_qkv=weight(attn + 2 * kv, hidden),
                  n1=vector(hidden), n2=vector(hidden), n3=vector(hidden), n4=vector(hidden))
    h = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    attn_out = torch.randn(tokens, attn, device="cuda").to(torch.bfloat16)
    residual = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)

    block = gated_block_fn(attn, ffn, kv)
    args = (h, attn_out, residual, *params.values())
    return f"gated decoder block body, {tokens} tokens, hidden {hidden}, ffn {ffn}", block, args


def _time_callable(fn, args, rounds: int = 7, launches: int = 4) -> float:
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream), torch.no_grad():
        for _ in range(3):
            fn(*args)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(launches):
                fn(*args)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        samples = []
        for _ in range(rounds):
            start.record(stream)
            graph.replay()
            stop.record(stream)
            stream.synchronize()
            samples.append(start.elapsed_time(stop) / launches)
    return statistics.median(samples)


def run_corpus_entry(name: str, fn, args, options: dict | None = None) -> dict:
    """The reference driver's three rows for one entry; ``options`` are Inductor settings both
    compiled arms run under (``{"freezing": True}`` for an entry whose weights are module parameters)."""
    options = dict(options or {})
    from torch._inductor.utils import run_and_get_code

    def first(result):
        return result[0] if isinstance(result, (tuple, list)) else result

    row: dict = {"entry": name, "data": "synthetic, random weights, bf16"}
    with torch.no_grad():
        row["eager_ms"] = _time_callable(fn, args)
        reference = first(fn(*args)).float()
    for arm, routed in (("compiled", False), ("ayla_compiled", True)):
        torch._dynamo.reset()
        if routed:
            routing.install()
        try:
            with torch.no_grad(), inductor_config.patch(force_disable_caches=True, **options):
                # Two lambdas, not one: Dynamo caches on the code object.  A module is compiled as
                # itself, so that freezing finds its parameters.
                target = fn if isinstance(fn, torch.nn.Module) else (
                    (lambda *a: fn(*a)) if routed else (lambda *b: fn(*b)))
                compiled = torch.compile(target, fullgraph=True, dynamic=False)
                _, code = run_and_get_code(compiled, *args)
                row[f"{arm}_ms"] = _time_callable(compiled, args)
                got = first(compiled(*args)).float()
        finally:
            if routed:
                routing.uninstall()
        row[f"{arm}_fro_rel_vs_eager"] = float((got - reference).norm() / reference.norm())
        if routed:
            text = "\n".join(code)
            row["routed_calls_in_generated_code"] = {
                op: text.count(f"torch.ops.ayla.{op}") for op in
                ("jit_mm_bf16_fn", "jit_mm_sigmoid_bf16_fn", "jit_mm_sigmoid_mul_bf16_fn", "jit_mm_rowmul_bf16_fn",
                 "swiglu_bf16_fn")}
            row["triton_matmuls_left"] = text.count("triton_tem_") + text.count("extern_kernels.mm(")
    row["speedup_vs_stock_inductor"] = row["compiled_ms"] / row["ayla_compiled_ms"]
    return row


def run_corpus(token_counts) -> list[dict]:
    entries = ([gemm_sigmoid_entry(), gated_pair_entry(), rmsnorm_projection_entry()]
               + [gated_block_entry(t) for t in token_counts])
    rows = []
    for name, fn, args, *options in entries:
        rows.append(run_corpus_entry(name, fn, args, *options))
        print(json.dumps(rows[-1]), flush=True)
        del fn, args
        torch.cuda.empty_cache()
    geomean = math.exp(sum(math.log(r["speedup_vs_stock_inductor"]) for r in rows) / len(rows))
    print(json.dumps({"geomean_stock_over_routed": geomean, "entries": len(rows)}), flush=True)
    return rows


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--corpus", action="store_true", help="run the reference's corpus forms instead")
    parser.add_argument("--tokens", default=None)
    parser.add_argument("--layers", type=int, default=4)
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--ffn", type=int, default=14336)
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    args = parser.parse_args()
    if args.corpus:
        run_corpus([int(t) for t in (args.tokens or "8,512").split(",")])
        return
    for tokens in (int(t) for t in (args.tokens or "8,512,4096").split(",")):
        print(json.dumps(run(tokens, args.layers, args.hidden, args.ffn, args.heads, args.kv_heads)), flush=True)


if __name__ == "__main__":
    main()
