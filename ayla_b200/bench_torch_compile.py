"""Whole-graph comparison: a decoder block compiled by stock Inductor against the same block
compiled with this backend's routing installed.

    python -m ayla_b200.bench_torch_compile [--tokens 8,512,4096] [--layers 4] [--hidden 4096] [--ffn 14336]

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


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--tokens", default="8,512,4096")
    parser.add_argument("--layers", type=int, default=4)
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--ffn", type=int, default=14336)
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    args = parser.parse_args()
    for tokens in (int(t) for t in args.tokens.split(",")):
        print(json.dumps(run(tokens, args.layers, args.hidden, args.ffn, args.heads, args.kv_heads)), flush=True)


if __name__ == "__main__":
    main()
