"""Launch one benchmark config a few times and exit -- the command profiled with ncu.

    python -m ayla_b200.profile_case C1 [--launches 6] [--schedule '{"tile_n":256,...}']

Configs: C1, C2a, C2b, C3a, C3b, C4 (SwiGLU), or ``mm:M,N,K`` / ``addmm:M,N,K`` /
``bmm:B,M,N,K`` for an arbitrary shape.  Inputs are random (timing and counters do not
depend on the values); nothing is checked here.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import _lib
from .gemm_jit import select_gemm_schedule

NAMED = {
    "C1": ("mm", 1, 4096, 4096, 4096),
    "C2a": ("addmm", 1, 8192, 768, 768),
    "C2b": ("addmm", 1, 256, 1024, 16384),
    "C3a": ("bmm", 64, 2048, 2048, 128),
    "C3b": ("bmm", 64, 2048, 128, 2048),
    "C4": ("swiglu", 1, 8192, 14336, 4096),
}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("config")
    parser.add_argument("--launches", type=int, default=6)
    parser.add_argument("--schedule", default=None)
    parser.add_argument("--dtype", default="bfloat16")
    args = parser.parse_args()
    if args.config in NAMED:
        op, batch, m, n, k = NAMED[args.config]
    else:
        op, dims = args.config.split(":")
        values = [int(v) for v in dims.split(",")]
        batch, (m, n, k) = (values[0], values[1:]) if op == "bmm" else (1, values)
    dev = "cuda:0"
    _lib.init(0)
    td = torch.bfloat16 if args.dtype == "bfloat16" else torch.float16
    stream = torch.cuda.current_stream().cuda_stream
    cfg = _lib.Config.from_dict(json.loads(args.schedule)) if args.schedule else None
    if op == "swiglu":
        x = torch.randn(m, k, device=dev).to(td)
        wg = (torch.randn(n, k, device=dev) * 0.02).to(td)
        wu = (torch.randn(n, k, device=dev) * 0.02).to(td)
        out = torch.empty(m, n, device=dev, dtype=td)
        for _ in range(args.launches):
            _lib.swiglu(args.dtype, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), out.data_ptr(), m, n, k, cfg, 0, stream)
    else:
        lead = (batch,) if op == "bmm" else ()
        a = torch.randn((*lead, m, k), device=dev).to(td)
        bt = (torch.randn((*lead, n, k), device=dev) * k ** -0.5).to(td)
        bias = torch.randn(n, device=dev).to(td)
        out = torch.empty((*lead, m, n), device=dev, dtype=td)
        if cfg is None:
            cfg = _lib.Config.from_dict(select_gemm_schedule(op, args.dtype, m, n, k, batch).builder_config)
        need = _lib.workspace_bytes(cfg, op, batch, m, n, k)
        ws = torch.zeros(max(need, 16), dtype=torch.uint8, device=dev)
        for _ in range(args.launches):
            _lib.gemm(op, args.dtype, bias.data_ptr() if op == "addmm" else 0, a.data_ptr(), bt.data_ptr(),
                      out.data_ptr(), batch, m, n, k, cfg, ws.data_ptr(), ws.numel(), 0, stream)
    torch.cuda.synchronize()
    print(f"{args.config}: {args.launches} launches of {op} {batch}x{m}x{n}x{k} done")


if __name__ == "__main__":
    main()
