"""Measurement of every benchmark config against cuBLAS (``torch.mm/addmm/bmm``).

Protocol: each row is timed with CUDA events around back-to-back launches that
rotate over enough copies of the operands to exceed twice the L2 capacity, so every
launch reads its operands from HBM (the reference's cold / "own copy of the weights
per layer" protocol, benchmarks/common.py:343-356, :380-400).  Both arms run the same
NT layout (benchmarks/common.py:184-198) in the same process.
"""

from __future__ import annotations

import torch

from . import _lib
from .gemm_jit import select_gemm_schedule

L2_BYTES = 126e6
SWEEP_M = (1, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384)
SWEEP_NK = ((4096, 4096), (14336, 4096), (4096, 14336))


def _time(fn, reps: int) -> float:
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    start.record()
    for i in range(reps):
        fn(i)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps


def _copies(nbytes: float, cap: int = 24) -> int:
    return int(max(2, min(cap, -(-2.5 * L2_BYTES // nbytes))))


def measure_gemm(operation: str, dtype: str, batch: int, m: int, n: int, k: int, peaks: dict,
                 cfg: dict | None = None, reps: int | None = None) -> dict:
    dev = "cuda"
    td = torch.bfloat16 if dtype == "bfloat16" else torch.float16
    lead = (batch,) if operation == "bmm" else ()
    nbytes = 2.0 * (batch * (m * k + n * k + m * n))
    copies = _copies(nbytes)
    sets = []
    for _ in range(copies):
        a = torch.randn((*lead, m, k), device=dev, dtype=torch.float32).mul_(k ** -0.5).to(td)
        bt = torch.randn((*lead, n, k), device=dev, dtype=torch.float32).to(td)
        out = torch.empty((*lead, m, n), device=dev, dtype=td)
        bias = torch.randn(n, device=dev).to(td) if operation == "addmm" else None
        sets.append((bias, a, bt, out))
    if cfg is None:
        seed = select_gemm_schedule(operation, dtype, m, n, k, batch)
        cfg = dict(seed.builder_config)
    config = _lib.Config.from_dict(cfg)
    need = _lib.workspace_bytes(config, operation, batch, m, n, k)
    ws = torch.zeros(max(need, 16), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def ours(i):
        bias, a, bt, out = sets[i % copies]
        _lib.gemm(operation, dtype, bias.data_ptr() if bias is not None else 0, a.data_ptr(), bt.data_ptr(),
                  out.data_ptr(), batch, m, n, k, config, ws.data_ptr(), ws.numel(), 0, stream)

    def cublas(i):
        bias, a, bt, out = sets[i % copies]
        if operation == "mm":
            torch.mm(a, bt.t(), out=out)
        elif operation == "addmm":
            torch.addmm(bias, a, bt.t(), out=out)
        else:
            torch.bmm(a, bt.transpose(1, 2), out=out)

    flops = 2.0 * batch * m * n * k
    if reps is None:
        est_ms = max(flops / 1.2e12, nbytes / 5e9) * 1e3 / 1e3 + 0.004
        reps = int(max(10, min(400, 60.0 / est_ms)))
    ms = _time(ours, reps)
    ms_t = _time(cublas, reps)
    row = {
        "op": operation, "dtype": dtype, "batch": batch, "m": m, "n": n, "k": k, "schedule": cfg,
        "operand_copies": copies, "reps": reps,
        "ms": ms, "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6,
        "frac_tensor_peak": flops / ms / 1e9 / peaks["bf16"], "frac_hbm_peak": nbytes / ms / 1e6 / peaks["hbm"],
        "torch_ms": ms_t, "torch_tflops": flops / ms_t / 1e9, "speedup_vs_torch": ms_t / ms,
    }
    del sets
    torch.cuda.empty_cache()
    return row


def run_suite(peaks: dict, sweep: bool = True) -> list[dict]:
    rows = []

    def add(label, *args, **kwargs):
        row = measure_gemm(*args, peaks=peaks, **kwargs)
        row["config"] = label
        rows.append(row)
        print(f"[suite] {label}: {row['ms']*1e3:.1f} us {row['tflops']:.1f} TF/s {row['gbs']:.0f} GB/s | "
              f"torch {row['torch_ms']*1e3:.1f} us | x{row['speedup_vs_torch']:.2f}", flush=True)

    add("C1", "mm", "bfloat16", 1, 4096, 4096, 4096)
    add("C2a-bf16", "addmm", "bfloat16", 1, 8192, 768, 768)
    add("C2a-f16", "addmm", "float16", 1, 8192, 768, 768)
    add("C2b-bf16", "addmm", "bfloat16", 1, 256, 1024, 16384)
    add("C2b-f16", "addmm", "float16", 1, 256, 1024, 16384)
    add("C3a", "bmm", "bfloat16", 64, 2048, 2048, 128)
    add("C3b", "bmm", "bfloat16", 64, 2048, 128, 2048)
    add("mm8192", "mm", "bfloat16", 1, 8192, 8192, 8192)
    if sweep:
        for n, k in SWEEP_NK:
            for m in SWEEP_M:
                add(f"C5 m={m} n={n} k={k}", "mm", "bfloat16", 1, m, n, k)
    return rows
