"""Measurement of every benchmark config against cuBLAS (``torch.mm/addmm/bmm``).

Protocol (the reference's, benchmarks/common.py:522-551, :632-736, adapted): each arm is
captured into a CUDA graph of back-to-back launches after three warm launches; the
launches of a graph rotate over enough copies of the operands to exceed 2.5x the L2
capacity, so every launch reads its operands from HBM (the reference's "own cold copy of
the weights per layer", benchmarks/common.py:380-400); the two arms are replayed
alternately, the starting arm rotating, and the median per-launch time over the rounds
is reported.  Both arms use the same NT layout (benchmarks/common.py:184-198) in the
same process.
"""

from __future__ import annotations

import statistics

import torch

from . import _lib
from .gemm_jit import select_gemm_schedule

L2_BYTES = 126e6
SWEEP_M = (1, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384)
SWEEP_NK = ((4096, 4096), (14336, 4096), (4096, 14336))


def _copies(nbytes: float, cap: int = 24) -> int:
    return int(max(2, min(cap, -(-2.5 * L2_BYTES // nbytes))))


def _capture(fn, launches: int, stream: torch.cuda.Stream) -> torch.cuda.CUDAGraph:
    with torch.cuda.stream(stream):
        for i in range(3):
            fn(i, stream.cuda_stream)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(launches):
                fn(i, stream.cuda_stream)
        graph.replay()
        stream.synchronize()
    return graph


def time_interleaved(fns: dict, launches: int, rounds: int = 9) -> dict:
    """Median per-launch milliseconds of each callable ``fn(i, raw_stream)``."""
    stream = torch.cuda.Stream()
    graphs = {name: _capture(fn, launches, stream) for name, fn in fns.items()}
    names = list(graphs)
    samples = {name: [] for name in names}
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for r in range(rounds):
            order = names[r % len(names):] + names[:r % len(names)]
            for name in order:
                start.record(stream)
                graphs[name].replay()
                stop.record(stream)
                stream.synchronize()
                samples[name].append(start.elapsed_time(stop) / launches)
    return {name: statistics.median(vals) for name, vals in samples.items()}


def measure_gemm(operation: str, dtype: str, batch: int, m: int, n: int, k: int, peaks: dict,
                 cfg: dict | None = None, rounds: int = 9, with_torch: bool = True) -> dict:
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
    source = "explicit"
    if cfg is None:
        seed = select_gemm_schedule(operation, dtype, m, n, k, batch)
        cfg = dict(seed.builder_config)
        source = "table" if seed.source_shape is not None else "default"
    config = _lib.Config.from_dict(cfg)
    need = _lib.workspace_bytes(config, operation, batch, m, n, k)
    ws = torch.zeros(max(need, 16), dtype=torch.uint8, device=dev)

    def ours(i, stream):
        bias, a, bt, out = sets[i % copies]
        _lib.gemm(operation, dtype, bias.data_ptr() if bias is not None else 0, a.data_ptr(), bt.data_ptr(),
                  out.data_ptr(), batch, m, n, k, config, ws.data_ptr(), ws.numel(), 0, stream)

    def cublas(i, stream):
        bias, a, bt, out = sets[i % copies]
        if operation == "mm":
            torch.mm(a, bt.t(), out=out)
        elif operation == "addmm":
            torch.addmm(bias, a, bt.t(), out=out)
        else:
            torch.bmm(a, bt.transpose(1, 2), out=out)

    flops = 2.0 * batch * m * n * k
    est_ms = max(flops / 1.2e15, nbytes / 4e12) * 1e3 + 0.004
    launches = int(max(4, min(40, 2.0 / est_ms)))
    fns = {"ours": ours}
    if with_torch:
        fns["torch"] = cublas
    times = time_interleaved(fns, launches, rounds)
    ms = times["ours"]
    row = {
        "op": operation, "dtype": dtype, "batch": batch, "m": m, "n": n, "k": k,
        "schedule": {key: val for key, val in config.to_dict().items() if val}, "schedule_source": source,
        "operand_copies": copies, "launches_per_graph": launches, "rounds": rounds,
        "ms": ms, "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6,
        "frac_tensor_peak": flops / ms / 1e9 / peaks["bf16"], "frac_hbm_peak": nbytes / ms / 1e6 / peaks["hbm"],
    }
    if with_torch:
        ms_t = times["torch"]
        row.update({"torch_ms": ms_t, "torch_tflops": flops / ms_t / 1e9, "speedup_vs_torch": ms_t / ms})
    del sets
    torch.cuda.empty_cache()
    return row


def measure_swiglu(m: int, n: int, k: int, peaks: dict, cfg: dict | None = None, rounds: int = 7) -> dict:
    dev = "cuda"
    td = torch.bfloat16
    x = torch.randn(m, k, device=dev).to(td)
    wg = (torch.randn(n, k, device=dev) * 0.02).to(td)
    wu = (torch.randn(n, k, device=dev) * 0.02).to(td)
    wcat = torch.cat([wg, wu]).contiguous()
    out = torch.empty(m, n, device=dev, dtype=td)
    config = _lib.Config.from_dict(cfg) if cfg else None

    def ours(i, stream):
        _lib.swiglu("bfloat16", x.data_ptr(), wg.data_ptr(), wu.data_ptr(), out.data_ptr(), m, n, k, config, 0, stream)

    def unfused(i, stream):
        torch.mul(torch.nn.functional.silu(torch.mm(x, wg.t())), torch.mm(x, wu.t()), out=out)

    def concat(i, stream):
        both = torch.mm(x, wcat.t())
        torch.mul(torch.nn.functional.silu(both[:, :n]), both[:, n:], out=out)

    flops = 4.0 * m * n * k
    times = time_interleaved({"ours": ours, "torch_unfused": unfused, "torch_concat": concat}, 4, rounds)
    nbytes = 2.0 * (m * k + 2 * n * k + m * n)
    ms = times["ours"]
    return {
        "op": "swiglu", "dtype": "bfloat16", "m": m, "n": n, "k": k, "ms": ms, "tflops": flops / ms / 1e9,
        "gbs": nbytes / ms / 1e6, "frac_tensor_peak": flops / ms / 1e9 / peaks["bf16"],
        "torch_unfused_ms": times["torch_unfused"], "torch_concat_ms": times["torch_concat"],
        "speedup_vs_torch": min(times["torch_unfused"], times["torch_concat"]) / ms,
    }


def run_suite(peaks: dict, sweep: bool = True) -> list[dict]:
    rows = []

    def add(label, *args, **kwargs):
        row = measure_gemm(*args, peaks=peaks, **kwargs)
        row["config"] = label
        rows.append(row)
        print(f"[suite] {label}: {row['ms']*1e3:.1f} us {row['tflops']:.1f} TF/s {row['gbs']:.0f} GB/s "
              f"{row['schedule']} | torch {row['torch_ms']*1e3:.1f} us | x{row['speedup_vs_torch']:.2f}", flush=True)

    add("C1", "mm", "bfloat16", 1, 4096, 4096, 4096)
    add("C2a-bf16", "addmm", "bfloat16", 1, 8192, 768, 768)
    add("C2a-f16", "addmm", "float16", 1, 8192, 768, 768)
    add("C2b-bf16", "addmm", "bfloat16", 1, 256, 1024, 16384)
    add("C2b-f16", "addmm", "float16", 1, 256, 1024, 16384)
    add("C3a", "bmm", "bfloat16", 64, 2048, 2048, 128)
    add("C3b", "bmm", "bfloat16", 64, 2048, 128, 2048)
    row = measure_swiglu(8192, 14336, 4096, peaks)
    row["config"] = "C4"
    rows.append(row)
    print(f"[suite] C4 swiglu: {row['ms']*1e3:.1f} us {row['tflops']:.1f} TF/s | torch unfused "
          f"{row['torch_unfused_ms']*1e3:.1f} us, concat {row['torch_concat_ms']*1e3:.1f} us | "
          f"x{row['speedup_vs_torch']:.2f}", flush=True)
    add("mm8192", "mm", "bfloat16", 1, 8192, 8192, 8192, rounds=5)
    if sweep:
        for n, k in SWEEP_NK:
            for m in SWEEP_M:
                add(f"C5 m={m} n={n} k={k}", "mm", "bfloat16", 1, m, n, k)
    return rows
