"""Benchmark of the GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--suite]
    python bench.py --case C1 [--launches 6] [--schedule '{"tile_n":256,...}'] [--torch]

Default arm: one JSON line for the headline workload, bf16 ``mm`` with
M = N = K = 4096 (``out = a @ bt.T``), one step = one launch through the C ABI:

* ``value``     TFLOP/s with operands resident in HBM (CUDA events around K launches);
                the K launches rotate over operand sets that together exceed L2;
* ``e2e``       the same metric through ``gemm_op`` with HOST operands: every step
                copies a and bt from pinned host memory, launches, and copies out back;
* ``roofline``  tensor-pipe roofline of the GEMM kernel against the measured cuBLAS
                bf16 burst peak in MEASURED_PEAKS.json (the sustained figure only when the
                timed region itself lasts a second or more; both fractions are printed);
* ``vs_cublas`` cuBLAS (torch.mm) on the same operand sets, timed in the same regime:
                blocks of launches of the two arms alternating, starting arm rotating;
* ``cpu_baseline`` the CPU oracle (PyTorch fp32 mm of the same operands) timed on the
                host cores;
* ``extra``     the fused SwiGLU config, and ``extra.hbm``: weight-streaming shapes
                (M = 8 and 64 on 14336x4096 and 4096x4096 weights) with operands rotating
                past L2, each with its HBM roofline.

The schedule timed is the one ``gemm_op`` runs for the shape
(``select_gemm_schedule(...).builder_config``).

``--case`` launches one benchmark config a few times and exits: the command that is put
under ``ncu`` (configs C1, C2a, C2b, C3a, C3b, C4, or ``mm:M,N,K`` / ``addmm:M,N,K`` /
``bmm:B,M,N,K``; ``--torch`` launches the cuBLAS counterpart instead).

``--impl reference`` times the reference's CPU path for this workload: the reference has
no CPU kernel of its own, its tests define the result as PyTorch's fp32 matmul
(tests/gemm_collection/test_correctness.py:419), which is what the oracle restates.

``--suite`` additionally measures every benchmark config (addmm, split-K, bmm, SwiGLU,
the dynamic-M sweep) against cuBLAS and writes the rows to ``--suite-out`` (default
``results/suite.json``).

With ``--gpus N`` (launched under torchrun, one rank per GPU) every rank runs the same
workload on its own GPU (the 4096^3 GEMM does not shard usefully: replicas, weak
scaling); ``sharded`` then reports the configs that do shard -- bmm by batch and the
N-sharded 32768^3 mm with an NCCL all-gather of out.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "bf16 TFLOP/s, mm M=N=K=4096 (out = a @ bt.T)"
WORKLOAD = "C1 mm bf16 4096x4096x4096"
M = N = K = 4096
FLOPS = 2.0 * M * N * K
ALGO_BYTES = 2.0 * (M * K + N * K + M * N)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from
# an ncu capture (--set full; 103.4 and 104.8 MB in the two launches captured of the current kernel,
# 100.4-102.6 MB in four of earlier versions).
NCU_TRAFFIC_BYTES = 104.1e6


def read_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return dict(bf16=float(data["bf16_tflops"]), bf16_sustained=float(data.get("bf16_tflops_sustained", 0)),
                    hbm=float(data["hbm_gbs"]), source="measured")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clocks, reasons, power = [], [], set(), []
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clocks.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c, p in zip(clocks, power) if p > 300.0] or clocks
        return {
            "sm_mhz": statistics.median(busy) if busy else None,
            "sm_max_mhz": max(max_clocks) if max_clocks else None,
            "power_w_max": max(power) if power else None,
            "samples": len(clocks),
            "reasons": sorted(reasons),
        }


def cuda_time_ms(fn, steps: int, stream=None) -> float:
    """Average milliseconds per call of fn(i), timed with CUDA events on the current stream."""
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(steps):
        fn(i)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def gpu_numa_cpus(device_index: int) -> tuple[int | None, set[int]]:
    """(NUMA node, CPUs of that node) of a GPU, read from sysfs through its PCI address."""
    props = torch.cuda.get_device_properties(device_index)
    bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    node = int(Path(f"/sys/bus/pci/devices/{bdf}/numa_node").read_text().strip())
    if node < 0:
        return None, set()
    cpus: set[int] = set()
    for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return node, cpus


class NumaLocal:
    """While active, this process runs on the CPUs of the GPU's NUMA node, so host buffers pinned
    inside the block get their pages there (first touch).  The previous affinity is restored on
    exit; nothing outside this process is changed."""

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.info: dict = {"node": None, "bound": False}
        self._previous = None

    def __enter__(self):
        try:
            node, cpus = gpu_numa_cpus(self.device_index)
            self._previous = os.sched_getaffinity(0)
            usable = cpus & self._previous
            self.info["node"] = node
            if usable:
                os.sched_setaffinity(0, usable)
                self.info.update(bound=True, cpus=len(usable))
        except (OSError, ValueError, AttributeError) as exc:
            self.info["error"] = f"{type(exc).__name__}: {exc}"
        return self

    def __exit__(self, *exc):
        if self._previous is not None and self.info.get("bound"):
            os.sched_setaffinity(0, self._previous)


def interleaved_blocks(arms: dict, block: int, rounds: int) -> dict:
    """Milliseconds per launch of each arm ``fn(i)``: the arms run in alternating blocks of `block`
    launches, the starting arm rotating from round to round, every block bracketed by CUDA events on
    the current stream -- so both arms see the same clocks, power state and cache contents."""
    names = list(arms)
    total = {name: 0.0 for name in names}
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for r in range(rounds):
        order = names[r % len(names):] + names[:r % len(names)]
        for name in order:
            fn = arms[name]
            start.record()
            for i in range(block):
                fn(i)
            stop.record()
            stop.synchronize()
            total[name] += start.elapsed_time(stop)
    return {name: total[name] / (block * rounds) for name in names}


CASES = {
    "C1": ("mm", 1, 4096, 4096, 4096),
    "C2a": ("addmm", 1, 8192, 768, 768),
    "C2b": ("addmm", 1, 256, 1024, 16384),
    "C3a": ("bmm", 64, 2048, 2048, 128),
    "C3b": ("bmm", 64, 2048, 128, 2048),
    "C4": ("swiglu", 1, 8192, 14336, 4096),
}


def run_case(args) -> None:
    """Launch one config ``--launches`` times and exit (random inputs, nothing checked): the
    command profiled with ncu."""
    from ayla_b200 import _lib
    from ayla_b200.gemm_jit import select_gemm_schedule

    if args.case in CASES:
        op, batch, m, n, k = CASES[args.case]
    else:
        op, dims = args.case.split(":")
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
            if args.torch:
                torch.mul(torch.nn.functional.silu(torch.mm(x, wg.t())), torch.mm(x, wu.t()), out=out)
            else:
                _lib.swiglu(args.dtype, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), out.data_ptr(), m, n, k, cfg,
                            0, stream)
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
            if args.torch:
                if op == "mm":
                    torch.mm(a, bt.t(), out=out)
                elif op == "addmm":
                    torch.addmm(bias, a, bt.t(), out=out)
                else:
                    torch.bmm(a, bt.transpose(1, 2), out=out)
            else:
                _lib.gemm(op, args.dtype, bias.data_ptr() if op == "addmm" else 0, a.data_ptr(), bt.data_ptr(),
                          out.data_ptr(), batch, m, n, k, cfg, ws.data_ptr(), ws.numel(), 0, stream)
    torch.cuda.synchronize()
    arm = "torch" if args.torch else "ayla_b200"
    print(f"{args.case}: {args.launches} {arm} launches of {op} {batch}x{m}x{n}x{k} done")


STAMPS = {"entry": 0, "set-up done": 1, "preceding launch complete": 14, "first TMA issued": 12,
          "first operands landed": 2, "last MMA committed": 3, "epilogue saw the accumulator": 13,
          "first chunk in registers": 16, "first chunk staged": 22, "second chunk staged": 23,
          "staging published (proxy fence)": 24, "first bulk store issued": 25,
          "split-k: cluster met": 6, "split-k: own part sent": 15, "split-k: peers' parts in": 7,
          "split-k: own partial in registers": 26, "split-k: first chunk summed": 27, 
          "first 64-column group done": 18, "second 64-column group done": 19,
          "last chunk handed to the stores": 17, "epilogue done": 4, "exit": 5}
INTERVALS = (("entry", "set-up done"), ("preceding launch complete", "first TMA issued"),
             ("preceding launch complete", "first operands landed"),
             ("first operands landed", "last MMA committed"), ("last MMA committed", "epilogue saw the accumulator"),
             ("last MMA committed", "first chunk in registers"),
             ("last MMA committed", "first chunk staged"), ("last MMA committed", "second chunk staged"),
             ("last MMA committed", "staging published (proxy fence)"),
             ("last MMA committed", "first bulk store issued"),
             ("last MMA committed", "split-k: cluster met"),
             ("last MMA committed", "split-k: own part sent"), ("last MMA committed", "split-k: peers' parts in"),
             ("last MMA committed", "split-k: own partial in registers"),
             ("last MMA committed", "split-k: first chunk summed"),
             ("last MMA committed", "first 64-column group done"),
             ("last MMA committed", "second 64-column group done"),
             ("last MMA committed", "last chunk handed to the stores"),
             ("last MMA committed", "epilogue done"), ("last MMA committed", "exit"), ("entry", "exit"))


def run_timeline(args) -> None:
    """Where one launch spends its time: the per-CTA stamps of the trace build
    (``python -m ayla_b200.build --trace``), read after a CUDA graph of ``--launches`` back-to-back
    launches on operand sets rotating past L2 (the suite's regime).  Consecutive launches stamp into
    two alternating buffers, so the last launch and the one before it are both kept.  Intervals
    inside a CTA come from the SM's cycle counter, comparisons across CTAs from ``globaltimer``.
    Only schedules without workspace slabs leave stamps (cluster k-splits do)."""
    from ayla_b200 import build as _build

    if "AYLA_B200_LIB" not in os.environ:
        if not _build.TRACE_LIB_PATH.exists():
            raise SystemExit("--timeline needs the trace build: python -m ayla_b200.build --trace")
        os.environ["AYLA_B200_LIB"] = str(_build.TRACE_LIB_PATH)
    from ayla_b200 import _lib
    from ayla_b200.gemm_jit import select_gemm_schedule
    from ayla_b200.suite import _copies

    if args.case in CASES:
        op, batch, m, n, k = CASES[args.case]
    else:
        op, dims = args.case.split(":")
        values = [int(v) for v in dims.split(",")]
        batch, (m, n, k) = (values[0], values[1:]) if op == "bmm" else (1, values)
    if op == "swiglu":
        raise SystemExit("--timeline covers mm, addmm and bmm")
    dev = "cuda:0"
    _lib.init(0)
    td = torch.bfloat16 if args.dtype == "bfloat16" else torch.float16
    schedule = json.loads(args.schedule) if args.schedule else dict(
        select_gemm_schedule(op, args.dtype, m, n, k, batch).builder_config)
    cfg = _lib.Config.from_dict(schedule)
    if _lib.workspace_bytes(cfg, op, batch, m, n, k) > 0:
        raise SystemExit("this schedule reduces through workspace slabs; the stamps need the workspace")
    lead = (batch,) if op == "bmm" else ()
    sets = []
    for _ in range(_copies(2.0 * batch * (m * k + n * k + m * n))):
        sets.append((torch.randn((*lead, m, k), device=dev).to(td),
                     (torch.randn((*lead, n, k), device=dev) * k ** -0.5).to(td),
                     torch.empty((*lead, m, n), device=dev, dtype=td)))
    bias = torch.randn(n, device=dev).to(td)
    sm_count = torch.cuda.get_device_properties(0).multi_processor_count
    words = 4096 + sm_count * 64
    buffers = torch.zeros(2, words, dtype=torch.int64, device=dev)
    stream = torch.cuda.Stream()

    def launch(i: int) -> None:
        a, bt, out = sets[i % len(sets)]
        _lib.gemm(op, args.dtype, bias.data_ptr() if op == "addmm" else 0, a.data_ptr(), bt.data_ptr(),
                  out.data_ptr(), batch, m, n, k, cfg, buffers[i % 2].data_ptr(), words * 8, 0, stream.cuda_stream)

    with torch.cuda.stream(stream):
        for i in range(3):
            launch(i)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(args.launches):
                launch(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(5):
            buffers.zero_()
            e0.record(stream)
            graph.replay()
            e1.record(stream)
            stream.synchronize()
    per_launch_us = e0.elapsed_time(e1) * 1e3 / args.launches

    def stamps_of(index: int) -> torch.Tensor:
        rows = buffers[index % 2][4096:].view(sm_count, 64).cpu()
        return rows[rows[:, STAMPS["exit"]] > 0].double()

    last, before = stamps_of(args.launches - 1), stamps_of(args.launches - 2)
    if last.numel() == 0:
        raise SystemExit("no stamps: is AYLA_B200_LIB a trace build?")
    entry_ns, exit_ns = last[:, 32], last[:, 33]
    cycles = last[:, STAMPS["exit"]] - last[:, STAMPS["entry"]]
    mhz = float((cycles / (exit_ns - entry_ns)).median() * 1e3)

    def on_shared_clock(rows: torch.Tensor, name: str) -> torch.Tensor:
        """ns on the time base all SMs share: the CTA's entry time plus its cycles since entry."""
        return rows[:, 32] + (rows[:, STAMPS[name]] - rows[:, STAMPS["entry"]]) * 1e3 / mhz

    print(f"{args.case}: {op} {batch}x{m}x{n}x{k} {args.dtype}, schedule {json.dumps(schedule)}")
    print(f"{per_launch_us:.2f} us per launch over {args.launches} back-to-back launches in a graph (trace build); "
          f"{last.shape[0]} CTAs; SM clock {mhz:.0f} MHz from the stamps")
    print("per-CTA intervals of the last launch, us at that clock from the SM cycle counter (min / median / max over CTAs):")
    for first, second in INTERVALS:
        a, b = last[:, STAMPS[first]], last[:, STAMPS[second]]
        ok = (a > 0) & (b > 0)
        if ok.any():
            d = (b[ok] - a[ok]) / mhz
            print(f"  {first:28s} -> {second:32s} {d.min():7.2f} / {d.median():7.2f} / {d.max():7.2f}")
    print("across CTAs, us (globaltimer at entry and exit, steps of 0.26 us on this GPU, cycles in between):")
    print(f"  first entry -> last exit: {(exit_ns.max() - entry_ns.min()) / 1e3:.2f}; entries spread over "
          f"{(entry_ns.max() - entry_ns.min()) / 1e3:.2f}, exits over {(exit_ns.max() - exit_ns.min()) / 1e3:.2f}")
    if before.numel():
        ready = on_shared_clock(last, "preceding launch complete")[last[:, STAMPS["preceding launch complete"]] > 0]
        prev_exit = before[:, 33].max()
        print(f"  last exit of the launch before -> this launch's producers released: "
              f"{(ready.min() - prev_exit) / 1e3:.2f} (first) / {(ready.median() - prev_exit) / 1e3:.2f} (median); "
              f"last exit to last exit {(exit_ns.max() - prev_exit) / 1e3:.2f}")


def _sm_clock_mhz() -> str:
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(0)
        return str(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
    except Exception:
        return "unknown"


def hbm_rows(peaks: dict) -> list[dict]:
    """Weight-streaming shapes (HBM-bound: the weight is read once per launch): graph replay with
    operand sets rotating through more than 2.5x L2, cuBLAS interleaved (``ayla_b200.suite``)."""
    from ayla_b200.suite import measure_gemm

    rows = []
    for m, n, k in ((8, 14336, 4096), (64, 14336, 4096), (8, 4096, 4096), (64, 4096, 4096)):
        row = measure_gemm("mm", "bfloat16", 1, m, n, k, peaks, rounds=7)
        nbytes = 2.0 * (m * k + n * k + m * n)
        rows.append({
            "workload": f"mm bf16 M={m} N={n} K={k}", "us": row["ms"] * 1e3, "torch_us": row["torch_ms"] * 1e3,
            "vs_cublas": row["speedup_vs_torch"], "schedule": row["schedule"],
            "roofline": {"bound": "hbm", "achieved": row["gbs"], "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": row["gbs"] / peaks["hbm"], "algorithmic_bytes": nbytes,
                         "peak_source": f"{peaks['source']} HBM copy bandwidth"},
        })
    return rows


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # Keep NCCL's kernels small enough to run on the SMs the sharded GEMM leaves free.
        os.environ.setdefault("NCCL_MAX_CTAS", "16")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, world, local


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def max_over_ranks_list(values: list[float], world: int) -> list[float]:
    """Element-wise maximum over ranks, so that every rank makes the same choice from the list."""
    if world == 1:
        return values
    import torch.distributed as dist

    t = torch.tensor(values, dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def make_c1_sets(count: int, device) -> list:
    """`count` operand sets of the C1 workload; set 0 holds the seeded benchmark inputs."""
    from oracle import gemm_oracle as O

    _, (a0, bt0) = O.make_inputs("C1", "bfloat16")
    sets = []
    for i in range(count):
        if i == 0:
            a, bt = a0.to(device), bt0.to(device)
        else:
            g = torch.Generator(device="cpu").manual_seed(1000 + i)
            a = torch.randn(M, K, generator=g).bfloat16().to(device)
            bt = torch.randn(N, K, generator=g).bfloat16().to(device)
        sets.append((a, bt, torch.empty(M, N, dtype=torch.bfloat16, device=device)))
    return (a0, bt0), sets


def cpu_baseline(a0, bt0, reps: int = 3) -> dict:
    from oracle import gemm_oracle as O

    O.mm_ref32(a0[:256], bt0)  # warm the thread pool
    best = float("inf")
    for _ in range(reps):
        t = time.perf_counter()
        O.mm_ref32(a0, bt0)
        best = min(best, time.perf_counter() - t)
    return {
        "value": FLOPS / best / 1e12,
        "unit": "TFLOP/s",
        "cores": torch.get_num_threads(),
        "kind": "port",
        "sample": f"full workload (fp32 torch.mm of the same 4096^3 operands), best of {reps}, {best:.3f} s each",
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1 for its workers; this arm runs on rank 0 alone and may
    # use every host core the process is allowed.
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        torch.set_num_threads(os.cpu_count() or 1)
    from oracle import gemm_oracle as O

    _, (a0, bt0) = O.make_inputs("C1", "bfloat16")
    for _ in range(max(1, min(args.warmup, 3))):
        O.mm_ref32(a0, bt0)
    steps = max(1, min(args.steps, 20))
    t = time.perf_counter()
    for _ in range(steps):
        O.mm_ref32(a0, bt0)
    per_step = (time.perf_counter() - t) / steps
    value = FLOPS / per_step / 1e12
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "reference CPU path = PyTorch fp32 mm of the up-cast operands "
                   "(the reference has no CPU kernel; its tests use this as the result definition)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{steps} x full 4096^3 fp32 mm on CPU"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def swiglu_extra(peaks: dict) -> dict:
    """Fused SwiGLU x[8192,4096], W[14336,4096] (operands 537 MB > L2) against the two torch
    formulations (two mm + eager epilogue; one mm on the concatenated weight + epilogue)."""
    from ayla_b200.suite import measure_swiglu

    row = measure_swiglu(8192, 14336, 4096, peaks)
    row["workload"] = "C4 fused SwiGLU bf16 x[8192,4096] W_gate,W_up[14336,4096]"
    return row


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=2000)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--suite", action="store_true")
    parser.add_argument("--suite-out", default="results/suite.json")
    parser.add_argument("--no-extra", action="store_true")
    parser.add_argument("--case", default=None, help="launch this config --launches times and exit (for ncu)")
    parser.add_argument("--launches", type=int, default=6)
    parser.add_argument("--schedule", default=None, help="JSON schedule for --case (default: the table's)")
    parser.add_argument("--dtype", default="bfloat16")
    parser.add_argument("--torch", action="store_true", help="--case launches the cuBLAS counterpart instead")
    parser.add_argument("--timeline", action="store_true",
                        help="--case prints the per-CTA stage times of a launch (needs the trace build)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path "
                         "(use --impl reference for the CPU baseline)")
    if args.case:
        run_timeline(args) if args.timeline else run_case(args)
        return

    # Only the JSON line may reach stdout: libraries that write there from native code (NCCL prints its
    # version at communicator creation) are sent to stderr until the line is printed.
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(line: dict) -> None:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps(line), flush=True)

    rank, world, local = dist_setup(args.gpus)
    from ayla_b200 import _lib, gemm_op

    device = torch.device("cuda", local if world > 1 else 0)
    _lib.init(device.index)
    peaks = read_peaks()
    # The weight-streaming rows first, before the compute-bound loops heat the GPU into its power
    # cap: they model decode steps, which draw a few hundred watts and run at full clocks.  (These
    # kernels do a fixed number of SM cycles of work per 64-deep block of K beside the HBM traffic,
    # so right after seconds of dense GEMMs, at 1.35 GHz, they measure up to a third slower.)
    hbm = None
    if world == 1 and not args.no_extra:
        hbm_sampler = ClockSampler(device.index)
        hbm_sampler.start()
        hbm = {"rows": hbm_rows(peaks), "clocks": hbm_sampler.stop(),
               "order": "measured first, before the compute-bound loops of this run"}
    sets_needed = 4  # 4 x 100.7 MB of operands+output > 126 MB L2
    (a0, bt0), sets = make_c1_sets(sets_needed, device)
    cfg = None  # the library's schedule for this shape (same one gemm_op selects)
    from ayla_b200.gemm_jit import select_gemm_schedule

    seed = select_gemm_schedule("mm", "bfloat16", M, N, K)
    cfg = _lib.Config.from_dict(seed.builder_config)
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=device)

    schedule_choice = "select_gemm_schedule('mm', 'bfloat16', 4096, 4096, 4096).builder_config, the schedule gemm_op runs"

    def step(i):
        a, bt, out = sets[i % len(sets)]
        _lib.gemm("mm", "bfloat16", 0, a.data_ptr(), bt.data_ptr(), out.data_ptr(), 1, M, N, K, cfg, 0, 0,
                  status.data_ptr(), stream)

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()

    # parity of the timed configuration before timing it
    from oracle import gemm_oracle as O

    parity = None
    if rank == 0:
        parity = O.compare(sets[0][2], O.mm_ref32(a0, bt0))
        if not parity.ok:
            raise SystemExit(f"parity failed before timing: {parity}")

    sampler = ClockSampler(device.index)
    barrier(world)
    if rank == 0:
        sampler.start()
        time.sleep(0.1)
    # nvidia-smi needs a moment before its first sample: keep the GPU in the loop's own regime meanwhile
    cuda_time_ms(step, 3000)
    barrier(world)
    ms = cuda_time_ms(step, args.steps)
    barrier(world)
    ms = max_over_ranks(ms, world)
    clocks = sampler.stop() if rank == 0 else None
    if int(status.item()) != 0:
        raise SystemExit(f"device status {int(status.item()):#x}: a bounded wait gave up")

    # ---- cuBLAS on the same operand sets, in the same regime: straight after the timed loop (the
    # GPU is as warm and as power-capped as it was there), blocks of launches of the two arms
    # alternating, the starting arm rotating.
    vs_cublas = None
    if world == 1 and not args.no_extra:
        def cublas(i):
            a, bt, out = sets[i % len(sets)]
            torch.mm(a, bt.t(), out=out)

        for i in range(3):
            cublas(i)
        block = max(50, min(250, args.steps // 4))
        per_arm = interleaved_blocks({"ours": step, "cublas": cublas}, block, rounds=6)
        vs_cublas = {"ratio": per_arm["cublas"] / per_arm["ours"], "ours_ms": per_arm["ours"],
                     "cublas_ms": per_arm["cublas"], "ours_tflops": FLOPS / per_arm["ours"] / 1e9,
                     "cublas_tflops": FLOPS / per_arm["cublas"] / 1e9,
                     "protocol": f"6 rounds of alternating blocks of {block} launches per arm, starting arm "
                                 "rotating, CUDA events per block, same operand sets, run directly after the timed loop"}

    # ---- end to end through the public op with host operands: every step copies its a and bt in
    # from pinned host memory and its result back out.  The three legs run on three streams over
    # two device buffer sets, so the copy-in of step i+1 and the copy-out of step i-1 overlap the
    # GEMM of step i (PCIe is full duplex); events keep each buffer's copy-in -> GEMM -> copy-out order.
    op = gemm_op("mm", "bfloat16")
    # The pinned buffers are allocated while this process runs on the CPUs of the GPU's own NUMA
    # node, so that with one process per GPU every rank copies from and to memory next to its GPU.
    with NumaLocal(device.index) as numa:
        host_a = a0.pin_memory()
        host_bt = bt0.pin_memory()
        host_outs = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    lanes = [sets[0], sets[1]]
    s_in, s_mm, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_mm = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        lane = i % 2
        dev_a, dev_bt, dev_out = lanes[lane]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_mm[lane])  # the GEMM that last read this lane's operands is done
            dev_a.copy_(host_a, non_blocking=True)
            dev_bt.copy_(host_bt, non_blocking=True)
            ev_in[lane].record(s_in)
        with torch.cuda.stream(s_mm):
            s_mm.wait_event(ev_in[lane])
            s_mm.wait_event(ev_out[lane])  # this lane's previous result has left the device
            op(dev_a, dev_bt, dev_out)
            ev_mm[lane].record(s_mm)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_mm[lane])
            host_outs[lane].copy_(dev_out, non_blocking=True)
            ev_out[lane].record(s_out)

    def e2e_run(steps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(steps):
            e2e_step(i)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps * 1e3

    e2e_run(4)
    e2e_steps = max(4, min(args.steps, 40))
    barrier(world)
    e2e_ms = max_over_ranks(e2e_run(e2e_steps), world)
    barrier(world)
    # The copy legs alone, all ranks at once (they share the host's PCIe root and memory): what the
    # end-to-end step is bounded by when it is slower than one GPU alone.
    dev_a, dev_bt, dev_out = lanes[0]

    def h2d(i):
        dev_a.copy_(host_a, non_blocking=True)
        dev_bt.copy_(host_bt, non_blocking=True)

    def d2h(i):
        host_outs[0].copy_(dev_out, non_blocking=True)

    barrier(world)
    h2d_ms = max_over_ranks(cuda_time_ms(h2d, 10), world)
    barrier(world)
    d2h_ms = max_over_ranks(cuda_time_ms(d2h, 10), world)
    barrier(world)
    if rank == 0 and not torch.equal(host_outs[0], sets[0][2].cpu()):
        raise SystemExit("end-to-end result differs from the device-resident result")

    if rank != 0:
        if world > 1:
            import torch.distributed as dist

            sharded_results(args, rank, world, device)
            dist.destroy_process_group()
        return

    value = world * FLOPS / ms / 1e9
    achieved = FLOPS / ms / 1e9
    # Denominator: the burst cuBLAS figure, unless the timed region itself lasts a second or more
    # (then the seconds-long sustained figure is the matching one).  Both fractions are printed.
    long_region = ms * args.steps >= 1000.0 and peaks["bf16_sustained"] > 0
    peak = peaks["bf16_sustained"] if long_region else peaks["bf16"]
    peak_kind = "sustained (timed region >= 1 s)" if long_region else "burst (timed region < 1 s)"
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "schedule": cfg.to_dict(), "schedule_choice": schedule_choice,
                   "untimed_launches_before_the_timed_region": "warmup + 3000 while the clock sampler starts",
                   "l2": f"launches rotate over {len(sets)} operand sets, {len(sets) * ALGO_BYTES / 1e6:.0f} MB > 126 MB L2",
                   "parallelism": "replicas" if world > 1 else "1 GPU",
                   "inputs": "a, bt ~ N(0,1) from seed 0 (set 0); fp32 accumulate, bf16 out"},
        "clocks": clocks,
        "e2e": {"value": world * FLOPS / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(2 * (M * K + N * K)), "d2h_bytes_per_step": int(2 * M * N),
                "h2d_gbs_per_gpu_alone_leg": 2.0 * (M * K + N * K) / h2d_ms / 1e6,
                "d2h_gbs_per_gpu_alone_leg": 2.0 * M * N / d2h_ms / 1e6,
                "copy_bound_ms_per_step": max(h2d_ms, d2h_ms), "host_buffers_numa": numa.info,
                "api": "gemm_op('mm','bfloat16')(a, bt, out); every step copies a and bt in from pinned host memory and out back, three streams, two buffer sets; wall clock around the loop with a device synchronise on both sides"},
        "gpu_launches": args.steps,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES,
                     "peak_source": f"{peaks['source']} cuBLAS bf16 {peak_kind}", "algorithmic_bytes": ALGO_BYTES,
                     "frac_of_burst_peak": achieved / peaks["bf16"],
                     "frac_of_sustained_peak": (achieved / peaks["bf16_sustained"]) if peaks["bf16_sustained"] else None,
                     "frac_of_nominal_2250": achieved / 2250.0},
        "parity": {"fro_rel": parity.fro_rel, "max_over_rms": parity.max_over_rms,
                   "over_bound": parity.over_bound, "over_bound_one_ulp": parity.over_bound_one_ulp},
    }
    if world == 1:
        line["cpu_baseline"] = cpu_baseline(a0, bt0)
        if not args.no_extra:
            line["vs_cublas"] = vs_cublas
            line["extra"] = {"swiglu": swiglu_extra(peaks), "hbm": hbm}
    else:
        line["sharded"] = sharded_results(args, rank, world, device)
        import torch.distributed as dist

        dist.destroy_process_group()
    if args.suite and world == 1:
        from ayla_b200.suite import run_suite

        rows = run_suite(peaks)
        suite_out = Path(args.suite_out)
        suite_out.parent.mkdir(parents=True, exist_ok=True)
        suite_out.write_text(json.dumps(rows, indent=1))
    emit(line)


def sharded_results(args, rank: int, world: int, device) -> dict:
    """The configs that shard: bmm by batch (no collective) and N-sharded mm with an NCCL
    all-gather of out.  Every rank takes part; rank 0 returns the numbers."""
    from ayla_b200.sharded import bench_sharded

    return bench_sharded(rank, world, device, steps=max(3, min(args.steps, 10)))


if __name__ == "__main__":
    main()
