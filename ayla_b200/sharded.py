"""Multi-GPU forms of the two GEMMs that shard, one process per GPU.

* ``bmm`` shards by batch: rank r owns a contiguous slice of the batch dimension of
  a, bt and out and runs the single-GPU kernel on it.  No data-path collective.
* a very large ``mm`` shards by N: rank r holds the row block ``bt[r*N/g:(r+1)*N/g]``
  (= a column block of out) and all of a, computes its column block M-panel by
  M-panel, and an NCCL all-gather of each finished panel overlaps the GEMM of the
  next one.  A column block of a row-major matrix is not contiguous, so a panel is
  gathered as ``[g][panel_m][N/g]`` and then copied into place.

The reference is single-GPU (it has no distributed code); these follow the
partitioning the benchmark configs ask for.  The partition arithmetic is pure
Python so it can be tested on CPU ranks.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


def partition(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block ``(start, count)`` of ``total`` units owned by ``rank``;
    the first ``total % world`` ranks take one extra unit."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def column_block(n: int, world: int, rank: int) -> tuple[int, int]:
    """Column block of an N-sharded mm.  N must split evenly into blocks whose width is
    a multiple of 8 (16-byte rows for TMA) so every rank gathers the same amount."""
    if n % world or (n // world) % 8:
        raise ValueError(f"N={n} does not split into {world} equal column blocks that are multiples of 8")
    return rank * (n // world), n // world


@dataclass(frozen=True)
class Panel:
    row0: int
    rows: int


def m_panels(m: int, panel_rows: int) -> list[Panel]:
    """Row panels of the N-sharded mm; the last one may be short."""
    if panel_rows <= 0:
        raise ValueError("panel_rows must be positive")
    return [Panel(r, min(panel_rows, m - r)) for r in range(0, m, panel_rows)]


def fit_panel_rows(m: int, width: int, gemm_sms: int, tile_rows: int = 256, tile_cols: int = 256,
                   min_fill: float = 0.95, max_panels: int = 24) -> int:
    """Rows per M-panel such that a panel's output tiles fill a whole number of waves of the SMs the
    GEMM may use (a 256-row tile occupies a CTA pair): the smallest such height that leaves at most
    ``max_panels`` panels.  A panel of 2048 rows by 4096 columns is 128 tiles, 2.2 waves of 58 pairs
    run as 3; 1792 rows are 112 tiles, 1.93 waves run as 2."""
    pairs = max(1, gemm_sms // 2)
    n_tiles = -(-width // tile_cols)
    fallback, fallback_fill = max(tile_rows, -(-m // 16)), 0.0
    for waves in range(1, 257):
        row_tiles = (waves * pairs) // n_tiles
        if row_tiles == 0:
            continue
        rows = row_tiles * tile_rows
        if -(-m // rows) > max_panels:
            continue
        fill = row_tiles * n_tiles / (waves * pairs)
        if fill >= min_fill:
            return min(rows, -(-m // tile_rows) * tile_rows)
        if fill > fallback_fill:
            fallback, fallback_fill = rows, fill
        if rows >= m:
            break
    return fallback


def place_gathered_panel(out: torch.Tensor, gathered: torch.Tensor, panel: Panel) -> None:
    """``gathered`` is ``[g][panel.rows][N/g]`` (rank-major, as all-gather delivers it);
    write it to rows ``panel.row0 ..`` of the row-major ``out[M][N]``."""
    g, rows, width = gathered.shape
    view = out[panel.row0:panel.row0 + rows].view(rows, g, width)
    view.copy_(gathered.permute(1, 0, 2))


def place_gathered_panel_dma(out: torch.Tensor, gathered: torch.Tensor, panel: Panel, stream: int) -> None:
    """Same placement as ``place_gathered_panel`` done by the copy engines: one strided 2-D copy
    per source rank, so no SM is taken from the GEMM that runs meanwhile."""
    from . import _lib

    g, rows, width = gathered.shape
    elt = out.element_size()
    n = out.shape[1]
    base = out.data_ptr() + panel.row0 * n * elt
    for j in range(g):
        _lib.copy_2d(base + j * width * elt, n * elt, gathered[j].data_ptr(), width * elt, width * elt, rows,
                     stream)


def bmm_sharded(a: torch.Tensor, bt: torch.Tensor, out: torch.Tensor, op) -> None:
    """Run ``op(a, bt, out)`` (a ``gemm_op('bmm', ...)``) on this rank's batch slice.
    The three tensors are this rank's local slices already."""
    op(a, bt, out)


@dataclass(frozen=True)
class Step:
    """One operation of the overlapped N-sharded mm: ``kind`` is ``"gemm"`` (this rank's column
    block of M-panel ``panel`` into local buffer ``buf``), ``"gather"`` (all-gather of that buffer
    into gather buffer ``buf``), ``"place"`` (the gathered panel into its rows of ``out``) or
    ``"push"`` (peer-to-peer copies of the local buffer into every rank's ``out``).  A step runs
    on ``stream`` after the steps before it on that stream and after the steps named in ``after``
    (indices into the plan)."""

    kind: str
    panel: int
    buf: int
    stream: str
    after: tuple[int, ...] = ()


def overlap_plan(n_panels: int, exchange: str = "nccl") -> list[Step]:
    """The order of work of ``NShardedMM`` as data: three in-order streams -- ``"main"`` (GEMMs),
    ``"comm"`` (all-gathers, or the pushes of the DMA exchange) and ``"place"`` (placement of
    gathered panels) -- with the cross-stream dependencies that double buffering needs:

    * the all-gather of panel i follows its GEMM;
    * the GEMM of panel i reuses local buffer i % 2, so it follows the all-gather (or push) of
      panel i - 2, which read that buffer;
    * the all-gather of panel i reuses gather buffer i % 2, so it follows the placement of
      panel i - 2;
    * the placement of panel i follows its all-gather.

    Anything this list does not order may run in any order or at the same time; the CPU test
    executes it in random orders that respect it and nothing else."""
    if exchange not in ("nccl", "dma"):
        raise ValueError(f"unknown exchange {exchange!r}")
    plan: list[Step] = []
    gemm_at: dict[int, int] = {}
    gather_at: dict[int, int] = {}
    place_at: dict[int, int] = {}
    for i in range(n_panels):
        buf = i % 2
        waits = (gather_at[i - 2],) if i >= 2 else ()
        gemm_at[i] = len(plan)
        plan.append(Step("gemm", i, buf, "main", waits))
        if exchange == "nccl":
            waits = (gemm_at[i],) + ((place_at[i - 2],) if i >= 2 else ())
            gather_at[i] = len(plan)
            plan.append(Step("gather", i, buf, "comm", waits))
            place_at[i] = len(plan)
            plan.append(Step("place", i, buf, "place", (gather_at[i],)))
        else:
            gather_at[i] = len(plan)
            plan.append(Step("push", i, buf, "comm", (gemm_at[i],)))
    return plan


def run_plan_in_order(plan: list[Step], execute, pick=None) -> list[int]:
    """Run ``execute(step)`` for every step in an order that respects the plan (stream order and
    ``after``) and nothing else: ``pick(ready_indices)`` chooses among the steps that may run next
    (default: the first).  Returns the order used.  This is how the CPU ranks run the plan."""
    heads = {}
    by_stream: dict[str, list[int]] = {}
    for index, step in enumerate(plan):
        by_stream.setdefault(step.stream, []).append(index)
    for stream in by_stream:
        heads[stream] = 0
    done: set[int] = set()
    order: list[int] = []
    while len(done) < len(plan):
        ready = [queue[heads[stream]] for stream, queue in by_stream.items()
                 if heads[stream] < len(queue) and all(dep in done for dep in plan[queue[heads[stream]]].after)]
        if not ready:
            raise RuntimeError("the plan deadlocks: no step is ready")
        index = pick(ready) if pick is not None else ready[0]
        execute(plan[index])
        done.add(index)
        heads[plan[index].stream] += 1
        order.append(index)
    return order


class NShardedMM:
    """``out[M, N] = a[M, K] @ bt[N, K]^T`` with bt sharded by rows across the group.

    Every rank ends up with the full ``out``.  The M extent is cut into panels; ``overlap_plan``
    gives the order of work.  Two ways to exchange the column blocks:

    * ``exchange="nccl"`` (the default): every finished M-panel is all-gathered with NCCL on a
      second stream as ``[g][rows][N/g]`` and put in place on a third stream by strided DMA
      copies while the GEMM of the next panel runs; ``reserve_sms`` SMs are left free of GEMM
      CTAs so NCCL's kernels can run beside it (pass a group created with a matching
      ``max_ctas``, see ``nccl_group``).  With ``layout="blocked"`` the gathered panels are the
      result (``runner.blocked``, shaped ``[g][M][N/g]``: rank j's column block of ``out`` is
      ``blocked[j]``) and nothing is un-permuted.
    * ``exchange="dma"``: ``out`` lives in symmetric memory and every rank pushes its finished
      panel block straight into every peer's ``out`` with strided peer-to-peer copies on the
      copy engines (plain stores over NVLink, no SMs, no staging, nothing to un-permute); one
      barrier at the end.  Use ``runner.out`` as the output tensor.  ``out`` is the same memory
      on every call: a rank may still be reading the previous result when a peer's next call
      pushes into it, so callers that reuse the runner put their own barrier between the last
      read of ``out`` and the next call.
    """

    def __init__(self, m: int, n: int, k: int, dtype: str, device: torch.device, group=None,
                 panel_rows: int | str | None = None, reserve_sms: int = 16, exchange: str = "nccl",
                 layout: str = "row_major"):
        from . import _lib
        from .gemm_jit import _TORCH_DTYPES, select_gemm_schedule

        if exchange not in ("nccl", "dma"):
            raise ValueError(f"unknown exchange {exchange!r}")
        if layout not in ("row_major", "blocked") or (layout == "blocked" and exchange != "nccl"):
            raise ValueError(f"unknown or unsupported layout {layout!r} for the {exchange} exchange")
        self.exchange, self.layout = exchange, layout
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.m, self.n, self.k, self.dtype = m, n, k, dtype
        self.col0, self.width = column_block(n, self.world, self.rank)
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        if panel_rows is None and exchange == "nccl":
            # Sixteen panels: only one sixteenth of the exchange is left uncovered by compute, and a
            # panel is still several waves of tiles.  (The all-gather, not the GEMM, bounds this path
            # at 8 GPUs: panels fitted to whole waves made the GEMM leg shorter and the whole longer,
            # 9.09 against 8.67 ms for 32768^3, because there were 19 gathers instead of 16.)
            panel_rows = max(1024, -(-m // 16))
        elif panel_rows is None or panel_rows == "fit":
            # Panels whose tiles fill whole waves of the SMs the GEMM keeps.
            reserved = reserve_sms if (exchange == "nccl" and self.world > 1) else 0
            panel_rows = fit_panel_rows(m, self.width, sms - reserved)
        self.panels = m_panels(m, panel_rows)
        self.plan = overlap_plan(len(self.panels), exchange)
        self.device = device
        _lib.init(device.index)
        self._lib = _lib
        torch_dtype = _TORCH_DTYPES[dtype]
        self.torch_dtype = torch_dtype
        rows = self.panels[0].rows
        # One schedule per distinct panel height (the last panel may be short); the workspace is
        # sized for the largest need.
        self.cfgs: dict[int, object] = {}
        need = 16
        for height in sorted({p.rows for p in self.panels}):
            seed = select_gemm_schedule("mm", dtype, height, self.width, k)
            if seed is None:
                raise ValueError(f"no schedule for panel {height}x{self.width}x{k}")
            cfg = dict(seed.builder_config)
            if exchange == "nccl" and self.world > 1 and reserve_sms > 0:
                cfg["grid_ctas"] = (sms - reserve_sms) & ~1
            self.cfgs[height] = _lib.Config.from_dict(cfg)
            need = max(need, _lib.workspace_bytes(self.cfgs[height], "mm", 1, height, self.width, k))
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=device)
        # double-buffered local panel (and gather target for the NCCL exchange)
        self.local = [torch.empty(rows, self.width, dtype=torch_dtype, device=device) for _ in range(2)]
        self.out = None
        self.blocked = None
        self.peer_out: list[torch.Tensor] = []
        if exchange == "nccl":
            if layout == "blocked":
                self.blocked = torch.empty(self.world, m, self.width, dtype=torch_dtype, device=device)
            else:
                self.gathered = [torch.empty(self.world, rows, self.width, dtype=torch_dtype, device=device)
                                 for _ in range(2)]
        else:
            import torch.distributed._symmetric_memory as symm_mem

            self.out = symm_mem.empty((m, n), dtype=torch_dtype, device=device)
            self._handle = symm_mem.rendezvous(self.out, self.group)
            self.peer_out = [self._handle.get_buffer(r, (m, n), torch_dtype) for r in range(self.world)]
        self.streams = {"comm": torch.cuda.Stream(device=device), "place": torch.cuda.Stream(device=device)}
        self.status = _lib.StatusWord()
        self.timings: dict[str, float] | None = None

    def __call__(self, a: torch.Tensor, bt_shard: torch.Tensor, out: torch.Tensor | None = None,
                 time_legs: bool = False) -> torch.Tensor:
        """Run the plan.  With ``time_legs`` every step is bracketed by CUDA events on its stream and
        ``self.timings`` afterwards holds the summed milliseconds per kind of step (the streams
        overlap, so the sums exceed the wall time; they say which leg is long)."""
        lib = self._lib
        if self.status.peek():
            code = self.status.peek()
            self.status.clear()
            self.workspace.zero_()
            raise RuntimeError(f"sharded mm: device wait timed out (code {code & 0xFF}, CTA {code >> 8})")
        if self.exchange == "dma":
            out = self.out
        elif self.layout == "blocked":
            out = self.blocked
        elif out is None:
            raise ValueError("the NCCL exchange needs an output tensor")
        main = torch.cuda.current_stream(self.device)
        streams = {"main": main, **self.streams}
        for side in self.streams.values():
            side.wait_stream(main)  # the operands were produced on the caller's stream
        elt = a.element_size()
        events: list[torch.cuda.Event] = []
        brackets: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        for step in self.plan:
            stream = streams[step.stream]
            panel = self.panels[step.panel]
            for dep in step.after:
                stream.wait_event(events[dep])
            with torch.cuda.stream(stream):
                if time_legs:
                    begin = torch.cuda.Event(enable_timing=True)
                    begin.record(stream)
                local = self.local[step.buf][:panel.rows]
                if step.kind == "gemm":
                    a_panel = a[panel.row0:panel.row0 + panel.rows]
                    lib.gemm("mm", self.dtype, 0, a_panel.data_ptr(), bt_shard.data_ptr(), local.data_ptr(), 1,
                             panel.rows, self.width, self.k, self.cfgs[panel.rows], self.workspace.data_ptr(),
                             self.workspace.numel(), self.status.ptr, stream.cuda_stream)
                elif step.kind == "gather":
                    if self.layout == "blocked":
                        pieces = [self.blocked[j, panel.row0:panel.row0 + panel.rows] for j in range(self.world)]
                        dist.all_gather(pieces, local, group=self.group)
                    else:
                        gathered = self.gathered[step.buf][:, :panel.rows]
                        if panel.rows == self.gathered[step.buf].shape[1]:
                            dist.all_gather_into_tensor(gathered, local, group=self.group)
                        else:
                            dist.all_gather([gathered[j] for j in range(self.world)], local.contiguous(),
                                            group=self.group)
                elif step.kind == "place":
                    if self.layout != "blocked":
                        place_gathered_panel_dma(out, self.gathered[step.buf][:, :panel.rows], panel,
                                                 stream.cuda_stream)
                else:  # push
                    offset = (panel.row0 * self.n + self.col0) * elt
                    for hop in range(self.world):
                        peer = (self.rank + hop) % self.world
                        lib.copy_2d(self.peer_out[peer].data_ptr() + offset, self.n * elt, local.data_ptr(),
                                    self.width * elt, self.width * elt, panel.rows, stream.cuda_stream)
                event = torch.cuda.Event(enable_timing=time_legs)
                event.record(stream)
                events.append(event)
                if time_legs:
                    brackets.append((step.kind, begin, event))
        if self.exchange == "dma":
            with torch.cuda.stream(self.streams["comm"]):
                # every rank's pushes must have landed before anyone reads its out
                self._handle.barrier()
        for side in self.streams.values():
            main.wait_stream(side)
        if time_legs:
            torch.cuda.synchronize(self.device)
            sums: dict[str, float] = {}
            for kind, begin, finish in brackets:
                sums[kind] = sums.get(kind, 0.0) + begin.elapsed_time(finish)
            self.timings = sums
        return out


def nccl_group(max_ctas: int | None = None):
    """A process group over all ranks whose NCCL communicator is limited to ``max_ctas`` thread
    blocks per kernel, so that its kernels fit on the SMs ``NShardedMM`` leaves free."""
    if max_ctas is None:
        return dist.group.WORLD
    options = dist.ProcessGroupNCCL.Options()
    options.config.max_ctas = int(max_ctas)
    options.config.min_ctas = min(int(max_ctas), 4)
    return dist.new_group(ranks=list(range(dist.get_world_size())), pg_options=options)


def bench_sharded(rank: int, world: int, device: torch.device, steps: int = 5) -> dict:
    """Timed runs of the sharded configs at this world size (device time, max over ranks).  Every
    N-sharded result is checked against a single-GPU product on one stripe of rows per M-panel; a
    mismatch ends the run (``SystemExit``)."""
    from .gemm_jit import gemm_op

    results: dict[str, object] = {}

    def timed(fn, reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        dist.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        t = torch.tensor([start.elapsed_time(stop) / reps], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_graph(fn, launches, rounds=5, collective=True):
        """Device time per call of a launch-only ``fn`` replayed from a CUDA graph (the host
        cannot keep up with 20 us kernels from eight processes); max over ranks."""
        stream = torch.cuda.Stream(device=device)
        with torch.cuda.stream(stream):
            for _ in range(3):
                fn()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(launches):
                    fn()
            graph.replay()
            stream.synchronize()
            if collective:
                dist.barrier()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            best = float("inf")
            for _ in range(rounds):
                start.record(stream)
                graph.replay()
                stop.record(stream)
                stream.synchronize()
                best = min(best, start.elapsed_time(stop) / launches)
        if not collective:
            return best
        t = torch.tensor([best], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_local(fn, reps):
        """Single-GPU reference time on this rank (no collective inside)."""
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / reps

    # ---- bmm, batch 64 sharded; operands ~ the benchmark distributions.  Rank 0 also runs the
    # whole batch alone (the other ranks idle) as the single-GPU reference of the speed-up.
    op = gemm_op("bmm", "bfloat16")
    for name, (mm, nn, kk) in (("C3a", (2048, 2048, 128)), ("C3b", (2048, 128, 2048))):
        _, count = partition(64, world, rank)
        a = torch.randn(count, mm, kk, device=device, dtype=torch.bfloat16)
        bt = torch.randn(count, nn, kk, device=device, dtype=torch.bfloat16)
        out = torch.empty(count, mm, nn, device=device, dtype=torch.bfloat16)
        ms = timed_graph(lambda: bmm_sharded(a, bt, out, op), 20)
        flops = 2.0 * 64 * mm * nn * kk
        results[name] = {"ms": ms, "tflops": flops / ms / 1e9, "gbs": 2.0 * 64 * (mm * kk + nn * kk + mm * nn) / ms / 1e6,
                         "partition": f"batch 64 -> {count} per rank, no collective"}
        del a, bt, out
        if rank == 0:
            a = torch.randn(64, mm, kk, device=device, dtype=torch.bfloat16)
            bt = torch.randn(64, nn, kk, device=device, dtype=torch.bfloat16)
            out = torch.empty(64, mm, nn, device=device, dtype=torch.bfloat16)
            one = timed_graph(lambda: op(a, bt, out), 20, collective=False)
            results[name]["one_gpu_ms"] = one
            results[name]["speedup_vs_one_gpu"] = one / ms
            del a, bt, out
        dist.barrier()

    # ---- mm 32768^3, N-sharded; identical seeded operands on every rank so that stripes of the
    # assembled out can be checked against a single-GPU product of the full operands
    big = int(os.environ.get("AYLA_B200_SHARDED_MM_SIZE", "32768"))
    gen = torch.Generator(device=device).manual_seed(200)
    a = torch.empty(big, big, device=device, dtype=torch.bfloat16)
    bt_full = torch.empty(big, big, device=device, dtype=torch.bfloat16)
    for t in (a, bt_full):
        for r0 in range(0, big, 4096):
            t[r0:r0 + 4096] = (torch.randn(4096, big, device=device, generator=gen) * big ** -0.5).bfloat16()
    col0, width = column_block(big, world, rank)
    bt = bt_full[col0:col0 + width].contiguous()
    # one 16-row stripe in the middle of every possible panel (64 stripes cover panels down to 512 rows)
    stripe_rows = torch.cat([torch.arange(r0 + 248, r0 + 264, device=device) for r0 in range(0, big, 512)])
    want = torch.mm(a[stripe_rows], bt_full.t())
    one_gpu_ms = None
    if rank == 0:
        mm_op = gemm_op("mm", "bfloat16")
        full_out = torch.empty(big, big, device=device, dtype=torch.bfloat16)
        one_gpu_ms = timed_local(lambda: mm_op(a, bt_full, full_out), 3)
        del full_out
    dist.barrier()
    del bt_full

    def check(got_rows: torch.Tensor, what: str) -> float:
        err = float((got_rows.float() - want.float()).norm() / want.float().norm())
        bad = torch.tensor([1.0 if not err < 2e-3 else 0.0], device=device)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if float(bad.item()) != 0.0:
            raise SystemExit(f"sharded mm ({what}): assembled result differs from the single-GPU product "
                             f"(Frobenius rel {err:.3e} on the checked stripes of rank {rank})")
        return err

    def run_variant(key, exchange, layout="row_major", max_ctas=None, reserve_sms=16, panel_rows=None, legs=False):
        group = nccl_group(max_ctas) if exchange == "nccl" else None
        runner = NShardedMM(big, big, big, "bfloat16", device, group=group, exchange=exchange, layout=layout,
                            reserve_sms=reserve_sms, panel_rows=panel_rows)
        out = None
        if exchange == "nccl" and layout == "row_major":
            out = torch.zeros(big, big, device=device, dtype=torch.bfloat16)
        elif exchange == "dma":
            runner.out.zero_()
        ms = timed(lambda: runner(a, bt, out), max(1, steps // 3))
        if layout == "blocked":
            got = torch.cat([runner.blocked[j][stripe_rows] for j in range(world)], dim=1)
        else:
            got = (runner.out if exchange == "dma" else out)[stripe_rows]
        err = check(got, key)
        row = {"ms": ms, "tflops": 2.0 * big ** 3 / ms / 1e9, "fro_rel_vs_full_product_on_64_stripes": err,
               "one_gpu_ms": one_gpu_ms, "speedup_vs_one_gpu": (one_gpu_ms / ms) if one_gpu_ms else None,
               "status": int(runner.status.peek()), "nccl_max_ctas": max_ctas, "reserve_sms": reserve_sms,
               "partition": f"N -> {runner.width} columns per rank, {exchange} exchange of out in "
                            f"{len(runner.panels)} M-panels, result layout {layout}"}
        if legs:
            runner(a, bt, out, time_legs=True)
            row["leg_ms_summed_over_panels"] = runner.timings
        del runner, out
        torch.cuda.empty_cache()
        return row

    # The NCCL all-gather path: a small sweep of how many thread blocks NCCL may use against how many
    # SMs the GEMM leaves it, then the best pair again with its legs timed.
    sweep = []
    # (NCCL thread blocks, SMs left free): NCCL's blocks are small enough to share an SM, so fewer SMs than
    # blocks may be set aside.
    # The third entry is the panel height: None = sixteen panels, "fit" = whole waves of the SMs the GEMM keeps.
    choices = (((32, 32, None), (32, 32, "fit"), (48, 48, None), (32, 16, None), (64, 24, None)) if world > 2
               else ((16, 16, None), (16, 16, "fit")))
    for max_ctas, reserve, rows in choices:
        try:
            row = run_variant(f"nccl max_ctas={max_ctas} reserve={reserve} rows={rows}", "nccl", max_ctas=max_ctas,
                              reserve_sms=reserve, panel_rows=rows)
            row["panel_rows"] = rows
            sweep.append(row)
        except SystemExit:
            raise
        except Exception as exc:  # noqa: BLE001 - reported, not fatal for the headline line
            sweep.append({"nccl_max_ctas": max_ctas, "reserve_sms": reserve, "panel_rows": rows,
                          "error": f"{type(exc).__name__}: {exc}"})
    good = [r for r in sweep if "ms" in r]
    if good:
        best = min(good, key=lambda r: r["ms"])
        try:
            results["mm32768"] = run_variant("nccl best", "nccl", max_ctas=best["nccl_max_ctas"],
                                             reserve_sms=best["reserve_sms"], panel_rows=best["panel_rows"], legs=True)
        except SystemExit:
            raise
        except Exception as exc:  # noqa: BLE001
            results["mm32768"] = {"error": f"{type(exc).__name__}: {exc}"}
        results["mm32768_sweep"] = [{k: r.get(k) for k in ("nccl_max_ctas", "reserve_sms", "panel_rows", "partition", "ms",
                                                           "speedup_vs_one_gpu", "error")}
                                    for r in sweep]
        for key, kwargs in (("mm32768_blocked_layout", dict(exchange="nccl", layout="blocked",
                                                            max_ctas=best["nccl_max_ctas"], reserve_sms=best["reserve_sms"],
                                                            panel_rows=best["panel_rows"])),
                            ("mm32768_dma", dict(exchange="dma"))):
            try:
                results[key] = run_variant(key, **kwargs)
            except SystemExit:
                raise
            except Exception as exc:  # noqa: BLE001
                results[key] = {"error": f"{type(exc).__name__}: {exc}"}
    else:
        results["mm32768"] = {"error": "; ".join(str(r.get("error")) for r in sweep)}
    return results if rank == 0 else {}


def n_sharded_mm_by_plan(a: torch.Tensor, bt_shard: torch.Tensor, out: torch.Tensor, gemm_fn, group=None,
                         panel_rows: int = 4096, pick=None) -> list[int]:
    """``NShardedMM``'s plan executed with ordinary tensor operations: the same steps, the same two
    local and two gather buffers reused across panels, run one at a time in an order that respects
    the plan's dependencies and is otherwise chosen by ``pick`` (see ``run_plan_in_order``).
    Device-agnostic, so CPU ranks can check that the dependencies alone keep the buffers safe.
    Collectives are all on one stream of the plan, hence issued in the same order on every rank."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    m, n = out.shape
    _, width = column_block(n, world, rank)
    if bt_shard.shape[0] != width:
        raise ValueError(f"rank {rank}: bt shard has {bt_shard.shape[0]} rows, expected {width}")
    panels = m_panels(m, panel_rows)
    rows = panels[0].rows
    local = [torch.full((rows, width), float("nan"), dtype=out.dtype, device=out.device) for _ in range(2)]
    gathered = [torch.full((world, rows, width), float("nan"), dtype=out.dtype, device=out.device) for _ in range(2)]

    def execute(step: Step) -> None:
        panel = panels[step.panel]
        if step.kind == "gemm":
            gemm_fn(a[panel.row0:panel.row0 + panel.rows], bt_shard, local[step.buf][:panel.rows])
        elif step.kind == "gather":
            pieces = [torch.empty(panel.rows, width, dtype=out.dtype, device=out.device) for _ in range(world)]
            dist.all_gather(pieces, local[step.buf][:panel.rows].contiguous(), group=group)
            gathered[step.buf][:, :panel.rows] = torch.stack(pieces)
            local[step.buf].fill_(float("nan"))  # the buffer is free again: a later reader must not rely on it
        elif step.kind == "place":
            place_gathered_panel(out, gathered[step.buf][:, :panel.rows], panel)
            gathered[step.buf].fill_(float("nan"))
        else:
            raise ValueError(f"step {step.kind} has no CPU form")

    return run_plan_in_order(overlap_plan(len(panels), "nccl"), execute, pick)


def n_sharded_mm_unoverlapped(a: torch.Tensor, bt_shard: torch.Tensor, out: torch.Tensor, gemm_fn,
                              group=None, panel_rows: int = 4096) -> None:
    """The same partition / panel / gather / placement sequence as ``NShardedMM`` without
    streams: ``gemm_fn(a_panel, bt_shard, local_out)`` computes one panel of this rank's
    column block.  Device-agnostic, so the data movement can be checked on CPU ranks."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    m, n = out.shape
    _, width = column_block(n, world, rank)
    if bt_shard.shape[0] != width:
        raise ValueError(f"rank {rank}: bt shard has {bt_shard.shape[0]} rows, expected {width}")
    for panel in m_panels(m, panel_rows):
        local = torch.empty(panel.rows, width, dtype=out.dtype, device=out.device)
        gemm_fn(a[panel.row0:panel.row0 + panel.rows], bt_shard, local)
        pieces = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(pieces, local, group=group)
        place_gathered_panel(out, torch.stack(pieces), panel)
