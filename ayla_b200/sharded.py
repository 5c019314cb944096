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


class NShardedMM:
    """``out[M, N] = a[M, K] @ bt[N, K]^T`` with bt sharded by rows across the group.

    Every rank ends up with the full ``out``.  Two ways to exchange the column blocks:

    * ``exchange="nccl"`` (the default): every finished M-panel is all-gathered with NCCL on
      a second stream as ``[g][rows][N/g]`` and put in place by strided DMA copies while the
      GEMM of the next panel runs; ``reserve_sms`` SMs are left free of GEMM CTAs so NCCL's
      kernels can run beside it.
    * ``exchange="dma"``: ``out`` lives in symmetric memory and every rank pushes its finished
      panel block straight into every peer's ``out`` with strided peer-to-peer copies on the
      copy engines (plain stores over NVLink, no SMs, no staging, nothing to un-permute); one
      barrier at the end.  Use ``runner.out`` as the output tensor.
    """

    def __init__(self, m: int, n: int, k: int, dtype: str, device: torch.device, group=None,
                 panel_rows: int | None = None, reserve_sms: int = 16, exchange: str = "nccl"):
        from . import _lib
        from .gemm_jit import _TORCH_DTYPES, select_gemm_schedule

        if exchange not in ("nccl", "dma"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.exchange = exchange
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.m, self.n, self.k, self.dtype = m, n, k, dtype
        self.col0, self.width = column_block(n, self.world, self.rank)
        if panel_rows is None:
            # Four panels: each is several full waves of tiles (little wave quantisation) and
            # only the last panel's exchange is left uncovered by compute.
            panel_rows = max(2048, -(-m // 4))
        self.panels = m_panels(m, panel_rows)
        self.device = device
        _lib.init(device.index)
        self._lib = _lib
        torch_dtype = _TORCH_DTYPES[dtype]
        self.torch_dtype = torch_dtype
        rows = self.panels[0].rows
        # double-buffered local panel (and gather target for the NCCL exchange)
        self.local = [torch.empty(rows, self.width, dtype=torch_dtype, device=device) for _ in range(2)]
        seed = select_gemm_schedule("mm", dtype, rows, self.width, k)
        if seed is None:
            raise ValueError(f"no schedule for panel {rows}x{self.width}x{k}")
        cfg = dict(seed.builder_config)
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.out = None
        self.peer_out: list[torch.Tensor] = []
        if exchange == "nccl":
            self.gathered = [torch.empty(self.world, rows, self.width, dtype=torch_dtype, device=device)
                             for _ in range(2)]
            if self.world > 1 and reserve_sms > 0:
                cfg["grid_ctas"] = (sms - reserve_sms) & ~1
        else:
            import torch.distributed._symmetric_memory as symm_mem

            self.out = symm_mem.empty((m, n), dtype=torch_dtype, device=device)
            self._handle = symm_mem.rendezvous(self.out, self.group)
            self.peer_out = [self._handle.get_buffer(r, (m, n), torch_dtype) for r in range(self.world)]
        self.cfg = _lib.Config.from_dict(cfg)
        need = _lib.workspace_bytes(self.cfg, "mm", 1, rows, self.width, k)
        self.workspace = torch.zeros(max(need, 16), dtype=torch.uint8, device=device)
        self.comm_stream = torch.cuda.Stream(device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def __call__(self, a: torch.Tensor, bt_shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        lib = self._lib
        if self.exchange == "dma":
            out = self.out
        elif out is None:
            raise ValueError("the NCCL exchange needs an output tensor")
        main = torch.cuda.current_stream(self.device)
        elt = out.element_size()
        done_events = []
        for i, panel in enumerate(self.panels):
            buf = i % 2
            if i >= 2:
                # the exchange that last read this local buffer must be finished
                main.wait_event(done_events[i - 2])
            local = self.local[buf][:panel.rows]
            a_panel = a[panel.row0:panel.row0 + panel.rows]
            lib.gemm("mm", self.dtype, 0, a_panel.data_ptr(), bt_shard.data_ptr(), local.data_ptr(), 1,
                     panel.rows, self.width, self.k, self.cfg, self.workspace.data_ptr(), self.workspace.numel(),
                     self.status.data_ptr(), main.cuda_stream)
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                if self.exchange == "nccl":
                    gathered = self.gathered[buf][:, :panel.rows]
                    if panel.rows == self.gathered[buf].shape[1]:
                        dist.all_gather_into_tensor(gathered, local, group=self.group)
                    else:
                        pieces = [torch.empty_like(local) for _ in range(self.world)]
                        dist.all_gather(pieces, local.contiguous(), group=self.group)
                        gathered = torch.stack(pieces)
                    place_gathered_panel_dma(out, gathered, panel, self.comm_stream.cuda_stream)
                else:
                    offset = (panel.row0 * self.n + self.col0) * elt
                    for step in range(self.world):
                        peer = (self.rank + step) % self.world
                        lib.copy_2d(self.peer_out[peer].data_ptr() + offset, self.n * elt, local.data_ptr(),
                                    self.width * elt, self.width * elt, panel.rows, self.comm_stream.cuda_stream)
                done = torch.cuda.Event()
                done.record(self.comm_stream)
            done_events.append(done)
        if self.exchange == "dma":
            with torch.cuda.stream(self.comm_stream):
                # every rank's pushes must have landed before anyone reads its out
                self._handle.barrier()
        main.wait_stream(self.comm_stream)
        return out


def bench_sharded(rank: int, world: int, device: torch.device, steps: int = 5) -> dict:
    """Timed runs of the sharded configs at this world size (device time, max over ranks)."""
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

    # ---- mm 32768^3, N-sharded; identical seeded operands on every rank so a row panel of
    # the assembled out can be checked against a single-GPU product of the full operands
    big = int(os.environ.get("AYLA_B200_SHARDED_MM_SIZE", "32768"))
    gen = torch.Generator(device=device).manual_seed(200)
    a = torch.empty(big, big, device=device, dtype=torch.bfloat16)
    bt_full = torch.empty(big, big, device=device, dtype=torch.bfloat16)
    for t in (a, bt_full):
        for r0 in range(0, big, 4096):
            t[r0:r0 + 4096] = (torch.randn(4096, big, device=device, generator=gen) * big ** -0.5).bfloat16()
    col0, width = column_block(big, world, rank)
    bt = bt_full[col0:col0 + width].contiguous()
    check_rows = slice(big // 2 - 128, big // 2 + 128)
    want = torch.mm(a[check_rows], bt_full.t())
    one_gpu_ms = None
    if rank == 0:
        mm_op = gemm_op("mm", "bfloat16")
        full_out = torch.empty(big, big, device=device, dtype=torch.bfloat16)
        one_gpu_ms = timed_local(lambda: mm_op(a, bt_full, full_out), 3)
        del full_out
    dist.barrier()
    del bt_full
    for exchange in ("nccl", "dma"):
        key = "mm32768" if exchange == "nccl" else "mm32768_dma"
        try:
            runner = NShardedMM(big, big, big, "bfloat16", device, exchange=exchange)
            out = runner.out if exchange == "dma" else torch.empty(big, big, device=device, dtype=torch.bfloat16)
            out.zero_()
            ms = timed(lambda: runner(a, bt, out), max(1, steps // 3))
            err = (out[check_rows].float() - want.float()).norm() / want.float().norm()
            results[key] = {"ms": ms, "tflops": 2.0 * big ** 3 / ms / 1e9, "fro_rel_vs_full_product": float(err),
                            "one_gpu_ms": one_gpu_ms,
                            "speedup_vs_one_gpu": (one_gpu_ms / ms) if one_gpu_ms else None,
                            "status": int(runner.status.item()),
                            "partition": f"N -> {runner.width} columns per rank, {exchange} exchange of out in "
                                         f"{len(runner.panels)} M-panels"}
            del runner, out
        except Exception as exc:  # noqa: BLE001 - reported, not fatal for the headline line
            results[key] = {"error": f"{type(exc).__name__}: {exc}"}
        torch.cuda.empty_cache()
    return results if rank == 0 else {}


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
