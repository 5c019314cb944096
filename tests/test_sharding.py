"""Partition arithmetic and the gather/placement data movement of the sharded GEMMs,
on two CPU ranks over gloo (no GPU).  The per-rank GEMM is played by the CPU oracle."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ayla_b200 import sharded
from oracle import gemm_oracle as O


def test_partition_covers_everything_once():
    for total, world in ((64, 8), (64, 4), (10, 4), (3, 8), (1, 1)):
        blocks = [sharded.partition(total, world, r) for r in range(world)]
        assert blocks[0][0] == 0
        for (s0, c0), (s1, _) in zip(blocks, blocks[1:]):
            assert s0 + c0 == s1
        assert blocks[-1][0] + blocks[-1][1] == total
        assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1
    with pytest.raises(ValueError):
        sharded.partition(8, 2, 2)


def test_column_blocks_and_panels():
    assert [sharded.column_block(32768, 8, r) for r in (0, 7)] == [(0, 4096), (28672, 4096)]
    with pytest.raises(ValueError):
        sharded.column_block(100, 8, 0)      # not divisible
    with pytest.raises(ValueError):
        sharded.column_block(8 * 12, 8, 0)   # blocks of 12 columns: not 16-byte rows
    panels = sharded.m_panels(10000, 4096)
    assert [(p.row0, p.rows) for p in panels] == [(0, 4096), (4096, 4096), (8192, 1808)]


def test_panel_height_is_fitted_to_whole_waves_of_the_sms_the_gemm_keeps():
    """A 256-row tile occupies a CTA pair: with 32 SMs left to NCCL, 58 pairs take the 16 column tiles
    of 7 row tiles (112 tiles) in two waves; 2048 rows (128 tiles) would need three."""
    assert sharded.fit_panel_rows(32768, 4096, 148 - 32) == 7 * 256
    assert sharded.fit_panel_rows(32768, 4096, 148) == 9 * 256           # 144 of 148 pair slots in two waves
    for m, width, sms in ((32768, 4096, 116), (32768, 16384, 132), (16384, 8192, 132), (32768, 4096, 100)):
        rows = sharded.fit_panel_rows(m, width, sms)
        tiles = (rows // 256) * -(-width // 256)
        waves = -(-tiles // (sms // 2))
        assert rows % 256 == 0 and tiles / (waves * (sms // 2)) >= 0.95
        assert len(sharded.m_panels(m, rows)) <= 24
    # small problems: one panel, never taller than the matrix rounded up to a tile
    assert sharded.fit_panel_rows(1000, 512, 148) == 1024
    assert len(sharded.m_panels(1000, sharded.fit_panel_rows(1000, 512, 148))) == 1


def test_place_gathered_panel_unpermutes():
    out = torch.zeros(6, 8)
    gathered = torch.arange(2 * 3 * 4, dtype=torch.float32).view(2, 3, 4)
    sharded.place_gathered_panel(out, gathered, sharded.Panel(2, 3))
    assert torch.equal(out[2], torch.tensor([0., 1, 2, 3, 12, 13, 14, 15]))
    assert torch.equal(out[4], torch.tensor([8., 9, 10, 11, 20, 21, 22, 23]))
    assert not out[:2].any() and not out[5:].any()


def test_overlap_plan_orders_exactly_what_double_buffering_needs():
    plan = sharded.overlap_plan(5, "nccl")
    kinds = [(s.kind, s.panel) for s in plan]
    assert kinds[:6] == [("gemm", 0), ("gather", 0), ("place", 0), ("gemm", 1), ("gather", 1), ("place", 1)]
    at = {(s.kind, s.panel): i for i, s in enumerate(plan)}
    for i in range(5):
        assert plan[at["gemm", i]].stream == "main" and plan[at["gather", i]].stream == "comm"
        assert plan[at["place", i]].stream == "place" and plan[at["gemm", i]].buf == i % 2
        assert at["gemm", i] in plan[at["gather", i]].after          # gather after its GEMM
        assert at["gather", i] in plan[at["place", i]].after         # placement after its gather
        if i >= 2:
            assert at["gather", i - 2] in plan[at["gemm", i]].after  # local buffer reuse
            assert at["place", i - 2] in plan[at["gather", i]].after  # gather buffer reuse
    # every dependency points backwards: the plan can be issued to streams in list order
    assert all(dep < i for i, s in enumerate(plan) for dep in s.after)
    dma = sharded.overlap_plan(3, "dma")
    assert [s.kind for s in dma] == ["gemm", "push"] * 3 and dma[4].after == (1,)
    with pytest.raises(ValueError):
        sharded.overlap_plan(3, "smoke signals")


def test_run_plan_in_order_respects_streams_and_dependencies():
    import random

    plan = sharded.overlap_plan(6, "nccl")
    rng = random.Random(5)
    for _ in range(20):
        order = sharded.run_plan_in_order(plan, lambda step: None, pick=rng.choice)
        assert sorted(order) == list(range(len(plan)))
        position = {index: at for at, index in enumerate(order)}
        for index, step in enumerate(plan):
            assert all(position[dep] < position[index] for dep in step.after)
        for stream in ("main", "comm", "place"):
            on_stream = [i for i in order if plan[i].stream == stream]
            assert on_stream == sorted(on_stream)
    # a plan that waits on something that never runs is reported, not spun on
    broken = [sharded.Step("gemm", 0, 0, "main", (1,)), sharded.Step("gather", 0, 0, "comm", (0,))]
    with pytest.raises(RuntimeError, match="deadlock"):
        sharded.run_plan_in_order(broken, lambda step: None)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)          # same operands on every rank
        m, n, k = 200, 64 * world, 96
        a = torch.randn(m, k, generator=g).bfloat16()
        bt = (torch.randn(n, k, generator=g) * k ** -0.5).bfloat16()
        full = O.gemm_ref("mm", torch.bfloat16, a, bt)

        # N-sharded mm: this rank only ever sees its row block of bt
        col0, width = sharded.column_block(n, world, rank)
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16)
        sharded.n_sharded_mm_unoverlapped(
            a, bt[col0:col0 + width].contiguous(), out,
            lambda ap, bs, local: local.copy_(O.gemm_ref("mm", torch.bfloat16, ap, bs)), panel_rows=64)
        ok_mm = torch.equal(out.view(torch.int16), full.view(torch.int16))

        # the overlapped runner's plan, its buffers reused across panels, executed in a random order
        # that respects the plan's dependencies only (a different order on every rank)
        import random

        out2 = torch.full((m, n), float("nan"), dtype=torch.bfloat16)
        rng = random.Random(100 + rank)
        order = sharded.n_sharded_mm_by_plan(
            a, bt[col0:col0 + width].contiguous(), out2,
            lambda ap, bs, local: local.copy_(O.gemm_ref("mm", torch.bfloat16, ap, bs)), panel_rows=24, pick=rng.choice)
        ok_mm = ok_mm and torch.equal(out2.view(torch.int16), full.view(torch.int16)) and len(order) == 3 * 9

        # batch-sharded bmm: slices are independent; gather only to compare
        batch = 5
        a3 = torch.randn(batch, 40, 32, generator=g).bfloat16()
        bt3 = torch.randn(batch, 24, 32, generator=g).bfloat16()
        start, count = sharded.partition(batch, world, rank)
        mine = torch.empty(count, 40, 24, dtype=torch.bfloat16)
        sharded.bmm_sharded(a3[start:start + count], bt3[start:start + count], mine,
                            lambda x, y, o: o.copy_(O.gemm_ref("bmm", torch.bfloat16, x, y)))
        gathered = [None] * world
        dist.all_gather_object(gathered, (start, mine))
        whole = torch.cat([t for _, t in sorted(gathered, key=lambda p: p[0])])
        ok_bmm = torch.equal(whole.view(torch.int16), O.gemm_ref("bmm", torch.bfloat16, a3, bt3).view(torch.int16))

        # a rank with a wrong shard is caught before any collective
        try:
            sharded.n_sharded_mm_unoverlapped(a, bt[: width + 8].contiguous(), out, None)
            ok_err = False
        except ValueError:
            ok_err = True
        results[rank] = (ok_mm, ok_bmm, ok_err)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_flows_on_gloo_ranks(world):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {rank: (True, True, True) for rank in range(world)}
