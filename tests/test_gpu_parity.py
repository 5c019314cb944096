"""Parity of the CUDA path with the CPU oracle, on a B200.

Every test reaches the kernels through the C ABI (directly via ``ayla_b200._lib`` or
through the ``torch.ops.ayla`` ops, whose CUDA implementation is a ctypes call into
the same ABI).  Tolerance (the project's, written once in ``oracle.gemm_oracle``):
Frobenius relative error <= 5e-3 and max elementwise error <= 2e-2 * rms(ref) against
the CPU fp32 result rounded to the output type; elements that miss the second bound
while being the neighbouring representable value of the reference are rounding flips
of the last bit and are counted, not failed (``Parity.ok``).
"""

import pytest
import torch

from ayla_b200 import _lib, gemm_op, gemm_op_compiler, swiglu_op, swiglu_op_compiler
from ayla_b200.gemm_jit import gemm_jit_compiler
from oracle import gemm_oracle as O
from tests.conftest import load_golden_cases

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TD = {"float16": torch.float16, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def device_state():
    _lib.init(0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    workspace = torch.zeros(64 << 20, dtype=torch.uint8, device=DEV)
    return status, workspace


def run_abi(operation, dtype, tensors, cfg, device_state, canary_rows=4):
    """Launch through the C ABI with an explicit schedule; returns (out, status)."""
    status, workspace = device_state
    status.zero_()
    dev = [t.to(DEV) for t in tensors]
    if operation == "swiglu":
        x, wg, wu = dev
        m, k = x.shape
        n = wg.shape[0]
        store = torch.full((m + canary_rows, n), float("nan"), dtype=x.dtype, device=DEV)
        out = store[:m]
        _lib.swiglu(dtype, x.data_ptr(), wg.data_ptr(), wu.data_ptr(), out.data_ptr(), m, n, k,
                    _lib.Config.from_dict(cfg) if cfg else None, status.data_ptr(),
                    torch.cuda.current_stream().cuda_stream)
    else:
        bias = dev[0] if operation == "addmm" else None
        a, bt = dev[-2:]
        batch = a.shape[0] if operation == "bmm" else 1
        m, k = a.shape[-2:]
        n = bt.shape[-2]
        rows = batch * m
        store = torch.full((rows + canary_rows, n), float("nan"), dtype=a.dtype, device=DEV)
        out = store[:rows].view(*a.shape[:-2], m, n)
        _lib.gemm(operation, dtype, bias.data_ptr() if bias is not None else 0, a.data_ptr(),
                  bt.data_ptr(), out.data_ptr(), batch, m, n, k,
                  _lib.Config.from_dict(cfg) if cfg else None, workspace.data_ptr(), workspace.numel(),
                  status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    # rows past the end of `out` must still hold their poison
    assert bool(torch.isnan(store[store.shape[0] - canary_rows:]).all()), "kernel wrote past the output"
    return out, int(status.item())


def assert_parity(out, ref32, what=""):
    parity = O.compare(out, ref32)
    assert parity.ok, f"{what}: {parity}"
    return parity


# ------------------------------------------------------------------ golden vectors

@pytest.mark.parametrize("case", load_golden_cases(), ids=repr)
def test_ops_reproduce_golden_vectors(case):
    operands = [t.to(DEV) for t in case.operands()]
    want = case.expected()
    out = torch.full(want.shape, float("nan"), dtype=case.torch_dtype, device=DEV)
    if case.operation == "swiglu":
        assert swiglu_op(case.dtype)(*operands, out) is None
    else:
        assert gemm_op(case.operation, case.dtype)(*operands, out) is None
    torch.cuda.synchronize()
    got = out.cpu()
    parity = O.compare(got, want.float())
    assert parity.ok, parity
    # Beyond the project tolerance: a different fp32 summation order can only flip the
    # last bit, and only on a small fraction of elements.
    differing = int((got.view(torch.int16) != want.view(torch.int16)).sum())
    assert differing <= max(2, got.numel() // 200), (differing, got.numel())
    rms = float(want.float().pow(2).mean().sqrt())
    ulp = O._ulp(want.float().abs().clamp_min(1e-2 * rms), case.torch_dtype)
    assert bool(((got.float() - want.float()).abs() <= ulp * 1.0001).all())


# ------------------------------------- the reference's own GPU test, op for op

@pytest.mark.parametrize("operation", ["mm", "addmm", "bmm"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(96, 128, 128), (256, 256, 256)])
def test_jit_matches_torch_and_replays_cuda_graph(operation, dtype, m, n, k):
    """tests/test_gemm_jit.py:49-75 of the reference, same shapes and tolerances."""
    compiler = gemm_jit_compiler(operation, str(dtype).removeprefix("torch."))
    lead = (2,) if operation == "bmm" else ()
    a = torch.randn((*lead, m, k), device=DEV, dtype=dtype)
    bt = torch.randn((*lead, n, k), device=DEV, dtype=dtype)
    out = torch.empty((*lead, m, n), device=DEV, dtype=dtype)
    args = [a, bt, out]
    expected = a @ bt.transpose(-1, -2)
    if operation == "addmm":
        bias = torch.randn(n, device=DEV, dtype=dtype)
        args.insert(0, bias)
        expected = torch.addmm(bias, a, bt.T)
    compiler(*args)
    torch.testing.assert_close(out, expected, atol=0.125, rtol=0.02)
    assert compiler.cache_size == 1
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        compiler(*args)
    out.zero_()
    graph.replay()
    torch.testing.assert_close(out, expected, atol=0.125, rtol=0.02)
    assert compiler.cache_size == 1


def test_capture_time_cache_miss_is_an_error():
    compiler = gemm_jit_compiler("mm", "bfloat16")
    a = torch.randn(64, 64, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(64, 64, device=DEV, dtype=torch.bfloat16)
    graph = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="before capture"):
        with torch.cuda.graph(graph):
            compiler(a, a, out)


# --------------------------------------------------- every kernel variant, ragged

ROW_MAJOR = [(tile_n, cta_group) for tile_n in (64, 128, 192, 256) for cta_group in (1, 2)]
SHAPES = [
    ("mm", 1, 128, 256, 64), ("mm", 1, 96, 128, 128), ("mm", 1, 333, 520, 200), ("mm", 1, 1, 8, 8),
    ("addmm", 1, 300, 264, 192), ("bmm", 3, 200, 136, 128), ("mm", 1, 1024, 768, 520),
]


@pytest.mark.parametrize("tile_n,cta_group", ROW_MAJOR)
@pytest.mark.parametrize("split_k", [1, 3])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_row_major_variants(tile_n, cta_group, split_k, dtype, device_state):
    torch.manual_seed(tile_n + cta_group + split_k)
    cfg = dict(tile_n=tile_n, cta_group=cta_group, split_k=split_k, group_m=3)
    for operation, batch, m, n, k in SHAPES:
        lead = (batch,) if operation == "bmm" else ()
        a = torch.randn((*lead, m, k)).to(TD[dtype])
        bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
        tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
        out, status = run_abi(operation, dtype, tensors, cfg, device_state)
        assert status == 0
        assert_parity(out, O.gemm_ref32(operation, *tensors), f"{operation} {batch}x{m}x{n}x{k} {cfg}")


@pytest.mark.parametrize("tile_n", [16, 32, 64, 128])
@pytest.mark.parametrize("split_k", [1, 4])
def test_swapped_variants(tile_n, split_k, device_state):
    torch.manual_seed(tile_n * 7 + split_k)
    cfg = dict(tile_n=tile_n, cta_group=1, swap_ab=1, split_k=split_k, group_m=1)
    for dtype in ("bfloat16", "float16"):
        for operation, batch, m, n, k in (("mm", 1, 1, 256, 512), ("mm", 1, tile_n, 520, 264),
                                          ("addmm", 1, max(1, tile_n - 3), 264, 192),
                                          ("bmm", 3, tile_n, 136, 128), ("mm", 1, 3 * tile_n + 5, 1024, 512)):
            lead = (batch,) if operation == "bmm" else ()
            a = torch.randn((*lead, m, k)).to(TD[dtype])
            bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
            tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
            out, status = run_abi(operation, dtype, tensors, cfg, device_state)
            assert status == 0
            assert_parity(out, O.gemm_ref32(operation, *tensors), f"{operation} {batch}x{m}x{n}x{k} {cfg}")


@pytest.mark.parametrize("tile_rows", [8, 56, 97, 104, 120])
def test_swapped_tiles_with_fewer_rows(tile_rows, device_state):
    """tile_rows < 128: more, lighter tiles of bt; rows past the trimmed tile are never stored."""
    torch.manual_seed(tile_rows)
    for tile_n, split in ((16, dict()), (32, dict(split_k=2)), (64, dict(split_k=2, cluster_split=1)), (128, dict())):
        cfg = dict(tile_n=tile_n, cta_group=1, swap_ab=1, group_m=1, tile_rows=tile_rows, **split)
        for operation, dtype, batch, m, n, k in (("mm", "bfloat16", 1, min(tile_n, 24), 1000, 512),
                                                 ("addmm", "float16", 1, tile_n, 776, 320),
                                                 ("bmm", "bfloat16", 2, max(1, tile_n - 5), 264, 256)):
            assert _lib.config_valid(_lib.Config.from_dict(cfg), operation, dtype, batch, m, n, k), cfg
            lead = (batch,) if operation == "bmm" else ()
            a = torch.randn((*lead, m, k)).to(TD[dtype])
            bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
            tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
            out, status = run_abi(operation, dtype, tensors, cfg, device_state)
            assert status == 0
            assert_parity(out, O.gemm_ref32(operation, *tensors), f"{operation} {batch}x{m}x{n}x{k} {cfg}")


@pytest.mark.parametrize("split_k", [2, 4, 8])
def test_cluster_split_k_variants(split_k, device_state):
    """k-splits as the CTAs of one cluster, reduced through distributed shared memory."""
    torch.manual_seed(split_k)
    for tile_n, swap in ((64, 0), (128, 0), (256, 0), (32, 1), (64, 1), (128, 1)):
        cfg = dict(tile_n=tile_n, cta_group=1, swap_ab=swap, split_k=split_k, cluster_split=1, group_m=1 if swap else 8)
        for operation, dtype, batch, m, n, k in (("mm", "bfloat16", 1, 333 if not swap else tile_n - 3, 520, 1000),
                                                 ("addmm", "float16", 1, 256 if not swap else tile_n, 264, 1024),
                                                 ("bmm", "bfloat16", 2, 200 if not swap else 8, 136, 512)):
            if not _lib.config_valid(_lib.Config.from_dict(cfg), operation, dtype, batch, m, n, k):
                continue
            lead = (batch,) if operation == "bmm" else ()
            a = torch.randn((*lead, m, k)).to(TD[dtype])
            bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
            tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
            out, status = run_abi(operation, dtype, tensors, cfg, device_state)
            assert status == 0
            assert_parity(out, O.gemm_ref32(operation, *tensors), f"{operation} {batch}x{m}x{n}x{k} {cfg}")
    # deterministic: the partials are added in rank order
    op, tensors = O.make_inputs("C2b", "bfloat16", scale_down=4)
    cfg = dict(tile_n=64, cta_group=1, split_k=split_k, cluster_split=1)
    first, _ = run_abi(op, "bfloat16", tensors, cfg, device_state)
    again, _ = run_abi(op, "bfloat16", tensors, cfg, device_state)
    assert torch.equal(first, again)


@pytest.mark.parametrize("tile_n,cta_group", [(128, 1), (256, 1), (128, 2), (256, 2)])
@pytest.mark.parametrize("grid_ctas", [0, 10, 36])
def test_stream_k_variants(tile_n, cta_group, grid_ctas, device_state):
    """Equal contiguous shares of the (tile, k-block) sequence per CTA: tiles cut between CTAs are
    finished by the last contributor, summing in CTA order."""
    torch.manual_seed(tile_n + cta_group + grid_ctas)
    cfg = dict(tile_n=tile_n, cta_group=cta_group, stream_k=1, group_m=3, grid_ctas=grid_ctas)
    for operation, dtype, batch, m, n, k in (("mm", "bfloat16", 1, 1024, 768, 520), ("addmm", "float16", 1, 300, 264, 1992),
                                             ("bmm", "bfloat16", 3, 200, 136, 1024), ("mm", "float16", 1, 333, 520, 4104)):
        assert _lib.config_valid(_lib.Config.from_dict(cfg), operation, dtype, batch, m, n, k), cfg
        lead = (batch,) if operation == "bmm" else ()
        a = torch.randn((*lead, m, k)).to(TD[dtype])
        bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
        tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
        out, status = run_abi(operation, dtype, tensors, cfg, device_state)
        assert status == 0
        assert_parity(out, O.gemm_ref32(operation, *tensors), f"{operation} {batch}x{m}x{n}x{k} {cfg}")
        again, _ = run_abi(operation, dtype, tensors, cfg, device_state)
        assert torch.equal(out, again)


@pytest.mark.parametrize("split_k", [2, 4])
@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_paired_cluster_split_k_variants(split_k, tile_n, device_state):
    """k-splits of a 256-row tile as the CTA pairs of one cluster (4 or 8 CTAs)."""
    torch.manual_seed(split_k * 1000 + tile_n)
    cfg = dict(tile_n=tile_n, cta_group=2, split_k=split_k, cluster_split=1, group_m=2)
    for operation, dtype, batch, m, n, k in (("mm", "bfloat16", 1, 333, 520, 1000), ("mm", "float16", 1, 256, 256, 512),
                                             ("addmm", "float16", 1, 512, 264, 1024), ("addmm", "bfloat16", 1, 130, 72, 2048),
                                             ("bmm", "bfloat16", 2, 200, 136, 512), ("mm", "bfloat16", 1, 1024, 1024, 4096)):
        assert _lib.config_valid(_lib.Config.from_dict(cfg), operation, dtype, batch, m, n, k)
        assert _lib.workspace_bytes(_lib.Config.from_dict(cfg), operation, batch, m, n, k) == 0
        lead = (batch,) if operation == "bmm" else ()
        a = torch.randn((*lead, m, k)).to(TD[dtype])
        bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
        tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
        out, status = run_abi(operation, dtype, tensors, cfg, device_state)
        assert status == 0
        assert_parity(out, O.gemm_ref32(operation, *tensors), f"{operation} {batch}x{m}x{n}x{k} {cfg}")
        again, _ = run_abi(operation, dtype, tensors, cfg, device_state)
        assert torch.equal(out, again)


def test_launch_overlap_keeps_stream_order(device_state):
    """A chain of launches, each reading what the one before wrote, gives the same bits whether
    or not a launch may start its set-up under its predecessor's tail."""
    torch.manual_seed(5)
    n = 1024
    x0 = torch.randn(256, n).to(torch.bfloat16).to(DEV)
    weights = [(torch.randn(n, n) * n ** -0.5).to(torch.bfloat16).to(DEV) for _ in range(3)]
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device=DEV)
    schedules = [dict(tile_n=128, cta_group=2), dict(tile_n=64, cta_group=1, split_k=4),
                 dict(tile_n=64, cta_group=1, split_k=4, cluster_split=1), dict(tile_n=128, cta_group=1, split_tail=2)]
    stream = torch.cuda.current_stream().cuda_stream

    def chain():
        bufs = [x0, torch.zeros_like(x0), torch.zeros_like(x0)]
        cur = 0
        for step in range(24):
            src, dst = bufs[cur], bufs[1 + (step % 2)]
            cfg = _lib.Config.from_dict(schedules[step % len(schedules)])
            _lib.gemm("mm", "bfloat16", 0, src.data_ptr(), weights[step % 3].data_ptr(), dst.data_ptr(),
                      1, 256, n, n, cfg, ws.data_ptr(), ws.numel(), 0, stream)
            cur = 1 + (step % 2)
        torch.cuda.synchronize()
        return bufs[cur].clone()

    try:
        _lib.set_launch_overlap(False)
        plain = chain()
        _lib.set_launch_overlap(True)
        overlapped = chain()
        out_buf = torch.zeros_like(x0)
        mid = torch.zeros_like(x0)
        cfg = _lib.Config.from_dict(schedules[0])
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            cap = torch.cuda.current_stream().cuda_stream
            _lib.gemm("mm", "bfloat16", 0, x0.data_ptr(), weights[0].data_ptr(), mid.data_ptr(), 1, 256, n, n,
                      cfg, 0, 0, 0, cap)
            _lib.gemm("mm", "bfloat16", 0, mid.data_ptr(), weights[1].data_ptr(), out_buf.data_ptr(), 1, 256, n, n,
                      cfg, 0, 0, 0, cap)
        graph.replay()
        torch.cuda.synchronize()
    finally:
        _lib.set_launch_overlap(True)
    assert torch.equal(plain, overlapped)
    assert torch.isfinite(plain.float()).all()
    expect_mid = O.gemm_ref32("mm", x0.cpu(), weights[0].cpu()).to(torch.bfloat16)
    expect = O.gemm_ref32("mm", expect_mid, weights[1].cpu())
    assert_parity(out_buf.cpu(), expect, "two dependent launches in a graph")


@pytest.mark.parametrize("activation", ["relu", "sigmoid", "silu", "gelu", "gelu_tanh"])
def test_fused_activation_epilogue(activation, device_state):
    """act([bias +] a @ bt.T) through every kind of epilogue: bulk-store, transposed, workspace
    split-K, cluster split-K (bulk-store, lone-chunk and narrow-slice forms)."""
    torch.manual_seed(len(activation))
    status, workspace = device_state
    schedules = [dict(tile_n=256, cta_group=2), dict(tile_n=128, cta_group=1, split_k=2),
                 dict(tile_n=128, cta_group=1, split_k=2, cluster_split=1),
                 dict(tile_n=128, cta_group=1, split_k=4, cluster_split=1),
                 dict(tile_n=64, cta_group=2, split_k=2, cluster_split=1),
                 dict(tile_n=16, cta_group=1, swap_ab=1, group_m=1),
                 dict(tile_n=32, cta_group=1, swap_ab=1, group_m=1, split_k=4, cluster_split=1),
                 dict(tile_n=128, cta_group=1, swap_ab=1, group_m=1, split_k=2, cluster_split=1),
                 dict(tile_n=64, cta_group=1, swap_ab=1, group_m=1, split_k=3)]
    for cfg in schedules:
        small = bool(cfg.get("swap_ab"))
        for operation, dtype, batch, m, n, k in (("mm", "bfloat16", 1, 24 if small else 300, 520, 1024),
                                                 ("addmm", "float16", 1, 16 if small else 256, 264, 512),
                                                 ("bmm", "bfloat16", 2, 8 if small else 200, 136, 512)):
            config = _lib.Config.from_dict(cfg)
            assert _lib.config_valid(config, operation, dtype, batch, m, n, k), cfg
            lead = (batch,) if operation == "bmm" else ()
            a = torch.randn((*lead, m, k)).to(TD[dtype])
            bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
            tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
            dev = [t.to(DEV) for t in tensors]
            out = torch.full((*lead, m, n), float("nan"), dtype=TD[dtype], device=DEV)
            status.zero_()
            _lib.gemm_act(operation, dtype, activation, dev[0].data_ptr() if operation == "addmm" else 0,
                          dev[-2].data_ptr(), dev[-1].data_ptr(), out.data_ptr(), batch, m, n, k, config,
                          workspace.data_ptr(), workspace.numel(), status.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            want = O.act_ref32(activation, O.gemm_ref32(operation, *tensors))
            assert_parity(out.cpu(), want, f"{activation} {operation} {batch}x{m}x{n}x{k} {cfg}")


@pytest.mark.parametrize("activation", ["none", "sigmoid", "silu"])
def test_gated_activation_epilogue(activation, device_state):
    """act([bias +] a @ bt.T) * mul through the bulk-store, transposed, workspace split-K and cluster
    split-K epilogues (ragged shapes: the gate is read only where `out` is written)."""
    torch.manual_seed(3 + len(activation))
    status, workspace = device_state
    schedules = [dict(tile_n=256, cta_group=2), dict(tile_n=128, cta_group=1, split_k=2),
                 dict(tile_n=128, cta_group=1, split_k=2, cluster_split=1),
                 dict(tile_n=128, cta_group=1, split_k=4, cluster_split=1),
                 dict(tile_n=64, cta_group=2, split_k=2, cluster_split=1),
                 dict(tile_n=16, cta_group=1, swap_ab=1, group_m=1),
                 dict(tile_n=32, cta_group=1, swap_ab=1, group_m=1, split_k=4, cluster_split=1),
                 dict(tile_n=64, cta_group=1, swap_ab=1, group_m=1, split_k=3)]
    for cfg in schedules:
        small = bool(cfg.get("swap_ab"))
        for operation, dtype, batch, m, n, k in (("mm", "bfloat16", 1, 24 if small else 300, 520, 1024),
                                                 ("addmm", "float16", 1, 16 if small else 256, 264, 512),
                                                 ("bmm", "bfloat16", 2, 8 if small else 200, 136, 512)):
            config = _lib.Config.from_dict(cfg)
            lead = (batch,) if operation == "bmm" else ()
            a = torch.randn((*lead, m, k)).to(TD[dtype])
            bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
            mul = torch.randn((*lead, m, n)).to(TD[dtype])
            tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
            dev = [t.to(DEV) for t in tensors]
            out = torch.full((*lead, m, n), float("nan"), dtype=TD[dtype], device=DEV)
            status.zero_()
            _lib.gemm_act_mul(operation, dtype, activation, dev[0].data_ptr() if operation == "addmm" else 0,
                              dev[-2].data_ptr(), dev[-1].data_ptr(), mul.to(DEV).data_ptr(), out.data_ptr(),
                              batch, m, n, k, config, workspace.data_ptr(), workspace.numel(), status.data_ptr(),
                              torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            want = O.act_ref32(activation, O.gemm_ref32(operation, *tensors)) * mul.float()
            assert_parity(out.cpu(), want, f"{activation}*mul {operation} {batch}x{m}x{n}x{k} {cfg}")


def test_row_factor_epilogue(device_state):
    """act([bias +] a @ bt.T) * row_mul[:, None] through the bulk-store, transposed, workspace split-K
    and cluster split-K epilogues."""
    torch.manual_seed(77)
    status, workspace = device_state
    schedules = [dict(tile_n=256, cta_group=2), dict(tile_n=192, cta_group=1), dict(tile_n=128, cta_group=1, split_k=2),
                 dict(tile_n=128, cta_group=1, split_k=2, cluster_split=1),
                 dict(tile_n=128, cta_group=1, split_k=4, cluster_split=1),
                 dict(tile_n=64, cta_group=2, split_k=2, cluster_split=1),
                 dict(tile_n=16, cta_group=1, swap_ab=1, group_m=1),
                 dict(tile_n=32, cta_group=1, swap_ab=1, group_m=1, split_k=4, cluster_split=1),
                 dict(tile_n=128, cta_group=1, swap_ab=1, group_m=1, split_k=2, cluster_split=1),
                 dict(tile_n=64, cta_group=1, swap_ab=1, group_m=1, split_k=3)]
    for cfg in schedules:
        small = bool(cfg.get("swap_ab"))
        for operation, dtype, activation, batch, m, n, k in (
                ("mm", "bfloat16", "none", 1, 24 if small else 300, 520, 1024),
                ("addmm", "float16", "relu", 1, 16 if small else 256, 264, 512),
                ("bmm", "bfloat16", "silu", 3, 8 if small else 200, 136, 512)):
            config = _lib.Config.from_dict(cfg)
            lead = (batch,) if operation == "bmm" else ()
            a = torch.randn((*lead, m, k)).to(TD[dtype])
            bt = (torch.randn((*lead, n, k)) * k ** -0.5).to(TD[dtype])
            row_mul = (torch.rand((*lead, m, 1)) + 0.5).to(TD[dtype])
            tensors = (a, bt) if operation != "addmm" else (torch.randn(n).to(TD[dtype]), a, bt)
            dev = [t.to(DEV) for t in tensors]
            out = torch.full((*lead, m, n), float("nan"), dtype=TD[dtype], device=DEV)
            status.zero_()
            _lib.gemm_act_rowmul(operation, dtype, activation, dev[0].data_ptr() if operation == "addmm" else 0,
                                 dev[-2].data_ptr(), dev[-1].data_ptr(), row_mul.to(DEV).data_ptr(), out.data_ptr(),
                                 batch, m, n, k, config, workspace.data_ptr(), workspace.numel(), status.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            want = O.act_ref32(activation, O.gemm_ref32(operation, *tensors)) * row_mul.float()
            assert_parity(out.cpu(), want, f"{activation}*row {operation} {batch}x{m}x{n}x{k} {cfg}")


def test_rms_norm_linear_matches_the_unfused_form():
    """One row reduction + one GEMM against normalise-then-project in fp32 on the CPU, on a decode and
    a prefill token count, through whichever schedules selection gives them."""
    from ayla_b200 import gemm_act_rowmul_op
    from ayla_b200.rmsnorm_linear import fold_norm_weight, rms_norm_linear

    torch.manual_seed(5)
    assert gemm_act_rowmul_op("mm", "none", "bfloat16") is torch.ops.ayla.jit_mm_rowmul_bf16.default
    hidden, features = 1024, 1536
    g = (1.0 + 0.1 * torch.randn(hidden)).to(torch.bfloat16)
    w = (torch.randn(features, hidden) * hidden ** -0.5).to(torch.bfloat16)
    folded = fold_norm_weight(w.to(DEV), g.to(DEV))
    for tokens in (8, 300):
        x = (torch.randn(tokens, hidden) * 3.0).to(torch.bfloat16)
        got = rms_norm_linear(x.to(DEV), folded, eps=1e-5)
        x32 = x.float()
        normed = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()
        want = normed @ w.float().T
        rel = float((got.cpu().float() - want).norm() / want.norm())
        # Three roundings separate the two forms (folded weight, row factor, output): each at most 2^-9.
        assert rel < 6e-3, (tokens, rel)
    with pytest.raises(ValueError, match="row factors must be"):
        gemm_act_rowmul_op("mm", "none", "bfloat16")(x.to(DEV), folded, torch.ones(300, device=DEV, dtype=torch.bfloat16)
                                                     .view(1, 300), torch.empty(300, features, device=DEV,
                                                                                dtype=torch.bfloat16))


def test_gemm_act_mul_op_matches_the_oracle():
    from ayla_b200 import gemm_act_mul_op

    torch.manual_seed(12)
    a = torch.randn(192, 320).to(torch.bfloat16)
    bt = (torch.randn(264, 320) * 320 ** -0.5).to(torch.bfloat16)
    mul = torch.randn(192, 264).to(torch.bfloat16)
    out = torch.empty(192, 264, dtype=torch.bfloat16, device=DEV)
    op = gemm_act_mul_op("mm", "sigmoid", "bfloat16")
    assert op is torch.ops.ayla.jit_mm_sigmoid_mul_bf16.default
    assert op(a.to(DEV), bt.to(DEV), mul.to(DEV), out) is None
    assert_parity(out.cpu(), torch.sigmoid(O.mm_ref32(a, bt)) * mul.float(), "jit_mm_sigmoid_mul_bf16")
    with pytest.raises(ValueError, match="mul must have the shape of out"):
        op(a.to(DEV), bt.to(DEV), mul[:100].contiguous().to(DEV), out)


def test_gemm_act_op_matches_the_oracle():
    from ayla_b200.gemm_jit import gemm_act_op

    torch.manual_seed(11)
    a = torch.randn(192, 320).to(torch.bfloat16)
    bt = (torch.randn(264, 320) * 320 ** -0.5).to(torch.bfloat16)
    bias = torch.randn(264).to(torch.bfloat16)
    out = torch.empty(192, 264, dtype=torch.bfloat16, device=DEV)
    op = gemm_act_op("addmm", "gelu", "bfloat16")
    assert op is gemm_act_op("addmm", "gelu", "bfloat16")
    assert op is torch.ops.ayla.jit_addmm_gelu_bf16.default
    assert gemm_act_op("mm", "none", "bfloat16") is gemm_op("mm", "bfloat16")
    assert op(bias.to(DEV), a.to(DEV), bt.to(DEV), out) is None
    assert_parity(out.cpu(), O.act_ref32("gelu", O.addmm_ref32(bias, a, bt)), "jit_addmm_gelu_bf16")


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_swiglu_variants(cta_group, dtype, device_state):
    torch.manual_seed(cta_group)
    for m, n, k in ((128, 128, 64), (200, 264, 192), (1, 8, 8), (1024, 2048, 1024), (520, 136, 72)):
        x = torch.randn(m, k).to(TD[dtype])
        wg = (torch.randn(n, k) * k ** -0.5).to(TD[dtype])
        wu = (torch.randn(n, k) * k ** -0.5).to(TD[dtype])
        out, status = run_abi("swiglu", dtype, (x, wg, wu), dict(cta_group=cta_group, group_m=2), device_state)
        assert status == 0
        assert_parity(out, O.swiglu_ref32(x, wg, wu), f"swiglu {m}x{n}x{k} cta_group={cta_group}")


# ------------------------------------------------------------- exactness properties

def test_identity_and_power_of_two_scaling_are_exact(device_state):
    torch.manual_seed(5)
    for dtype in ("bfloat16", "float16"):
        td = TD[dtype]
        a = torch.randn(300, 256).to(td)
        eye = torch.eye(256).to(td)
        for cfg in (dict(tile_n=256, cta_group=2), dict(tile_n=64, cta_group=1, split_k=2), None):
            out, _ = run_abi("mm", dtype, (a, eye), cfg, device_state)
            assert torch.equal(out.cpu(), a), cfg                      # a @ I^T == a, bit for bit
        bt = torch.randn(264, 256).to(td)
        base, _ = run_abi("mm", dtype, (a, bt), None, device_state)
        scaled, _ = run_abi("mm", dtype, ((a.float() * 4).to(td), (bt.float() * 0.5).to(td)), None, device_state)
        assert torch.equal(scaled.float().cpu(), base.float().cpu() * 2)  # exact in binary floating point


def test_small_k_results_are_bit_exact(device_state):
    """For K <= 128 every partial sum of 16-bit products fits fp32 exactly often enough
    that the reference pins bit-equality with torch.mm
    (tests/gemm_collection/test_correctness.py:216-234, :302-314); same here against the
    CPU oracle, allowing last-bit flips on at most 0.1 % of elements."""
    for m, n, k, seed in ((128, 256, 128, 7), (3, 256, 64, 3), (128, 256, 64, 128), (256, 256, 64, 256)):
        g = torch.Generator().manual_seed(seed)
        a = torch.randn(m, k, generator=g).bfloat16()
        bt = torch.randn(n, k, generator=g).bfloat16()
        out, _ = run_abi("mm", "bfloat16", (a, bt), None, device_state)
        want = O.gemm_ref("mm", torch.bfloat16, a, bt)
        differing = int((out.cpu().view(torch.int16) != want.view(torch.int16)).sum())
        assert differing <= max(1, out.numel() // 1000), (m, n, k, differing)


def test_repeated_launches_are_deterministic(device_state):
    """Split-K partials are reduced in a fixed order, so results do not depend on
    which CTA finishes last."""
    op, tensors = O.make_inputs("C2b", "bfloat16", scale_down=4)
    cfg = dict(tile_n=64, cta_group=1, split_k=8)
    first, _ = run_abi(op, "bfloat16", tensors, cfg, device_state)
    for _ in range(5):
        again, status = run_abi(op, "bfloat16", tensors, cfg, device_state)
        assert status == 0 and torch.equal(first, again)


# ------------------------------------------------------------ the benchmark configs

def run_op(operation, dtype, tensors):
    dev = [t.to(DEV) for t in tensors]
    if operation == "swiglu":
        out = torch.empty((dev[0].shape[0], dev[1].shape[0]), dtype=dev[0].dtype, device=DEV)
        swiglu_op(dtype)(*dev, out)
        compiler = swiglu_op_compiler(dtype)
    else:
        a, bt = dev[-2:]
        out = torch.empty((*a.shape[:-1], bt.shape[-2]), dtype=a.dtype, device=DEV)
        gemm_op(operation, dtype)(*dev, out)
        compiler = gemm_op_compiler(operation, dtype)
    torch.cuda.synchronize()
    for launcher in compiler._cache.values():
        launcher.check_status()
    return out


@pytest.mark.parametrize("config,dtype", [("C1", "bfloat16"), ("C2a", "bfloat16"), ("C2a", "float16"),
                                          ("C2b", "bfloat16"), ("C2b", "float16"), ("C3a", "bfloat16"),
                                          ("C3b", "bfloat16"), ("C4", "bfloat16")])
def test_benchmark_configs_full_size(config, dtype):
    operation, tensors = O.make_inputs(config, dtype)
    out = run_op(operation, dtype, tensors)
    parity = assert_parity(out, O.gemm_ref32(operation, *tensors), config)
    print(f"\n{config} {dtype}: {parity}")


@pytest.mark.parametrize("index", range(len(O.SWEEP_M) * len(O.SWEEP_NK)))
def test_dynamic_m_sweep(index):
    (m, n, k), (a, bt) = O.make_sweep_inputs(index)
    out = run_op("mm", "bfloat16", (a, bt))
    assert_parity(out, O.mm_ref32(a, bt), f"sweep m={m} n={n} k={k}")


def test_linearity_at_full_size():
    """out(a1 + a2) == out(a1) + out(a2) within rounding, at the 4096^3 size, with
    operands whose sums are exact in bf16 (small integers)."""
    g = torch.Generator().manual_seed(9)
    a1 = torch.randint(-3, 4, (4096, 4096), generator=g).bfloat16()
    a2 = torch.randint(-3, 4, (4096, 4096), generator=g).bfloat16()
    bt = torch.randint(-2, 3, (4096, 4096), generator=g).bfloat16()
    o1 = run_op("mm", "bfloat16", (a1, bt)).float()
    o2 = run_op("mm", "bfloat16", (a2, bt)).float()
    o12 = run_op("mm", "bfloat16", (a1 + a2, bt)).float()
    # integer sums below 2^24 are exact in the fp32 accumulator; only the final rounding differs
    exact = torch.mm((a1 + a2).float(), bt.float().t()).bfloat16().float()
    assert torch.equal(o12.cpu(), exact)
    assert ((o1 + o2) - o12).abs().max().item() <= 2 * float(O._ulp(o12.abs().max().cpu(), torch.bfloat16))


# ------------------------------------------------------------------ error behaviour

def test_op_level_validation():
    a = torch.randn(64, 64, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(64, 64, device=DEV, dtype=torch.bfloat16)
    op = gemm_op("mm", "bfloat16")
    with pytest.raises(ValueError, match="contiguous"):
        op(a.t(), a, out)
    with pytest.raises(ValueError, match="expected dtype"):
        op(a.half(), a, out)
    with pytest.raises(ValueError, match="CUDA tensors"):
        op(a.cpu(), a, out)
    with pytest.raises(ValueError, match="bt must be"):
        op(a, torch.empty(64, 32, device=DEV, dtype=torch.bfloat16), out)
    with pytest.raises(ValueError, match="out must be"):
        op(a, a, torch.empty(64, 32, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="no schedule"):
        op(torch.empty(8, 12, device=DEV, dtype=torch.bfloat16), torch.empty(8, 12, device=DEV, dtype=torch.bfloat16),
           torch.empty(8, 8, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="bias must be"):
        gemm_op("addmm", "bfloat16")(torch.empty(32, device=DEV, dtype=torch.bfloat16), a, a, out)


def test_abi_workspace_and_init_errors(device_state):
    status, workspace = device_state
    a = torch.randn(256, 1024, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(256, 256, device=DEV, dtype=torch.bfloat16)
    cfg = _lib.Config.from_dict(dict(tile_n=64, cta_group=1, split_k=4))
    with pytest.raises(ValueError, match="workspace"):
        _lib.gemm("mm", "bfloat16", 0, a.data_ptr(), a.data_ptr(), out.data_ptr(), 1, 256, 256, 1024, cfg,
                  workspace.data_ptr(), 1024, 0, torch.cuda.current_stream().cuda_stream)
    with pytest.raises(ValueError, match="workspace"):
        _lib.gemm("mm", "bfloat16", 0, a.data_ptr(), a.data_ptr(), out.data_ptr(), 1, 256, 256, 1024, cfg,
                  0, 0, 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()


@pytest.mark.parametrize("m", [3, 128, 256])
def test_dynamic_m_matmul(m):
    """tests/gemm_collection/test_correctness.py:302-314 of the reference: m in {3, 128, 256},
    n = 256, k = 64, seed = m; one cached schedule per shape."""
    from ayla_b200.dynamic_m import make_dynamic_m_matmul

    op = make_dynamic_m_matmul(256, 64, namespace=f"ayla_b200_dynamic_m_test_{m}")
    g = torch.Generator().manual_seed(m)
    lhs = torch.randn(m, 64, generator=g).bfloat16()
    rhs = torch.randn(256, 64, generator=g).bfloat16()
    out = op(lhs.to(DEV), rhs.to(DEV))
    assert out.shape == (m, 256)
    want = O.gemm_ref("mm", torch.bfloat16, lhs, rhs)
    differing = int((out.cpu().view(torch.int16) != want.view(torch.int16)).sum())
    assert differing <= max(1, out.numel() // 1000)


# ------------------------------------------------------- failure detection (no GPU fault)

@pytest.mark.parametrize("cfg", [dict(tile_n=128, cta_group=1), dict(tile_n=256, cta_group=2),
                                 dict(tile_n=16, cta_group=1, swap_ab=1, group_m=1)])
def test_bounded_wait_reports_a_stalled_pipeline_and_the_context_survives(cfg, device_state):
    """A launch whose producer never delivers operands must not hang: the MMA warp's wait
    runs out, the kernel finishes, the status word says which wait gave up (code 2 = waiting
    for operands), and the next ordinary launch on the same context is correct."""
    lib = _lib.load()
    g = torch.Generator().manual_seed(3)
    a = torch.randn(300, 264, generator=g).bfloat16()
    bt = torch.randn(264, 264, generator=g).bfloat16()
    try:
        lib.ayla_b200_set_wait_timeout_ms(30)
        lib.ayla_b200_debug_set_flags(1)
        _, status = run_abi("mm", "bfloat16", (a, bt), cfg, device_state)
        assert status & 0xFF in (2, 4), hex(status)   # the MMA wait (2) or, racing it, the epilogue's (4)
    finally:
        lib.ayla_b200_debug_set_flags(0)
        lib.ayla_b200_set_wait_timeout_ms(2000)
    device_state[1].zero_()
    out, status = run_abi("mm", "bfloat16", (a, bt), cfg, device_state)
    assert status == 0
    assert_parity(out, O.mm_ref32(a, bt), "launch after a timed-out one")


def test_launcher_check_status_raises_on_timeout():
    lib = _lib.load()
    compiler = gemm_jit_compiler("mm", "bfloat16")
    a = torch.randn(256, 256, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(256, 256, device=DEV, dtype=torch.bfloat16)
    compiler(a, a, out)
    [launcher] = compiler._cache.values()
    try:
        lib.ayla_b200_set_wait_timeout_ms(30)
        lib.ayla_b200_debug_set_flags(1)
        compiler(a, a, out)
        with pytest.raises(RuntimeError, match="timed out"):
            launcher.check_status()
    finally:
        lib.ayla_b200_debug_set_flags(0)
        lib.ayla_b200_set_wait_timeout_ms(2000)
    compiler(a, a, out)
    launcher.check_status()
    torch.testing.assert_close(out, a @ a.T, atol=0.125, rtol=0.02)


def test_timed_out_split_k_launch_is_reported_by_the_next_call_without_the_debug_switch(monkeypatch):
    """The status word sits in pinned host memory and is read before every launch: after a k-split
    launch that ran into a bounded wait, the next call of that shape raises (no AYLA_B200_DEBUG, no
    explicit check_status), and the call after it is correct -- the arrival counters a timed-out
    k-split may leave behind are cleared with the report."""
    from ayla_b200.gemm_jit import GemmLauncher, GemmScheduleSeed, _DEFAULTS

    monkeypatch.delenv("AYLA_B200_DEBUG", raising=False)
    lib = _lib.load()
    m, n, k = 256, 256, 2048
    captured = {**_DEFAULTS, "tile_n": 64, "cta_group": 1, "split_k": 4}
    seed = GemmScheduleSeed(captured, {key: int(captured[key]) for key in _lib.Config.FIELDS}, (), (m, n, k))
    launcher = GemmLauncher("mm", "bfloat16", 1, m, n, k, seed, torch.device(DEV))
    assert launcher.workspace is not None and not launcher._debug
    g = torch.Generator().manual_seed(11)
    a = torch.randn(m, k, generator=g).bfloat16()
    bt = (torch.randn(n, k, generator=g) * k ** -0.5).bfloat16()
    da, dbt = a.to(DEV), bt.to(DEV)
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    launcher(da, dbt, out)
    torch.cuda.synchronize()
    assert launcher.status.peek() == 0
    assert_parity(out, O.mm_ref32(a, bt), "k-split launch before the failure")
    try:
        lib.ayla_b200_set_wait_timeout_ms(30)
        lib.ayla_b200_debug_set_flags(1)
        launcher(da, dbt, out)          # the producer delivers nothing: the waits run out
        torch.cuda.synchronize()
    finally:
        lib.ayla_b200_debug_set_flags(0)
        lib.ayla_b200_set_wait_timeout_ms(2000)
    assert launcher.status.peek() & 0xFF in (2, 4)
    with pytest.raises(RuntimeError, match="timed out"):
        launcher(da, dbt, out)
    out.zero_()
    launcher(da, dbt, out)
    torch.cuda.synchronize()
    assert launcher.status.peek() == 0
    assert_parity(out, O.mm_ref32(a, bt), "k-split launch after a reported timeout")


def test_random_shapes_through_the_public_ops():
    """Schedule selection on shapes nobody measured: transferred table entries (trimmed tiles, 192-wide
    tiles, cluster k-splits, eviction hints) and the default heuristic must all stay correct on ragged
    extents.  Checked against the GPU's own fp32-accumulating matmul with the reference's test tolerances
    (tests/test_gemm_jit.py:59-63 of the reference)."""
    import random

    rng = random.Random(1234)
    torch.manual_seed(1234)
    picks_m = [1, 3, 8, 17, 33, 64, 100, 128, 200, 256, 384, 512, 777, 1024, 1536, 2048, 3000]
    picks_n = [8, 64, 136, 512, 1000, 2048, 4096, 6144, 7168, 8192, 11008, 14336]
    picks_k = [8, 72, 128, 520, 1024, 2048, 4096, 5120, 8192, 14336]
    for trial in range(120):
        operation = rng.choice(["mm", "mm", "addmm", "bmm"])
        m, n, k = rng.choice(picks_m), rng.choice(picks_n), rng.choice(picks_k)
        batch = rng.choice([2, 3, 5]) if operation == "bmm" else 1
        if batch * (m * k + n * k + m * n) > 160e6:
            k = min(k, 1024)
        dtype = rng.choice(["bfloat16", "float16"])
        td = TD[dtype]
        lead = (batch,) if operation == "bmm" else ()
        a = torch.randn((*lead, m, k), device=DEV).to(td)
        bt = (torch.randn((*lead, n, k), device=DEV) * k ** -0.5).to(td)
        out = torch.full((*lead, m, n), float("nan"), device=DEV, dtype=td)
        if operation == "addmm":
            bias = torch.randn(n, device=DEV).to(td)
            gemm_op(operation, dtype)(bias, a, bt, out)
            want = torch.addmm(bias.float(), a.float(), bt.float().T)
        else:
            gemm_op(operation, dtype)(a, bt, out)
            want = a.float() @ bt.float().transpose(-1, -2)
        torch.testing.assert_close(out.float(), want, atol=0.125, rtol=0.02,
                                   msg=lambda msg: f"{operation} {dtype} {batch}x{m}x{n}x{k}: {msg}")


def test_random_shapes_through_the_fused_ops():
    """SwiGLU, activation and gated epilogues on ragged shapes nobody measured, against fp32 math on
    the GPU rounded once (same tolerances as the plain ops)."""
    import random

    from ayla_b200 import ACTIVATIONS, gemm_act_mul_op, gemm_act_op

    rng = random.Random(4321)
    torch.manual_seed(4321)
    acts = {"relu": torch.relu, "sigmoid": torch.sigmoid, "silu": torch.nn.functional.silu,
            "gelu": torch.nn.functional.gelu,
            "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}
    assert set(acts) == set(ACTIVATIONS) - {"none"}
    for trial in range(60):
        m = rng.choice([1, 8, 24, 64, 130, 256, 512, 1000, 2048])
        n = rng.choice([8, 72, 512, 1000, 4096, 6144, 14336])
        k = rng.choice([8, 136, 1024, 4096, 5120])
        dtype = rng.choice(["bfloat16", "float16"])
        td = TD[dtype]
        a = torch.randn(m, k, device=DEV).to(td)
        w0 = (torch.randn(n, k, device=DEV) * k ** -0.5).to(td)
        out = torch.full((m, n), float("nan"), device=DEV, dtype=td)
        kind = rng.choice(["swiglu", "act", "gated"])
        if kind == "swiglu":
            w1 = (torch.randn(n, k, device=DEV) * k ** -0.5).to(td)
            swiglu_op(dtype)(a, w0, w1, out)
            want = torch.nn.functional.silu(a.float() @ w0.float().T) * (a.float() @ w1.float().T)
            label = "swiglu"
        else:
            act = rng.choice(sorted(acts))
            with_bias = rng.random() < 0.5
            bias = torch.randn(n, device=DEV).to(td)
            want = a.float() @ w0.float().T
            if with_bias:
                want = want + bias.float()
            want = acts[act](want)
            operation = "addmm" if with_bias else "mm"
            lead = (bias,) if with_bias else ()
            if kind == "act":
                gemm_act_op(operation, act, dtype)(*lead, a, w0, out)
            else:
                mul = torch.randn(m, n, device=DEV).to(td)
                gemm_act_mul_op(operation, act, dtype)(*lead, a, w0, mul, out)
                want = want * mul.float()
            label = f"{kind} {operation} {act}"
        torch.testing.assert_close(out.float(), want, atol=0.125, rtol=0.02,
                                   msg=lambda msg: f"{label} {dtype} {m}x{n}x{k}: {msg}")
