"""The allocation-free entry point, ``ayla_b200_gemm_static_scratch``.

Some hosts of this library cannot hand it a workspace and must not let it allocate one:
plugins that live under another runtime's memory pool (a stray cudaMalloc stalls the
device and escapes the pool's books) or glue that only sees one op's operand pointers.
For them the split-K scratch is an 8 MiB array inside the library.  This test calls that
entry point through the C ABI with split-K schedules, twice in a row (the second call
meets whatever the first left in the shared array), and requires the result to be
bit-identical to the ordinary entry point with a caller workspace -- the reduction order
is fixed, so nothing weaker than equality is needed.  Collected last on purpose.
"""

import pytest
import torch

from ayla_b200 import _lib

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _both(op, dtype, tensors, cfg_dict, repeats=2):
    _lib.init(0)
    td = torch.bfloat16 if dtype == "bfloat16" else torch.float16
    dev = [t.to(DEV) for t in tensors]
    bias = dev[0] if op == "addmm" else None
    a, bt = dev[-2:]
    batch = a.shape[0] if op == "bmm" else 1
    m, k = a.shape[-2:]
    n = bt.shape[-2]
    cfg = _lib.Config.from_dict(cfg_dict)
    need = _lib.workspace_bytes(cfg, op, batch, m, n, k)
    assert 0 < need <= _lib.STATIC_SCRATCH_BYTES
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    workspace = torch.zeros(need, dtype=torch.uint8, device=DEV)
    want = torch.full((*a.shape[:-1], n), float("nan"), dtype=td, device=DEV)
    _lib.gemm(op, dtype, bias.data_ptr() if bias is not None else 0, a.data_ptr(), bt.data_ptr(),
              want.data_ptr(), batch, m, n, k, cfg, workspace.data_ptr(), need, status.data_ptr(), stream)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and not torch.isnan(want).any()
    for _ in range(repeats):
        got = torch.full_like(want, float("nan"))
        free_before = torch.cuda.mem_get_info()[0]
        _lib.gemm_static_scratch(op, dtype, bias.data_ptr() if bias is not None else 0, a.data_ptr(),
                                 bt.data_ptr(), got.data_ptr(), batch, m, n, k, cfg, status.data_ptr(), stream)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert int(status.item()) == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_static_scratch_matches_caller_workspace_on_consecutive_calls():
    g = torch.Generator().manual_seed(77)
    a = torch.randn(256, 4096, generator=g).bfloat16()
    bt = (torch.randn(1024, 4096, generator=g) * 4096 ** -0.5).bfloat16()
    bias = torch.randn(1024, generator=g).bfloat16()
    # row-major split-K, then a different shape and schedule reusing the same array
    _both("addmm", "bfloat16", (bias, a, bt), dict(tile_n=64, cta_group=1, split_k=4))
    _both("mm", "bfloat16", (a[:200], bt[:520]), dict(tile_n=128, cta_group=2, split_k=3))
    # swapped small-M form
    _both("mm", "float16", (a[:8].half(), bt.half()), dict(tile_n=16, cta_group=1, swap_ab=1, split_k=8, group_m=1))
    _both("bmm", "bfloat16", (a[:192].reshape(3, 64, 4096), bt[:384].reshape(3, 128, 4096)),
          dict(tile_n=64, cta_group=1, split_k=2))


def test_static_scratch_without_split_k_needs_no_scratch():
    _lib.init(0)
    a = torch.randn(300, 264, device=DEV).bfloat16()
    bt = torch.randn(304, 264, device=DEV).bfloat16()
    out = torch.empty(300, 304, device=DEV, dtype=torch.bfloat16)
    want = torch.empty_like(out)
    cfg = _lib.Config.from_dict(dict(tile_n=128, cta_group=1))
    stream = torch.cuda.current_stream().cuda_stream
    _lib.gemm("mm", "bfloat16", 0, a.data_ptr(), bt.data_ptr(), want.data_ptr(), 1, 300, 304, 264, cfg, 0, 0, 0, stream)
    _lib.gemm_static_scratch("mm", "bfloat16", 0, a.data_ptr(), bt.data_ptr(), out.data_ptr(), 1, 300, 304, 264, cfg, 0, stream)
    torch.cuda.synchronize()
    assert torch.equal(out, want)


def test_static_scratch_rejects_oversized_requests():
    _lib.init(0)
    a = torch.empty(4096, 8192, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(4096, 4096, device=DEV, dtype=torch.bfloat16)
    cfg = _lib.Config.from_dict(dict(tile_n=256, cta_group=1, split_k=4))
    assert _lib.workspace_bytes(cfg, "mm", 1, 4096, 4096, 8192) > _lib.STATIC_SCRATCH_BYTES
    with pytest.raises(ValueError, match="built-in array holds"):
        _lib.gemm_static_scratch("mm", "bfloat16", 0, a.data_ptr(), a.data_ptr(), out.data_ptr(), 1, 4096, 4096,
                                 8192, cfg, 0, torch.cuda.current_stream().cuda_stream)
