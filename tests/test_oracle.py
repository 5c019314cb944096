"""The CPU oracle against the committed golden vectors, and the C restatement
against the oracle.  Runs without a GPU."""

import pytest
import torch

from oracle import gemm_oracle as O
from oracle.c_oracle import gemm_c
from tests.conftest import load_golden_cases

CASES = load_golden_cases()


@pytest.mark.parametrize("case", CASES, ids=repr)
def test_oracle_reproduces_golden_vectors_bit_exactly(case):
    got = O.gemm_ref(case.operation, case.torch_dtype, *case.operands())
    assert got.shape == case.expected().shape
    assert torch.equal(got.view(torch.int16), case.expected().view(torch.int16))


@pytest.mark.parametrize("case", [c for c in CASES if c.m * c.n * c.k * c.batch <= 96 * 256 * 128 * 2], ids=repr)
def test_c_restatement_agrees_with_golden_up_to_rounding_flips(case):
    """The C oracle accumulates in fp64, the golden vectors in fp32: they may differ
    only by a flip of the final rounding, never by more than one output ulp."""
    got = gemm_c(case.operation, *case.operands())
    want = case.expected()
    parity = O.compare(got, want.float())
    differing = int((got.view(torch.int16) != want.view(torch.int16)).sum())
    assert parity.nonfinite == 0
    assert differing <= max(2, got.numel() // 500), differing
    # One output ulp, except where cancellation leaves a result far below the
    # operands' scale: there fp32 summation error dominates the (tiny) ulp.
    rms = float(want.float().pow(2).mean().sqrt())
    ulp = O._ulp(want.float().abs().clamp_min(1e-2 * rms), case.torch_dtype)
    assert bool(((got.float() - want.float()).abs() <= ulp * 1.0001).all())
    assert parity.ok


@pytest.mark.parametrize("operation, dtype, m, n, k, a_scale, b_scale", [
    ("mm", torch.bfloat16, 64, 256, 4096, 1.0, 4096 ** -0.5),      # a long accumulation, sweep-like operands
    ("addmm", torch.float16, 32, 128, 16384, 1.0, 16384 ** -0.5),  # the split-K config's depth, scaled down in M and N
    ("mm", torch.bfloat16, 48, 64, 8192, 1.0, 1.0),                # unscaled operands: results far from 1
])
def test_deep_k_torch_oracle_against_the_independent_c_restatement(operation, dtype, m, n, k, a_scale, b_scale):
    """Something that is not torch checks torch on long accumulations: the fp64 plain-C
    restatement and the fp32 torch oracle may differ only by flips of the final rounding
    (one output ulp), and the C result must satisfy the project's tolerance against torch's."""
    g = torch.Generator().manual_seed(k + m)
    a = (torch.randn(m, k, generator=g) * a_scale).to(dtype)
    bt = (torch.randn(n, k, generator=g) * b_scale).to(dtype)
    bias = (torch.randn(n, generator=g) * 0.1).to(dtype)
    operands = (bias, a, bt) if operation == "addmm" else (a, bt)
    want32 = O.addmm_ref32(*operands) if operation == "addmm" else O.mm_ref32(*operands)
    want = want32.to(dtype)
    got = gemm_c(operation, *operands)
    parity = O.compare(got, want32)
    assert parity.ok and parity.nonfinite == 0, parity
    differing = int((got.view(torch.int16) != want.view(torch.int16)).sum())
    assert differing <= max(2, got.numel() // 100), differing
    rms = float(want32.pow(2).mean().sqrt())
    ulp = O._ulp(want32.abs().clamp_min(1e-2 * rms), dtype)
    assert bool(((got.float() - want.float()).abs() <= ulp * 1.0001).all())


def test_c_restatement_known_answers():
    """Identity and one-hot operands give exactly representable results."""
    for dtype in (torch.bfloat16, torch.float16):
        eye = torch.eye(16, dtype=dtype)
        a = torch.arange(16 * 16, dtype=torch.float32).reshape(16, 16).to(dtype)
        assert torch.equal(gemm_c("mm", a, eye), a)          # a @ I^T
        assert torch.equal(gemm_c("mm", eye, a), a.t().contiguous())  # I @ a^T
        bias = torch.arange(16, dtype=torch.float32).to(dtype)
        assert torch.equal(gemm_c("addmm", bias, a, eye), (a.float() + bias.float()).to(dtype))
    # 0.5 + 2^-9 is a tie between two bf16 neighbours: round to even.
    a = torch.tensor([[1.0, 2.0 ** -8]], dtype=torch.bfloat16)
    b = torch.tensor([[0.5, 0.5]], dtype=torch.bfloat16)
    out = gemm_c("mm", torch.cat([a, torch.zeros(1, 6, dtype=torch.bfloat16)], 1),
                 torch.cat([b, torch.zeros(1, 6, dtype=torch.bfloat16)], 1))
    assert out.item() == 0.5


def test_fp16_conversions_of_c_restatement_are_exhaustively_exact():
    """Every finite fp16 value survives x*1 through the C oracle (decode + RNE encode)."""
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16)
    vals = bits.view(torch.float16)
    finite = torch.isfinite(vals)
    v = vals[finite]
    pad = (-v.numel()) % 8
    v = torch.cat([v, torch.zeros(pad, dtype=torch.float16)])
    # out[i, 0] = v[i] * 1 with k padded to 8
    a = torch.zeros(v.numel(), 8, dtype=torch.float16)
    a[:, 0] = v
    bt = torch.zeros(8, 8, dtype=torch.float16)
    bt[0, 0] = 1.0
    out = gemm_c("mm", a, bt)[:, 0]
    assert torch.equal(out.view(torch.int16)[v != 0], v.view(torch.int16)[v != 0])


def test_compare_reports_rounding_flips_separately():
    ref32 = torch.full((64, 64), 300.0)
    ref32[0, 0] = 257.0  # rounds to 256 (ulp 2); 258 is the next bf16 value
    out = ref32.to(torch.bfloat16).clone()
    out[0, 0] = 258.0
    parity = O.compare(out, ref32)
    assert parity.over_bound == 0 or parity.over_bound == parity.over_bound_one_ulp
    assert parity.ok
    out[1, 1] = 400.0
    assert not O.compare(out, ref32).ok


def test_seeded_inputs_are_reproducible_and_scaled():
    op, (bias, a, bt) = O.make_inputs("C2a", "float16", scale_down=64)
    op2, again = O.make_inputs("C2a", "float16", scale_down=64)
    assert op == op2 == "addmm" and all(torch.equal(x, y) for x, y in zip((bias, a, bt), again))
    assert a.shape == (128, 768) and bt.shape == (768, 768) and bias.shape == (768,)
    assert abs(bt.float().std().item() - 768 ** -0.5) < 2e-3
    op, (x, wg, wu) = O.make_inputs("C4", scale_down=64)
    assert op == "swiglu" and abs(wg.float().std().item() - 0.02) < 1e-3
    (m, n, k), (a, bt) = O.make_sweep_inputs(0)
    assert (m, n, k) == (1, 4096, 4096) and a.shape == (1, 4096)
