"""Generate the committed fixtures under tests/golden/.

Run from the repository root in a container that holds the reference checkout:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/ayla

Two files are written:

* ``gemm_vectors.npz`` -- small seeded operands (16-bit patterns) and the
  reference result for mm / addmm / bmm / swiglu in fp16 and bf16.  The reference
  result is what the reference's own tests compare against
  (tests/gemm_collection/test_correctness.py:419, tests/test_gemm_jit.py:59-63):
  PyTorch's fp32 matmul of the up-cast operands on CPU, rounded once to the output
  type.  It is computed here with plain ``torch`` calls, NOT through the oracle
  module, so the oracle can be checked against it.
* ``reference_api.json`` -- behaviour of the reference's schedule/dispatch API
  recorded by importing it (``ayla.gemm_jit``, ``ayla.jit_compiler``,
  ``ayla.torch_custom_call``): which shapes ``select_gemm_schedule`` declines, the
  op schemas ``gemm_op`` registers, and the validation messages of the dispatch
  cache.  Skipped (file left untouched) when the reference is not present.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent

# (name, operation, dtype, batch, m, n, k, seed); shapes follow the reference's GPU
# tests: (96,128,128) and (256,256,256) (tests/test_gemm_jit.py:51), 128x256x128 seed 7
# (tests/gemm_collection/test_correctness.py:216-234), dynamic-M m in {3,128,256},
# n=256, k=64, seed=m (:302-314), plus ragged shapes with n % 8 == 0, k % 8 == 0.
CASES = [
    ("mm_bf16_96x128x128", "mm", "bfloat16", 1, 96, 128, 128, 11),
    ("mm_f16_96x128x128", "mm", "float16", 1, 96, 128, 128, 12),
    ("mm_bf16_256x256x256", "mm", "bfloat16", 1, 256, 256, 256, 13),
    ("mm_bf16_128x256x128_seed7", "mm", "bfloat16", 1, 128, 256, 128, 7),
    ("mm_bf16_dynm3", "mm", "bfloat16", 1, 3, 256, 64, 3),
    ("mm_bf16_dynm128", "mm", "bfloat16", 1, 128, 256, 64, 128),
    ("mm_bf16_dynm256", "mm", "bfloat16", 1, 256, 256, 64, 256),
    ("mm_f16_ragged_77x72x40", "mm", "float16", 1, 77, 72, 40, 14),
    ("mm_bf16_m1_256x512", "mm", "bfloat16", 1, 1, 256, 512, 15),
    ("addmm_bf16_96x128x128", "addmm", "bfloat16", 1, 96, 128, 128, 21),
    ("addmm_f16_64x136x256", "addmm", "float16", 1, 64, 136, 256, 22),
    ("addmm_bf16_splitk_64x128x1024", "addmm", "bfloat16", 1, 64, 128, 1024, 23),
    ("bmm_bf16_2x96x128x64", "bmm", "bfloat16", 2, 96, 128, 64, 31),
    ("bmm_f16_2x64x72x256", "bmm", "float16", 2, 64, 72, 256, 32),
    ("bmm_bf16_3x70x72x72", "bmm", "bfloat16", 3, 70, 72, 72, 33),
    ("swiglu_bf16_96x128x128", "swiglu", "bfloat16", 1, 96, 128, 128, 41),
    ("swiglu_bf16_72x136x192", "swiglu", "bfloat16", 1, 72, 136, 192, 42),
    ("swiglu_f16_64x128x128", "swiglu", "float16", 1, 64, 128, 128, 43),
]

TD = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def make_vectors() -> None:
    arrays: dict[str, np.ndarray] = {}
    meta = []
    for name, op, dtype, batch, m, n, k, seed in CASES:
        g = torch.Generator(device="cpu")
        g.manual_seed(seed)
        td = TD[dtype]
        lead = (batch,) if op == "bmm" else ()
        a = torch.randn((*lead, m, k), generator=g).to(td)
        scale = k ** -0.5 if op == "swiglu" else 1.0
        bt = (torch.randn((*lead, n, k), generator=g) * scale).to(td)
        arrays[f"{name}/a"] = bits(a)
        arrays[f"{name}/bt"] = bits(bt)
        if op == "mm":
            ref32 = torch.mm(a.float(), bt.float().t())
        elif op == "addmm":
            bias = torch.randn((n,), generator=g).to(td)
            arrays[f"{name}/bias"] = bits(bias)
            ref32 = torch.addmm(bias.float(), a.float(), bt.float().t())
        elif op == "bmm":
            ref32 = torch.bmm(a.float(), bt.float().transpose(1, 2))
        else:
            wu = (torch.randn((n, k), generator=g) * scale).to(td)
            arrays[f"{name}/wu"] = bits(wu)
            ref32 = F.silu(torch.mm(a.float(), bt.float().t())) * torch.mm(a.float(), wu.float().t())
        arrays[f"{name}/out"] = bits(ref32.to(td))
        meta.append(dict(name=name, operation=op, dtype=dtype, batch=batch, m=m, n=n, k=k, seed=seed))
    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "gemm_vectors.npz", **arrays)
    print(f"wrote {HERE / 'gemm_vectors.npz'} ({(HERE / 'gemm_vectors.npz').stat().st_size} bytes, torch {torch.__version__})")


def make_reference_api(reference: Path) -> None:
    if not (reference / "ayla" / "gemm_jit.py").exists():
        print(f"reference not found at {reference}; reference_api.json left untouched")
        return
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(reference))
    from ayla.gemm_jit import gemm_jit_compiler, gemm_op, measured_gemm_configs, select_gemm_schedule

    record: dict[str, object] = {"torch": torch.__version__}

    queries = [
        ("mm", "bfloat16", 0, 64, 64, 1),
        ("mm", "bfloat16", 64, 65, 64, 1),
        ("mm", "bfloat16", 64, 64, 32, 1),
        ("mm", "float32", 256, 256, 128, 1),
        ("mm", "bfloat16", 256, 256, 128, 1),
        ("mm", "bfloat16", 4096, 4096, 4096, 1),
        ("mm", "float16", 4096, 4096, 4096, 1),
        ("addmm", "bfloat16", 8192, 768, 768, 1),
        ("addmm", "float16", 8192, 768, 768, 1),
        ("bmm", "bfloat16", 2048, 2048, 128, 64),
        ("bmm", "bfloat16", 2048, 128, 2048, 64),
        ("bmm", "bfloat16", 96, 128, 128, 2),
        ("mm", "bfloat16", 96, 128, 128, 1),
        ("mm", "bfloat16", 3, 256, 64, 1),
        ("gemv", "bfloat16", 64, 64, 64, 1),
        ("mm", "bfloat16", 64, 64, 64, 0),
        ("mm", "bfloat16", 64, 64, -64, 1),
    ]
    selections = []
    for op, dtype, m, n, k, batch in queries:
        seed = select_gemm_schedule(op, dtype, m, n, k, batch)
        selections.append(
            dict(operation=op, dtype=dtype, m=m, n=n, k=k, batch=batch, selected=seed is not None,
                 exact=(seed is not None and seed.adaptations == ()),
                 has_source_shape=(seed is not None and seed.source_shape is not None))
        )
    record["select_gemm_schedule"] = selections

    first = measured_gemm_configs("mm", "bfloat16", 4096, 4096, 4096)
    record["measured_4096_count"] = len(first)
    first[0]["operand_stages"] = -1
    record["measured_returns_fresh_copies"] = (
        measured_gemm_configs("mm", "bfloat16", 4096, 4096, 4096)[0]["operand_stages"] != -1
    )
    record["measured_unknown_shape"] = list(measured_gemm_configs("mm", "bfloat16", 5, 8, 64))

    schemas = {}
    for op in ("mm", "addmm", "bmm"):
        for dtype in ("float16", "bfloat16"):
            overload = gemm_op(op, dtype, "ayla_fixture")
            schemas[f"{op}/{dtype}"] = str(overload._schema).replace("ayla_fixture::", "ayla::")
    record["schemas"] = schemas
    record["gemm_op_is_cached"] = gemm_op("mm", "bfloat16", "ayla_fixture") is gemm_op("mm", "bfloat16", "ayla_fixture")

    compiler = gemm_jit_compiler("mm", "bfloat16")
    messages = {}
    cpu = torch.empty(8, 8, dtype=torch.bfloat16)
    for label, args in (("wrong_count", (cpu, cpu)), ("not_cuda", (cpu, cpu, cpu))):
        try:
            compiler(*args)
        except Exception as exc:  # noqa: BLE001 - recording the type is the point
            messages[label] = dict(type=type(exc).__name__, message=str(exc))
    try:
        gemm_jit_compiler("gemv", "bfloat16")
    except Exception as exc:  # noqa: BLE001
        messages["unknown_operation"] = dict(type=type(exc).__name__, message=str(exc))
    record["errors"] = messages

    out = HERE / "reference_api.json"
    out.write_text(json.dumps(record, indent=1, sort_keys=True) + "\n")
    print(f"wrote {out}")


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = parser.parse_args()
    make_vectors()
    make_reference_api(Path(args.reference))
