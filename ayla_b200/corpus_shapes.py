"""Turn the operator-call records of the reference's shape corpora into the list of GEMM shapes
the sweep measures.

    python -m ayla_b200.corpus_shapes [--from DIR] [--out ayla_b200/corpus_shapes.json]

The reference measures its schedule table on two corpora of recorded ``mm`` / ``addmm`` / ``bmm``
calls (``benchmarks/oss_pytorch_gemm_shapes.json`` and ``benchmarks/better_benchmark_gemm_shapes.json``:
operand shapes, strides, dtypes and call counts, nothing else).  It pools calls by their mathematical
shape and benchmarks canonical contiguous ``a`` / ``bt`` operands, whatever data order was recorded
(benchmarks/oss_gemm_corpus.py:78-108, :296-330).  This script does the same pooling and keeps what
this backend supports: fp16 / bf16, positive extents, ``n`` and ``k`` multiples of 8, ``bmm`` with a
batch of more than one.  The classes the reference's harness has to skip on Hopper -- ``split_k``
(deep reductions over few output tiles) and ``small_m`` (M below its 64-row MMA tile),
benchmarks/oss_gemm_corpus.py:252-294 -- are kept and labelled, since this backend has schedules for
both.  The output is a data table (shape, dtype, count, class); it is committed so that the sweep can
run where the reference's checkout is not present.
"""

from __future__ import annotations

import argparse
import json
from collections import defaultdict
from pathlib import Path

CORPORA = ("oss_pytorch_gemm_shapes.json", "better_benchmark_gemm_shapes.json")
DEFAULT_OUT = Path(__file__).resolve().parent / "corpus_shapes.json"
_TILE = 64  # the granularity the reference's planner counts tiles in


def shape_class(op: str, batch: int, m: int, n: int, k: int) -> str:
    """``"split_k"``, ``"small_m"`` or ``"plain"``, with the reference planner's thresholds
    (benchmarks/oss_gemm_corpus.py:20-27, :252-294)."""
    output_tiles = -(-m // _TILE) * -(-n // _TILE) * (batch if op == "bmm" else 1)
    reduction_tiles = -(-k // _TILE)
    needs_split = (reduction_tiles >= 32 * output_tiles
                   or (output_tiles < 128 and reduction_tiles >= output_tiles)
                   or (output_tiles < 256 and reduction_tiles >= 8 * output_tiles))
    if needs_split:
        return "split_k"
    if m < _TILE:
        return "small_m"
    return "plain"


def pool(records: list[dict]) -> dict[tuple, dict]:
    pooled: dict[tuple, dict] = defaultdict(lambda: {"count": 0, "suites": set()})
    for rec in records:
        op = str(rec["op"])
        dtypes = {str(arg["dtype"]) for arg in rec["args"]}
        if op not in ("mm", "addmm", "bmm") or len(dtypes) != 1:
            continue
        dtype = dtypes.pop()
        batch = rec.get("b")
        batch = 1 if batch is None else int(batch)
        m, n, k = int(rec["m"]), int(rec["n"]), int(rec["k"])
        if dtype not in ("float16", "bfloat16") or min(m, n, k, batch) <= 0:
            continue
        if (op == "bmm") != (rec.get("b") is not None) or (op == "bmm" and batch <= 1):
            continue
        if n % 8 or k % 8:
            continue
        entry = pooled[(op, dtype, batch, m, n, k)]
        entry["count"] += int(rec["count"])
        entry["suites"].add(str(rec["suite"]).split("/")[0])
    return pooled


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--from", dest="source", required=True,
                        help="directory that holds the reference's two corpus files (its benchmarks/ folder)")
    parser.add_argument("--out", default=str(DEFAULT_OUT))
    args = parser.parse_args()
    records: list[dict] = []
    for name in CORPORA:
        records += json.loads((Path(args.source) / name).read_text())
    pooled = pool(records)
    rows = [
        {"op": op, "dtype": dtype, "batch": batch, "m": m, "n": n, "k": k, "count": entry["count"],
         "class": shape_class(op, batch, m, n, k), "suites": sorted(entry["suites"])}
        for (op, dtype, batch, m, n, k), entry in pooled.items()
    ]
    rows.sort(key=lambda r: (-r["count"], r["op"], r["dtype"], r["batch"], r["m"], r["n"], r["k"]))
    Path(args.out).write_text("[\n" + ",\n".join(json.dumps(r) for r in rows) + "\n]\n")
    by_class: dict[str, int] = defaultdict(int)
    for r in rows:
        by_class[r["class"]] += 1
    print(f"{len(records)} records -> {len(rows)} shapes {dict(by_class)} -> {args.out}")


if __name__ == "__main__":
    main()
