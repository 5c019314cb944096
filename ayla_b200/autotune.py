"""Measure candidate schedules per shape on a B200 and regenerate the schedule table.

    python -m ayla_b200.autotune --out results/autotune.json            # measure (resumable)
    python -m ayla_b200.autotune --out results/autotune.json --emit ayla_b200/gemm_schedule_table.py

The sweep mirrors how the reference's table was produced (per-shape sweeps whose winners are
stored first, ayla/gemm_schedule_table.py:1-12) and its harness' resume behaviour: results are
rewritten atomically after every shape and finished shapes are skipped on a re-run
(benchmarks/oss_gemm_corpus.py:418-442, benchmarks/benchmark_oss_pytorch_gemm_shapes.py:294-318).
The results file has to be present where the sweep runs for finished shapes to be skipped and kept:
a run that starts without it writes only the shapes it measured.  Timing protocol: see
:mod:`ayla_b200.suite`.
"""

from __future__ import annotations

import argparse
import json
import math
import os
from pathlib import Path

import torch

from . import _lib
from .suite import SWEEP_M, SWEEP_NK, _copies, time_interleaved

MAX_WORKSPACE = 512 << 20
SM_COUNT = 148

HEADLINE_SHAPES = [
    ("mm", "bfloat16", 1, 4096, 4096, 4096),
    ("mm", "float16", 1, 4096, 4096, 4096),
    ("mm", "bfloat16", 1, 8192, 8192, 8192),
    ("addmm", "bfloat16", 1, 8192, 768, 768),
    ("addmm", "float16", 1, 8192, 768, 768),
    ("addmm", "bfloat16", 1, 256, 1024, 16384),
    ("addmm", "float16", 1, 256, 1024, 16384),
    ("bmm", "bfloat16", 64, 2048, 2048, 128),
    ("bmm", "bfloat16", 64, 2048, 128, 2048),
    ("bmm", "bfloat16", 8, 2048, 2048, 128),
    ("bmm", "bfloat16", 8, 2048, 128, 2048),
    ("mm", "bfloat16", 1, 4096, 4096, 32768),
]
# Projections of an 8B-class decoder that the sweep does not cover (fused QKV, concatenated gate/up).
DECODER_SHAPES = ([("mm", "bfloat16", 1, m, 6144, 4096) for m in (8, 64, 256, 512, 1024, 2048, 4096)]
                  + [("mm", "bfloat16", 1, m, 28672, 4096) for m in (8, 64, 512, 4096)])
# Larger models: hidden 8192, FFN 28672 (70B-class layer shapes), decode and prefill row counts.
LARGE_SHAPES = [("mm", "bfloat16", 1, m, n, k) for (n, k) in ((8192, 8192), (10240, 8192), (28672, 8192), (8192, 28672))
                for m in (8, 64, 512, 4096)]
SWEEP_SHAPES = [("mm", "bfloat16", 1, m, n, k) for n, k in SWEEP_NK for m in SWEEP_M]


def corpus_shapes(limit: int = 0) -> list[tuple]:
    """The reference's shape corpora as pooled by :mod:`ayla_b200.corpus_shapes`, most frequent first.
    fp16 and bf16 run the same kernels at the same speed and ``select_gemm_schedule`` lets a shape
    measured in one serve the other, so a shape recorded in both is measured once (in bf16)."""
    rows = json.loads((Path(__file__).resolve().parent / "corpus_shapes.json").read_text())
    seen: dict[tuple, tuple] = {}
    for r in rows:
        key = (r["op"], r["batch"], r["m"], r["n"], r["k"])
        if key not in seen or r["dtype"] == "bfloat16":
            seen[key] = (r["op"], r["dtype"], r["batch"], r["m"], r["n"], r["k"])
    shapes = list(seen.values())
    return shapes[:limit] if limit else shapes


def candidates(op: str, batch: int, m: int, n: int, k: int) -> list[dict]:
    k_blocks = -(-k // 64)
    out: list[dict] = []
    splits = [s for s in (2, 4, 8, 16) if k_blocks >= 4 * s]
    if m <= 128 and n >= 128:
        widths = sorted({w for w in (16, 32, 64, 128) if w >= min(m, 128)} | {128})
        # Trimmed tiles: as many rows per tile as spread bt over a whole number of waves.
        waves = -(-(batch * -(-n // 128)) // SM_COUNT)
        rows = -(-n * batch // (SM_COUNT * waves))
        trims = sorted({r for r in (rows, -(-rows // 8) * 8) if 8 <= r < 128}) if batch == 1 else []
        for w in widths[:3]:
            base = dict(tile_n=w, cta_group=1, swap_ab=1, group_m=1)
            out.append(dict(base))
            for r in trims:
                out.append(dict(base, tile_rows=r))
            for s in splits[:3]:
                out.append(dict(base, split_k=s))
            for s in (2, 4, 8):
                if k_blocks >= 4 * s and w % (4 * s) == 0:
                    out.append(dict(base, split_k=s, cluster_split=1))
    for tile_n in (64, 128, 192, 256):
        if tile_n > 64 and n < tile_n // 2:
            continue
        for cta_group in (1, 2):
            if cta_group == 2 and m <= 128:
                continue
            base = dict(tile_n=tile_n, cta_group=cta_group, group_m=8)
            out.append(dict(base))
            if tile_n % 128 == 0:
                out.append(dict(base, split_tail=2))
            tiles = batch * -(-m // (128 * cta_group)) * -(-n // tile_n)
            if tiles * cta_group <= SM_COUNT:
                for s in splits[:3]:
                    out.append(dict(base, split_k=s))
                # Very deep reductions over a handful of tiles (weight gradients: K = tokens): split until the
                # grid is full, as long as every split keeps at least eight k-blocks.
                if tile_n <= 128:
                    for s in (16, 32, 64, 128):
                        if s not in splits[:3] and k_blocks >= 8 * s and tiles * s * cta_group <= 2 * SM_COUNT:
                            out.append(dict(base, split_k=s))
                for s in (2, 4, 8):
                    if tile_n != 192 and s * cta_group <= 4 and k_blocks >= 4 * s and tiles * s * cta_group <= 2 * SM_COUNT:
                        out.append(dict(base, split_k=s, cluster_split=1))
                if tile_n != 192 and cta_group == 1 and k_blocks >= 32 and tiles * 8 <= 2 * SM_COUNT:
                    out.append(dict(base, split_k=8, cluster_split=1))
    return out


def tune_shape(op: str, dtype: str, batch: int, m: int, n: int, k: int, rounds: int = 5, light: bool = False,
               only: list[dict] | None = None) -> dict:
    """Rank schedules for one shape next to cuBLAS.  With ``only`` (a play-off between the winners of
    earlier sweeps) just those schedules are timed, twice -- on the GPU as it is and again right after
    a third of a second of dense GEMMs, when the SM clock sits under the power cap -- and ranked by the
    product of the two times: the weight-streaming schedules rank differently in the two states."""
    dev = "cuda"
    td = torch.bfloat16 if dtype == "bfloat16" else torch.float16
    lead = (batch,) if op == "bmm" else ()
    nbytes = 2.0 * batch * (m * k + n * k + m * n)
    copies = _copies(nbytes, cap=12)
    sets = []
    for _ in range(copies):
        a = torch.randn((*lead, m, k), device=dev, dtype=torch.float32).mul_(k ** -0.5).to(td)
        bt = torch.randn((*lead, n, k), device=dev, dtype=torch.float32).to(td)
        out = torch.empty((*lead, m, n), device=dev, dtype=td)
        bias = torch.randn(n, device=dev).to(td) if op == "addmm" else None
        sets.append((bias, a, bt, out))
    flops = 2.0 * batch * m * n * k
    est_ms = max(flops / 1.0e15, nbytes / 3e12) * 1e3 + 0.006
    launches = int(max(4, min(30, 1.5 / est_ms)))
    workspace = torch.zeros(16, dtype=torch.uint8, device=dev)
    fns = {}
    configs = {}
    for i, cand in enumerate(only if only is not None else candidates(op, batch, m, n, k)):
        cfg = _lib.Config.from_dict(cand)
        if not _lib.config_valid(cfg, op, dtype, batch, m, n, k):
            continue
        need = _lib.workspace_bytes(cfg, op, batch, m, n, k)
        if need > MAX_WORKSPACE:
            continue
        if need > workspace.numel():
            workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        configs[f"c{i}"] = cand

    def make(cand):
        cfg = _lib.Config.from_dict(cand)

        def run(j, stream):
            bias, a, bt, out = sets[j % copies]
            _lib.gemm(op, dtype, bias.data_ptr() if bias is not None else 0, a.data_ptr(), bt.data_ptr(),
                      out.data_ptr(), batch, m, n, k, cfg, workspace.data_ptr(), workspace.numel(), 0, stream)

        return run

    for name, cand in configs.items():
        fns[name] = make(cand)

    def cublas(j, stream):
        bias, a, bt, out = sets[j % copies]
        if op == "mm":
            torch.mm(a, bt.t(), out=out)
        elif op == "addmm":
            torch.addmm(bias, a, bt.t(), out=out)
        else:
            torch.bmm(a, bt.transpose(1, 2), out=out)

    fns["torch"] = cublas
    times = time_interleaved(fns, launches, rounds)
    if only is not None and len(fns) > 1:
        heater = torch.randn(8192, 8192, device=dev).to(torch.bfloat16)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(400):  # about 0.7 ms each: stop after a third of a second
            torch.mm(heater, heater)
            stop.record()
            if stop.query() and start.elapsed_time(stop) > 330.0:
                break
        torch.cuda.synchronize()
        del heater
        hot = time_interleaved(fns, launches, rounds)
        times = {name: math.sqrt(ms * hot[name]) for name, ms in times.items()}
    torch_ms = times.pop("torch")
    ranked = sorted(times.items(), key=lambda kv: kv[1])
    if not ranked or only is not None:
        del sets
        torch.cuda.empty_cache()
        results = [dict(config=configs[name], us=ms * 1e3, tflops=flops / ms / 1e9, gbs=nbytes / ms / 1e6,
                        percentage_of_torch=100.0 * torch_ms / ms) for name, ms in ranked]
        return dict(op=op, dtype=dtype, batch=batch, m=m, n=n, k=k, torch_us=torch_ms * 1e3, results=results)

    def refine_pass(tweaks_for, label):
        """Time variations of the two fastest schedules next to the fastest itself (the yardstick that
        ties this pass's times to the first pass's) and merge them into the ranking."""
        nonlocal ranked
        refine = {}
        for name, _ in ranked[:2]:
            base = configs[name]
            for j, tweak in enumerate(tweaks_for(base)):
                cand = {**base, **tweak}
                if cand != base and _lib.config_valid(_lib.Config.from_dict(cand), op, dtype, batch, m, n, k):
                    refine[f"{name}{label}{j}"] = cand
        if not refine:
            return
        fns2 = {name: make(cand) for name, cand in refine.items()}
        fns2[ranked[0][0]] = make(configs[ranked[0][0]])
        times2 = time_interleaved(fns2, launches, rounds)
        scale = times[ranked[0][0]] / times2.pop(ranked[0][0])
        for name, ms in times2.items():
            configs[name] = refine[name]
            times[name] = ms * scale
        ranked = sorted(times.items(), key=lambda kv: kv[1])

    # Second pass: raster width and L2 eviction hints around the two fastest schedules.
    def hint_tweaks(base):
        tweaks = [dict(l2_hint_a=a, l2_hint_b=b) for a in (0, 1, 2) for b in (0, 1, 2) if a or b]
        if not base.get("swap_ab"):
            tweaks += [dict(group_m=g) for g in (2, 4, 16) if g != base.get("group_m")]
        return tweaks

    if not light:
        refine_pass(hint_tweaks, "r")
    if flops / nbytes < 250.0:
        # Third pass, HBM-bound shapes (ridge ~ 248 flop/byte at the measured peaks): how many k-blocks of
        # its first tile a CTA asks into L2 before it waits for the preceding launch.
        def early_tweaks(base):
            share = -(-k // 64) // int(base.get("split_k", 1))
            return [dict(early_prefetch=e) for e in (4, 8, 12, 16, 24, 32) if e <= share]

        refine_pass(early_tweaks, "e")
    elif flops >= 5e10 and not light:
        # Large compute-bound shapes run for seconds under the power cap in real use, where the schedules
        # rank differently than in short bursts (the L2 hints that keep operands resident save power).
        # Rank the three fastest again in that regime: back-to-back launches for a quarter of a second each,
        # after the GPU has been brought to its capped state, arms alternating twice.
        top = [name for name, _ in ranked[:3]]
        runners = {name: make(configs[name]) for name in top}
        stream = torch.cuda.current_stream().cuda_stream
        per_launch = times[top[0]]
        block = int(max(50, min(4000, 250.0 / per_launch)))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for j in range(2 * block):
            runners[top[0]](j, stream)
        sustained = {name: 0.0 for name in top}
        for rnd in range(2):
            for name in top[rnd % len(top):] + top[:rnd % len(top)]:
                start.record()
                for j in range(block):
                    runners[name](j, stream)
                stop.record()
                stop.synchronize()
                sustained[name] += start.elapsed_time(stop) / (2 * block)
        order = sorted(top, key=sustained.__getitem__)
        rest = [name for name, _ in ranked if name not in top]
        ranked = [(name, times[name]) for name in order + rest]
        for name in top:
            configs[name] = dict(configs[name], sustained_us=round(sustained[name] * 1e3, 2))
    if flops / nbytes < 250.0 or flops < 5e10 or light:
        # Final pass (everything the sustained-regime pass did not order): the three fastest again, alone
        # with cuBLAS.  In the big interleaved passes a launch meets whatever the forty other schedules
        # left in L2, and eviction hints in particular can rank differently there than between two arms
        # (C3a: both operands evict-first read 110 us among forty candidates, 140 us next to cuBLAS alone).
        top = [name for name, _ in ranked[:3]]
        final = time_interleaved({**{name: make(configs[name]) for name in top}, "torch": cublas}, launches, rounds)
        torch_ms = final.pop("torch")
        for name in top:
            times[name] = final[name]
        order = sorted(top, key=final.__getitem__)
        rest = [(name, ms) for name, ms in ranked if name not in top]
        ranked = [(name, times[name]) for name in order] + rest
    results = [dict(config=configs[name], us=ms * 1e3, tflops=flops / ms / 1e9, gbs=nbytes / ms / 1e6,
                    percentage_of_torch=100.0 * torch_ms / ms) for name, ms in ranked]
    del sets
    torch.cuda.empty_cache()
    return dict(op=op, dtype=dtype, batch=batch, m=m, n=n, k=k, torch_us=torch_ms * 1e3, results=results)


_KEY = ("op", "dtype", "batch", "m", "n", "k")


def _load_done(out_path: Path) -> dict[tuple, dict]:
    if not out_path.exists():
        return {}
    return {tuple(r[key] for key in _KEY): r for r in json.loads(out_path.read_text())}


def _write_done(done: dict[tuple, dict], out_path: Path) -> None:
    tmp = out_path.with_suffix(".tmp")
    tmp.write_text(json.dumps(list(done.values()), indent=1))
    os.replace(tmp, out_path)


def measure(shapes, out_path: Path, rounds: int = 5, progress_path: Path | None = None, light: bool = False) -> None:
    """Measure every shape not yet in ``out_path``, rewriting the file atomically after each one.
    ``progress_path``, if given, names the shape being measured (for the supervising process of
    :func:`measure_isolated`)."""
    _lib.init(torch.cuda.current_device())
    done = _load_done(out_path)
    for shape in shapes:
        if tuple(shape) in done:
            continue
        if progress_path is not None:
            progress_path.write_text(json.dumps(list(shape)))
        row = tune_shape(*shape, rounds=rounds, light=light)
        done[tuple(shape)] = row
        if not row["results"]:
            print(f"[autotune] {shape}: no valid schedule", flush=True)
        else:
            best = row["results"][0]
            print(f"[autotune] {shape}: best {best['us']:.1f} us {best['tflops']:.0f} TF/s {best['gbs']:.0f} GB/s "
                  f"({best['percentage_of_torch']:.0f}% of torch) {best['config']}", flush=True)
        _write_done(done, out_path)


def measure_isolated(shapes, out_path: Path, shapes_file: Path, rounds: int = 3,
                     per_shape_timeout: float = 120.0, light: bool = False) -> None:
    """The sweep in a worker process, supervised from this one (which never touches the GPU).

    The reference's harness spawns one process per shape with a timeout and resumes finished shapes
    (benchmarks/benchmark_oss_pytorch_gemm_shapes.py:198-227, :294-318).  A process per shape would
    spend seconds of start-up on every sub-millisecond measurement here, so one worker measures
    shape after shape and names the shape it is on in a progress file; this process watches that
    file.  A worker that dies, or that stays on one shape beyond ``per_shape_timeout`` seconds, is
    stopped (its own process id, nothing else), the shape is recorded as failed so that a resumed
    sweep skips it, and a fresh worker carries on with the rest."""
    import subprocess
    import sys
    import time

    progress = out_path.with_suffix(".progress")
    wanted = [tuple(s) for s in shapes]
    while True:
        done = _load_done(out_path)
        if all(s in done for s in wanted):
            return
        progress.unlink(missing_ok=True)
        worker = subprocess.Popen([sys.executable, "-m", "ayla_b200.autotune", "--worker", "--out", str(out_path),
                                   "--shapes-file", str(shapes_file), "--rounds", str(rounds)]
                                  + (["--light"] if light else []))
        last_shape, since = None, time.monotonic()
        failed = None
        while worker.poll() is None:
            time.sleep(0.5)
            current = progress.read_text() if progress.exists() else None
            if current != last_shape:
                last_shape, since = current, time.monotonic()
            elif time.monotonic() - since > per_shape_timeout:
                worker.kill()
                worker.wait()
                failed = "timeout"
        if failed is None and worker.returncode == 0:
            continue  # the loop's first lines decide whether anything is left
        reason = failed or f"worker exited with code {worker.returncode}"
        done = _load_done(out_path)
        stuck = tuple(json.loads(last_shape)) if last_shape else next(s for s in wanted if s not in done)
        if stuck not in done:
            done[stuck] = dict(zip(_KEY, stuck), torch_us=None, results=[], error=reason)
            _write_done(done, out_path)
        print(f"[autotune] {stuck}: {reason}; restarting the worker", flush=True)


def playoff(results_paths: list[Path], out_path: Path, keep: int = 3, rounds: int = 5, limit: int = 0) -> None:
    """Time the ``keep`` fastest schedules of every results file against each other, shape by shape in
    the first file's order, and write the ranking to ``out_path`` (same format, resumable): two sweeps
    of the same shape, run at different times, rank close schedules differently, and their own times
    cannot be compared across runs."""
    _lib.init(torch.cuda.current_device())
    sweeps = [_load_done(path) for path in results_paths]
    done = _load_done(out_path)
    for index, shape in enumerate(sweeps[0]):
        if limit and index >= limit:
            break
        if shape in done:
            continue
        seeds: list[dict] = []
        for sweep in sweeps:
            for entry in sweep.get(shape, {}).get("results", [])[:keep]:
                cand = {key: value for key, value in entry["config"].items() if key != "sustained_us"}
                if cand not in seeds:
                    seeds.append(cand)
        if not seeds:
            continue
        row = tune_shape(*shape, rounds=rounds, only=seeds)
        done[shape] = row
        if row["results"]:
            best = row["results"][0]
            print(f"[playoff] {shape}: {len(seeds)} schedules, best {best['us']:.1f} us "
                  f"({best['percentage_of_torch']:.0f}% of torch) {best['config']}", flush=True)
        _write_done(done, out_path)


def emit_table(results_paths: list[Path], table_path: Path, keep: tuple[int, ...] = (3,)) -> None:
    """Write the schedule table from one or more results files.  A shape present in several files takes
    its rows from the first file that has it; ``keep[i]`` schedules per shape are kept from file i
    (the last value serves the remaining files)."""
    rows: list[dict] = []
    seen: set[tuple] = set()
    for index, path in enumerate(results_paths):
        limit = keep[min(index, len(keep) - 1)]
        for row in json.loads(path.read_text()):
            key = tuple(row[k] for k in _KEY)
            if key in seen:
                continue
            seen.add(key)
            rows.append(dict(row, results=row["results"][:limit]))
    configs: list[dict] = []
    index: dict[str, int] = {}
    schedules: dict[tuple[str, str], dict[tuple[int, int, int, int], list[int]]] = {}
    for row in rows:
        if not row["results"]:
            continue  # a shape whose measurement failed or that has no valid schedule
        picks = []
        for res in row["results"]:
            entry = dict(res["config"])
            entry["us"] = round(res["us"], 2)
            entry["tflops"] = round(res["tflops"], 1)
            entry["percentage_of_torch"] = round(res["percentage_of_torch"], 1)
            key = json.dumps(entry, sort_keys=True)
            if key not in index:
                index[key] = len(configs)
                configs.append(entry)
            picks.append(index[key])
        schedules.setdefault((row["op"], row["dtype"]), {})[(row["batch"], row["m"], row["n"], row["k"])] = picks
    lines = [
        '"""Measured sm_100a GEMM schedules, keyed by the shapes they were measured on.',
        "",
        "Same two-level structure as the reference's table (ayla/gemm_schedule_table.py:14,",
        ":1881): ``CONFIGS`` is a tuple of schedule dictionaries and",
        "``SCHEDULES[(operation, dtype)][(batch, m, n, k)]`` lists indices into it, the",
        "fastest measured schedule first.  The schedule keys are the fields of",
        "``struct ayla_b200_config`` (``include/ayla_b200.h``); fields not listed take the",
        "defaults in :mod:`ayla_b200.gemm_jit`.  ``us`` is the median CUDA-event time per launch",
        "on a B200 (graph replay, operands rotating through more than 2.5x L2), ``tflops`` the",
        "matching throughput and ``percentage_of_torch`` 100 x cuBLAS time / this time in the same",
        "run; all three are informational and ignored by the launcher.  Large compute-bound shapes carry",
        "``sustained_us`` on their three fastest schedules: the time per launch in a quarter-second",
        "back-to-back loop under the power cap, which is what orders those three.",
        "",
        "Generated by ``python -m ayla_b200.autotune``; do not edit by hand.",
        '"""',
        "# fmt: off",
        "CONFIGS: tuple[dict[str, object], ...] = (",
    ]
    for entry in configs:
        body = ", ".join(f"{k}={v!r}" for k, v in entry.items())
        lines.append(f"    dict({body}),")
    lines.append(")")
    lines.append("")
    lines.append("SCHEDULES: dict[tuple[str, str], dict[tuple[int, int, int, int], tuple[int, ...]]] = {")
    for (op, dtype), shapes in sorted(schedules.items()):
        lines.append(f"    ({op!r}, {dtype!r}): {{")
        for shape, picks in sorted(shapes.items()):
            lines.append(f"        {shape!r}: {tuple(picks)!r},")
        lines.append("    },")
    lines.append("}")
    lines.append("# fmt: on")
    table_path.write_text("\n".join(lines) + "\n")
    print(f"wrote {table_path}: {len(configs)} configs, {sum(len(v) for v in schedules.values())} shapes")


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--out", default="results/autotune.json")
    parser.add_argument("--shapes", default="all", choices=["all", "baseline", "sweep", "decoder", "large", "corpus"])
    parser.add_argument("--emit", default=None,
                        help="write the schedule table to this path instead of measuring (--out may then list "
                             "several results files, comma separated; the first file that has a shape wins)")
    parser.add_argument("--emit-keep", default="3", help="schedules kept per shape, per results file (comma separated)")
    parser.add_argument("--isolate", action="store_true", help="measure in a supervised worker process")
    parser.add_argument("--rounds", type=int, default=5)
    parser.add_argument("--limit", type=int, default=0, help="corpus, play-off: only the first N shapes (0 = all)")
    parser.add_argument("--light", action="store_true",
                        help="no eviction-hint pass and no sustained-regime pass (the broad corpus sweep)")
    parser.add_argument("--playoff", default=None,
                        help="comma-separated results files: time their fastest schedules against each other "
                             "and write the ranking to --out")
    parser.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    parser.add_argument("--shapes-file", default=None, help=argparse.SUPPRESS)
    args = parser.parse_args()
    if args.emit:
        emit_table([Path(p) for p in args.out.split(",")], Path(args.emit),
                   tuple(int(v) for v in args.emit_keep.split(",")))
        return
    out = Path(args.out)
    out.parent.mkdir(parents=True, exist_ok=True)
    if args.playoff:
        playoff([Path(p) for p in args.playoff.split(",")], out, keep=int(args.emit_keep.split(",")[0]),
                rounds=args.rounds, limit=args.limit)
        return
    if args.worker:
        shapes = [tuple(s) for s in json.loads(Path(args.shapes_file).read_text())]
        measure(shapes, out, rounds=args.rounds, progress_path=out.with_suffix(".progress"), light=args.light)
        return
    shapes = []
    if args.shapes == "corpus":
        shapes += corpus_shapes(args.limit)
    if args.shapes in ("all", "baseline"):
        shapes += HEADLINE_SHAPES
    if args.shapes in ("all", "sweep"):
        shapes += SWEEP_SHAPES
    if args.shapes in ("all", "decoder"):
        shapes += DECODER_SHAPES
    if args.shapes in ("all", "large"):
        shapes += LARGE_SHAPES
    if args.isolate:
        shapes_file = out.with_suffix(".shapes")
        shapes_file.write_text(json.dumps([list(s) for s in shapes]))
        measure_isolated(shapes, out, shapes_file, rounds=args.rounds, light=args.light)
    else:
        measure(shapes, out, rounds=args.rounds, light=args.light)


if __name__ == "__main__":
    main()
