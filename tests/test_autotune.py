"""Host logic of the schedule sweep (``ayla_b200.autotune``): which schedules are tried, how the results
of several sweeps are merged into the table, and the play-off between sweeps.  No GPU: the timing
function is replaced by a fake."""

import importlib.util
import json

import pytest
import torch

from ayla_b200 import autotune


def _row(op, dtype, batch, m, n, k, configs, torch_us=10.0):
    results = [dict(config=c, us=5.0 + i, tflops=1.0, gbs=1.0, percentage_of_torch=100.0 * torch_us / (5.0 + i))
               for i, c in enumerate(configs)]
    return dict(op=op, dtype=dtype, batch=batch, m=m, n=n, k=k, torch_us=torch_us, results=results)


def _load_table(path):
    spec = importlib.util.spec_from_file_location("table_under_test", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_candidates_cover_the_regimes_the_table_relies_on():
    small = autotune.candidates("mm", 1, 8, 14336, 4096)
    assert any(c.get("swap_ab") and c.get("tile_rows") for c in small)          # trimmed weight tiles
    assert any(c.get("swap_ab") and c.get("cluster_split") for c in small)      # cluster k-split of the swapped form
    deep = autotune.candidates("mm", 1, 16, 16, 663552)
    assert max(c.get("split_k", 1) for c in deep) >= 64                          # weight gradients: deep k-splits
    large = autotune.candidates("mm", 1, 4096, 4096, 4096)
    assert dict(tile_n=256, cta_group=2, group_m=8) in large and dict(tile_n=256, cta_group=2, group_m=8, split_tail=2) in large
    assert not any(c.get("swap_ab") for c in large)


def test_emit_table_takes_a_shape_from_the_first_file_that_has_it(tmp_path):
    a, b = dict(tile_n=256, cta_group=2), dict(tile_n=128, cta_group=1)
    c, d = dict(tile_n=64, cta_group=1), dict(tile_n=192, cta_group=2)
    first = tmp_path / "first.json"
    second = tmp_path / "second.json"
    first.write_text(json.dumps([_row("mm", "bfloat16", 1, 512, 512, 512, [a, b, c])]))
    second.write_text(json.dumps([_row("mm", "bfloat16", 1, 512, 512, 512, [d]),
                                  _row("mm", "bfloat16", 1, 64, 512, 512, [c, d, a]),
                                  _row("bmm", "float16", 4, 64, 64, 64, [])]))       # failed shape: no entry
    table = tmp_path / "table.py"
    autotune.emit_table([first, second], table, keep=(2, 1))
    module = _load_table(table)
    picks = module.SCHEDULES[("mm", "bfloat16")][(1, 512, 512, 512)]
    assert [module.CONFIGS[i]["tile_n"] for i in picks] == [256, 128]                # first file, two kept
    picks = module.SCHEDULES[("mm", "bfloat16")][(1, 64, 512, 512)]
    assert [module.CONFIGS[i]["tile_n"] for i in picks] == [64]                      # second file, one kept
    assert ("bmm", "float16") not in module.SCHEDULES


def test_playoff_times_the_union_of_the_sweeps_winners_and_resumes(tmp_path, monkeypatch):
    a, b, c = dict(tile_n=256, cta_group=2), dict(tile_n=128, cta_group=1), dict(tile_n=64, cta_group=1)
    new = tmp_path / "new.json"
    old = tmp_path / "old.json"
    shape1, shape2 = ("mm", "bfloat16", 1, 512, 512, 512), ("mm", "bfloat16", 1, 64, 512, 512)
    new.write_text(json.dumps([_row(*shape1, [dict(a, sustained_us=9.0), b]), _row(*shape2, [c])]))
    old.write_text(json.dumps([_row(*shape1, [b, c]), _row("mm", "float16", 1, 8, 8, 8, [a])]))
    calls = []

    def fake_tune_shape(op, dtype, batch, m, n, k, rounds=5, light=False, only=None):
        calls.append(((op, dtype, batch, m, n, k), only))
        return _row(op, dtype, batch, m, n, k, list(reversed(only)))

    monkeypatch.setattr(autotune, "tune_shape", fake_tune_shape)
    monkeypatch.setattr(autotune._lib, "init", lambda device: None)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    out = tmp_path / "playoff.json"
    autotune.playoff([new, old], out, keep=2, rounds=1, limit=1)
    assert [shape for shape, _ in calls] == [shape1]                                 # limit: first shape only
    assert calls[0][1] == [a, b, c]                                                  # union, no duplicates, no sustained_us
    autotune.playoff([new, old], out, keep=2, rounds=1)
    assert [shape for shape, _ in calls] == [shape1, shape2]                         # resumed: shape1 not timed again
    rows = {tuple(r[k] for k in ("op", "dtype", "batch", "m", "n", "k")): r for r in json.loads(out.read_text())}
    assert set(rows) == {shape1, shape2}                                             # only the first file's shapes
    assert rows[shape1]["results"][0]["config"] == c                                 # the fake's ranking is what is kept
