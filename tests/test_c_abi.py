"""The C-ABI library on a machine without a GPU: it loads, exports everything the
header declares, and its host-side logic (validation, schedule choice, workspace
sizing) behaves.  No kernel is launched here."""

import ctypes
import re
from pathlib import Path

import pytest

from ayla_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "ayla_b200.h"


def declared_symbols() -> list[str]:
    return re.findall(r"AYLA_B200_API[^;(]*?\b(ayla_b200_\w+)\s*\(", HEADER.read_text())


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 12
    lib = _lib.load()
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(_lib.EXPORTS)


def test_version_and_variants():
    assert "sm_100a" in _lib.version()
    variants = _lib.kernel_variants()
    keys = {(v["tile_n"], v["cta_group"], v["epilogue"], v["transposed_out"]) for v in variants}
    assert len(keys) == len(variants)
    for tile_n in (64, 128, 192, 256):
        for cta_group in (1, 2):
            for epilogue in (0, 1):
                assert (tile_n, cta_group, epilogue, 0) in keys
    for tile_n in (16, 32, 64, 128):
        assert (tile_n, 1, 0, 1) in keys and (tile_n, 1, 1, 1) in keys
    assert (256, 1, 2, 0) in keys and (256, 2, 2, 0) in keys
    for v in variants:
        assert v["smem_bytes"] <= 232448 and v["stages"] >= 3


def test_struct_layout_matches_header():
    fields = re.search(r"typedef struct ayla_b200_config \{(.*?)\} ayla_b200_config;", HEADER.read_text(), re.S)
    names = re.findall(r"int32_t\s+(\w+);", fields.group(1))
    assert tuple(names) == _lib.Config.FIELDS
    assert ctypes.sizeof(_lib.Config) == 4 * len(names)


@pytest.mark.parametrize(
    "args, code",
    [
        ((0, 1, 1, 64, 64, 64), 0),
        ((7, 1, 1, 64, 64, 64), _lib.E_INVALID),      # unknown op
        ((0, 5, 1, 64, 64, 64), _lib.E_INVALID),      # unknown dtype
        ((0, 1, 1, 0, 64, 64), _lib.E_INVALID),       # non-positive extent
        ((0, 1, 2, 64, 64, 64), _lib.E_INVALID),      # batch on mm
        ((2, 1, 2, 64, 64, 64), 0),                   # batch on bmm
        ((0, 1, 1, 64, 65, 64), _lib.E_UNSUPPORTED),  # n % 8
        ((0, 1, 1, 64, 64, 36), _lib.E_UNSUPPORTED),  # k % 8
        ((0, 1, 1, 64, 64, 40), 0),                   # k % 8 == 0 is enough (TMA zero-fills the tail)
    ],
)
def test_default_config_validates_shapes(args, code):
    cfg = _lib.Config()
    assert _lib.load().ayla_b200_default_config(*args, ctypes.byref(cfg)) == code
    if code:
        assert _lib.last_error()


def test_default_schedules_for_the_benchmark_shapes():
    big = _lib.default_config("mm", "bfloat16", 1, 4096, 4096, 4096)
    # 256 paired tiles on 74 SM pairs = 3.46 waves: the 34 tiles of the last wave run at half width
    assert (big.tile_n, big.cta_group, big.swap_ab, big.split_k, big.split_tail) == (256, 2, 0, 1, 2)
    assert _lib.workspace_bytes(big, "mm", 1, 4096, 4096, 4096) == 0
    ksplit = _lib.Config.from_dict(dict(tile_n=256, cta_group=2, split_k=2, split_tail=1))
    assert _lib.workspace_bytes(ksplit, "mm", 1, 4096, 4096, 4096) == 65536 + 34 * 2 * 2 * 128 * 256 * 4
    whole = _lib.default_config("mm", "bfloat16", 1, 8192, 8192, 8192)  # 13.8 waves: no split
    assert (whole.split_k, whole.split_tail) == (1, 0)
    decode = _lib.default_config("mm", "bfloat16", 1, 1, 4096, 4096)
    assert decode.swap_ab == 1 and decode.tile_n == 16 and decode.split_k >= 2
    # 112 tiles of bt leave no room to split K: a few dozen rows of `a` go through the plain 128-wide
    # tile (its `a` box trimmed), a handful stay on the swapped form
    m64 = _lib.default_config("mm", "bfloat16", 1, 64, 14336, 4096)
    assert (m64.swap_ab, m64.tile_n, m64.split_k) == (0, 128, 1)
    m8 = _lib.default_config("mm", "bfloat16", 1, 8, 14336, 4096)
    assert (m8.swap_ab, m8.tile_n) == (1, 16)
    m64_k = _lib.default_config("mm", "bfloat16", 1, 64, 4096, 4096)  # 32 tiles: K split over a cluster of 4
    assert (m64_k.swap_ab, m64_k.tile_n, m64_k.split_k, m64_k.cluster_split) == (1, 64, 4, 1)
    m256 = _lib.default_config("mm", "bfloat16", 1, 256, 4096, 4096)  # pairs, K split over two pairs
    assert (m256.tile_n, m256.cta_group, m256.split_k, m256.cluster_split) == (128, 2, 2, 1)
    deep = _lib.default_config("addmm", "bfloat16", 1, 256, 1024, 16384)
    assert deep.swap_ab == 0 and deep.split_k > 1
    for cfg, shape in ((big, (1, 4096, 4096, 4096)), (decode, (1, 1, 4096, 4096)),
                       (deep, (1, 256, 1024, 16384))):
        assert _lib.config_valid(cfg, "mm", "bfloat16", *shape)


def test_config_validation():
    ok = _lib.Config.from_dict(dict(tile_n=128, cta_group=2))
    assert _lib.config_valid(ok, "mm", "bfloat16", 1, 512, 512, 512)
    for bad in (dict(tile_n=48), dict(tile_n=16), dict(cta_group=3), dict(split_k=0), dict(group_m=0),
                dict(tile_n=256, swap_ab=1), dict(tile_n=64, swap_ab=1, cta_group=2), dict(l2_hint_a=3)):
        cfg = _lib.Config.from_dict({**dict(tile_n=128, cta_group=1), **bad})
        assert not _lib.config_valid(cfg, "mm", "bfloat16", 1, 512, 512, 512), bad
    assert _lib.config_valid(_lib.Config.from_dict(dict(tile_n=16, swap_ab=1)), "mm", "float16", 1, 8, 512, 512)
    # cluster split-K: cluster of at most 8 CTAs, tile columns divisible among the k-splits
    csk = dict(tile_n=64, cta_group=1, split_k=4, cluster_split=1)
    assert _lib.config_valid(_lib.Config.from_dict(csk), "mm", "bfloat16", 1, 64, 512, 4096)
    assert _lib.workspace_bytes(_lib.Config.from_dict(csk), "mm", 1, 64, 512, 4096) == 0
    assert _lib.config_valid(_lib.Config.from_dict({**csk, "cta_group": 2}), "mm", "bfloat16", 1, 64, 512, 4096)
    for bad in (dict(split_k=3), dict(cta_group=2, split_k=8), dict(tile_n=16, swap_ab=1, split_k=8), dict(stream_k=1)):
        assert not _lib.config_valid(_lib.Config.from_dict({**csk, **bad}), "mm", "bfloat16", 1, 64, 512, 4096), bad
    assert not _lib.config_valid(_lib.Config.from_dict(csk), "mm", "bfloat16", 1, 64, 512, 128)  # 2 k-blocks, 4 CTAs
    # trimmed tiles exist only in the swapped form
    trimmed = dict(tile_n=16, swap_ab=1, tile_rows=97)
    assert _lib.config_valid(_lib.Config.from_dict(trimmed), "mm", "bfloat16", 1, 8, 14336, 4096)
    for bad in (dict(tile_rows=4), dict(tile_rows=129), dict(swap_ab=0, tile_n=64)):
        assert not _lib.config_valid(_lib.Config.from_dict({**trimmed, **bad}), "mm", "bfloat16", 1, 8, 14336, 4096), bad


def test_workspace_sizing():
    none = _lib.Config.from_dict(dict(tile_n=256, cta_group=1, split_k=1))
    assert _lib.workspace_bytes(none, "mm", 1, 256, 1024, 16384) == 0
    cfg = _lib.Config.from_dict(dict(tile_n=64, cta_group=1, split_k=4))
    # 2 row tiles x 16 column tiles, 4 splits, 128 x 64 fp32 slabs, + the fixed 64 KiB counter header
    counters = _lib.workspace_counter_bytes(cfg, "mm", 1, 256, 1024, 16384)
    assert counters == 65536
    assert _lib.workspace_bytes(cfg, "mm", 1, 256, 1024, 16384) == counters + 32 * 4 * 128 * 64 * 4
    # more splits than 64-wide k blocks are clamped
    deep = _lib.Config.from_dict(dict(tile_n=64, cta_group=1, split_k=64))
    assert _lib.workspace_bytes(deep, "mm", 1, 128, 64, 128) == 65536 + 1 * 2 * 128 * 64 * 4
    huge = _lib.Config.from_dict(dict(tile_n=64, cta_group=1, split_k=2))
    assert not _lib.config_valid(huge, "mm", "bfloat16", 1, 128 * 200, 64 * 100, 256)  # 20000 tiles
    pair = _lib.Config.from_dict(dict(tile_n=128, cta_group=2, split_k=2))
    assert _lib.workspace_bytes(pair, "mm", 1, 256, 128, 1024) == 65536 + 2 * 2 * 128 * 128 * 4


def test_gemm_rejects_bad_arguments_before_touching_the_device():
    lib = _lib.load()
    one = ctypes.c_void_p(16)
    assert lib.ayla_b200_gemm(0, 1, None, None, one, one, 1, 64, 64, 64, None, None, 0, None, None) == _lib.E_INVALID
    assert "non-null" in _lib.last_error()
    assert lib.ayla_b200_gemm(1, 1, None, one, one, one, 1, 64, 64, 64, None, None, 0, None, None) == _lib.E_INVALID
    assert "bias" in _lib.last_error()
    odd = ctypes.c_void_p(24)
    assert lib.ayla_b200_gemm(0, 1, None, odd, one, one, 1, 64, 64, 64, None, None, 0, None, None) == _lib.E_UNSUPPORTED
    assert "16-byte" in _lib.last_error()
    assert lib.ayla_b200_swiglu(1, one, one, None, one, 64, 64, 64, None, None, None) == _lib.E_INVALID
    with pytest.raises(ValueError, match="multiple of 8"):
        _lib.check(lib.ayla_b200_gemm(0, 1, None, one, one, one, 1, 64, 65, 64, None, None, 0, None, None))
