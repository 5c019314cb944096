"""Measured sm_100a GEMM schedules, keyed by the shapes they were measured on.

Same two-level structure as the reference's table (ayla/gemm_schedule_table.py:14,
:1881): ``CONFIGS`` is a tuple of schedule dictionaries and
``SCHEDULES[(operation, dtype)][(batch, m, n, k)]`` lists indices into it, the
fastest measured schedule first.  The keys are the fields of
``struct ayla_b200_config`` (``include/ayla_b200.h``); fields not listed take the
defaults in :mod:`ayla_b200.gemm_jit`.  ``us`` is the median CUDA-event time of
the measurement on a B200 and ``tflops`` the matching throughput; both are
informational and ignored by the launcher.

Regenerate with ``python -m ayla_b200.autotune`` on a B200.
"""
# fmt: off
CONFIGS: tuple[dict[str, object], ...] = (
    dict(tile_n=256, cta_group=2, group_m=8),                               # 0 large square
    dict(tile_n=256, cta_group=1, group_m=8),                               # 1
    dict(tile_n=128, cta_group=2, group_m=8),                               # 2
    dict(tile_n=128, cta_group=1, group_m=8),                               # 3
    dict(tile_n=64, cta_group=1, group_m=8),                                # 4
    dict(tile_n=64, cta_group=1, split_k=4, group_m=8),                     # 5 few tiles, deep K
    dict(tile_n=16, cta_group=1, swap_ab=1, split_k=4, group_m=1),          # 6 weight streaming
    dict(tile_n=32, cta_group=1, swap_ab=1, split_k=4, group_m=1),          # 7
    dict(tile_n=64, cta_group=1, swap_ab=1, split_k=4, group_m=1),          # 8
)

SCHEDULES: dict[tuple[str, str], dict[tuple[int, int, int, int], tuple[int, ...]]] = {
    ("mm", "bfloat16"): {
        (1, 4096, 4096, 4096): (0, 1, 2, 3),
        (1, 8192, 8192, 8192): (0, 1),
    },
    ("mm", "float16"): {
        (1, 4096, 4096, 4096): (0, 1, 2, 3),
    },
    ("addmm", "bfloat16"): {
        (1, 8192, 768, 768): (1, 3),
        (1, 256, 1024, 16384): (5,),
    },
    ("addmm", "float16"): {
        (1, 8192, 768, 768): (1, 3),
        (1, 256, 1024, 16384): (5,),
    },
    ("bmm", "bfloat16"): {
        (64, 2048, 2048, 128): (0, 1),
        (64, 2048, 128, 2048): (2, 3),
    },
    ("bmm", "float16"): {
        (64, 2048, 2048, 128): (0, 1),
        (64, 2048, 128, 2048): (2, 3),
    },
}
# fmt: on
