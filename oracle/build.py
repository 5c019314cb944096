"""Compile the plain-C oracle (``gemm_ref.c``) into ``oracle/libgemm_ref.so`` with gcc.

The reference under test is pure Python whose GPU kernels are generated Hopper PTX,
so there is no reference C/C++ source to build into ``oracle/_ref``; this script
only builds the restatement.
"""

from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "gemm_ref.c"
LIB = HERE / "libgemm_ref.so"


def build(force: bool = False) -> Path:
    if force or not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
        subprocess.run(
            ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", str(SRC), "-o", str(LIB), "-lm"],
            check=True,
        )
    return LIB


if __name__ == "__main__":
    print(build(force=True))
