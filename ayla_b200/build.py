"""Build the sm_100a shared library in-tree with nvcc.

``python -m ayla_b200.build`` compiles every ``csrc/*.cu`` for
``compute_100a/sm_100a`` and links ``ayla_b200/lib/libayla_b200.so`` (CUDA runtime
linked statically, the driver API resolved at run time, so the library loads on
a machine without a GPU).  Objects are rebuilt only when a source or header is
newer than the object.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
BUILD_DIR = PACKAGE_DIR / "build"
LIB_DIR = PACKAGE_DIR / "lib"
LIB_PATH = LIB_DIR / "libayla_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built")
    return nvcc


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    headers.append(PACKAGE_DIR.parent / "include" / "ayla_b200.h")
    return max(h.stat().st_mtime for h in headers)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = _nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_time = _newest_header()
    jobs = []
    for src in sources:
        obj = BUILD_DIR / (src.stem + ".o")
        stale = (
            force
            or not obj.exists()
            or obj.stat().st_mtime < max(src.stat().st_mtime, header_time)
        )
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, proc

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for cmd, proc in pool.map(run, jobs):
                if verbose or proc.returncode != 0 or ptxas_info:
                    sys.stderr.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
                if proc.returncode != 0:
                    raise RuntimeError(f"nvcc failed for {cmd[-3]}")
    objects = [str(BUILD_DIR / (src.stem + ".o")) for src in sources]
    relink = (
        force
        or bool(jobs)
        or not LIB_PATH.exists()
        or LIB_PATH.stat().st_mtime < max(os.stat(o).st_mtime for o in objects)
    )
    if relink:
        cmd = [
            nvcc, "-shared", "-o", str(LIB_PATH), *objects,
            "-gencode", "arch=compute_100a,code=sm_100a",
            "-cudart", "static", "-Xcompiler", "-fPIC",
        ]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or proc.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError("linking libayla_b200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
