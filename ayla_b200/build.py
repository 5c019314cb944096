"""Build the sm_100a shared library in-tree with nvcc.

``python -m ayla_b200.build`` compiles every ``csrc/*.cu`` for
``compute_100a/sm_100a`` and links ``ayla_b200/lib/libayla_b200.so`` (CUDA runtime
linked statically, the driver API resolved at run time, so the library loads on
a machine without a GPU).  Objects are rebuilt only when a source or header is
newer than the object.  ``--trace`` builds ``libayla_b200_trace.so`` beside it from the
same sources with ``-DAYLA_B200_TRACE``: every CTA stamps ``globaltimer`` at the stages of a
launch into the caller's workspace (read by ``bench.py --case ... --timeline``).
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


TRACE_LIB_PATH = LIB_DIR / "libayla_b200_trace.so"


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False, trace: bool = False) -> Path:
    nvcc = _nvcc()
    build_dir = BUILD_DIR / "trace" if trace else BUILD_DIR
    lib_path = TRACE_LIB_PATH if trace else LIB_PATH
    flags = [*NVCC_FLAGS, "-DAYLA_B200_TRACE"] if trace else NVCC_FLAGS
    build_dir.mkdir(exist_ok=True, parents=True)
    LIB_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_time = _newest_header()
    jobs = []
    for src in sources:
        obj = build_dir / (src.stem + ".o")
        stale = (
            force
            or not obj.exists()
            or obj.stat().st_mtime < max(src.stat().st_mtime, header_time)
        )
        if stale:
            cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
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
    objects = [str(build_dir / (src.stem + ".o")) for src in sources]
    relink = (
        force
        or bool(jobs)
        or not lib_path.exists()
        or lib_path.stat().st_mtime < max(os.stat(o).st_mtime for o in objects)
    )
    if relink:
        cmd = [
            nvcc, "-shared", "-o", str(lib_path), *objects,
            "-gencode", "arch=compute_100a,code=sm_100a",
            "-cudart", "static", "-Xcompiler", "-fPIC",
        ]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or proc.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"linking {lib_path.name} failed")
    return lib_path


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv,
                 trace="--trace" in sys.argv)
    print(path)
