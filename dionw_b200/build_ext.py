"""Build ``libdionw_b200.so`` in-tree with nvcc for sm_100a.

    python -m dionw_b200.build_ext [--force] [--verbose]

The library links the CUDA runtime statically and nothing else, so it loads on
a machine without a GPU or driver (every entry point then returns an error).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "lib" / "libdionw_b200.so"
SOURCES = ("api.cu", "momentum.cu", "update.cu", "gemm.cu", "newton_schulz.cu", "newton_schulz_static.cu")
FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-cudart", "static",
    # host code: no fused multiply-adds the source does not spell out (the CPU EMA's lerp is bit-checked)
    "-Xcompiler", "-ffp-contract=off",
)


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: dionw_b200 needs the CUDA 12.8+ toolkit to build its kernels")
    return found


def _stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    deps = [*CSRC.glob("*.cu"), *CSRC.glob("*.cuh"), PACKAGE.parent / "include" / "dionw_b200.h"]
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources."""
    if not force and not _stale():
        return LIBRARY
    LIBRARY.parent.mkdir(exist_ok=True)
    objects = []
    jobs = []
    for name in SOURCES:
        obj = LIBRARY.parent / (name + ".o")
        cmd = [_nvcc(), *FLAGS, "-c", str(CSRC / name), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        jobs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    failed = False
    for name, proc in jobs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            print(f"--- {name}\n{out}", file=sys.stderr)
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the output above")
    link = [_nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
            "-o", str(LIBRARY), *objects, "-lpthread"]
    subprocess.run(link, check=True)
    for obj in objects:
        os.remove(obj)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
