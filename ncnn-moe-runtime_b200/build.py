"""Builds libmoe_b200_sampler.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python ncnn-moe-runtime_b200/build.py [--force]

nvcc cross-compiles without a GPU.  The library is written next to this file so
that it travels with the working tree.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
LIBRARY = HERE / "libmoe_b200_sampler.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-shared",
]


def sources() -> list[Path]:
    return sorted(Path(p) for p in glob.glob(str(CSRC / "*.cu")))


def _inputs() -> list[Path]:
    return sources() + sorted(Path(p) for p in glob.glob(str(CSRC / "*.cuh"))) + sorted(Path(p) for p in glob.glob(str(CSRC / "*.h"))) + \
        sorted(Path(p) for p in glob.glob(str(INCLUDE / "*.h")))


def up_to_date() -> bool:
    if not LIBRARY.exists():
        return False
    built = LIBRARY.stat().st_mtime
    return all(p.stat().st_mtime <= built for p in _inputs())


def _stdcxx_link_flags() -> list[str]:
    # Some compiler drivers only find the static libstdc++; a second copy of the
    # C++ runtime inside a Python process clashes with the one already loaded.
    for candidate in sorted(glob.glob("/usr/lib/gcc/*/*/libstdc++.so")):
        return ["-L" + os.path.dirname(candidate)]
    return []


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and up_to_date():
        return LIBRARY
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    command = [nvcc, *NVCC_FLAGS, *_stdcxx_link_flags(), "-o", str(LIBRARY), *[str(s) for s in sources()]]
    if verbose:
        command[1:1] = ["-Xptxas", "-v"]
        print(" ".join(command))
    subprocess.run(command, check=True, cwd=str(HERE))
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
