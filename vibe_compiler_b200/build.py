"""Builds libwb200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Usage: ``python -m vibe_compiler_b200.build [--force]``. nvcc cross-compiles for sm_100a, so the
build needs no GPU. Objects go to ``vibe_compiler_b200/_build``; the shared library is written next
to this file so that it travels with a source snapshot.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
BUILD_DIR = PACKAGE_DIR / "_build"
LIBRARY = PACKAGE_DIR / "libwb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; libwb200.so cannot be built")
    return nvcc


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [PACKAGE_DIR.parent / "include" / "wb200.h"]
    return max(h.stat().st_mtime for h in headers)


def _compile(source: Path, header_mtime: float, force: bool) -> Path:
    obj = BUILD_DIR / (source.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime > max(source.stat().st_mtime, header_mtime):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(source), "-o", str(obj)]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source.name}:\n{result.stdout}\n{result.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_mtime = _newest_header_mtime()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objects = list(pool.map(lambda s: _compile(s, header_mtime, force), sources))
    newest_obj = max(o.stat().st_mtime for o in objects)
    if force or not LIBRARY.exists() or LIBRARY.stat().st_mtime < newest_obj:
        cmd = [_nvcc(), "-shared", "-o", str(LIBRARY), *map(str, objects), "-gencode", "arch=compute_100a,code=sm_100a"]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    if verbose:
        print(f"built {LIBRARY}")
    return LIBRARY


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
