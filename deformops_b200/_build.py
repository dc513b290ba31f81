"""Compile the CUDA sources under ``csrc/`` into ``_lib/libmsda_b200.so`` for sm_100a.

Plain ``nvcc`` (cross-compiles without a GPU); the library depends on nothing but the
CUDA runtime, which is linked statically.  The reference's counterpart is its JIT/AOT
loader ``sources/deformops/core/build.py:1116-1296``; here there is exactly one local
build and no download path.
"""

from __future__ import annotations

import concurrent.futures
import os
import pathlib
import shutil
import subprocess

__all__ = ["LIB_PATH", "SOURCES", "build_library", "is_stale"]

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB_PATH = LIB_DIR / "libmsda_b200.so"
SOURCES = ["msda_forward.cu", "msda_backward.cu", "msda_abi.cu", "msda_static_scratch.cu",
           "msda_l2_window.cu", "msda_backward_region.cu", "msda_f64.cu"]
HEADERS = [CSRC / "msda_common.cuh", PKG.parent / "include" / "msda_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _existing_sources() -> list[pathlib.Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not pathlib.Path(cand).exists():
        raise RuntimeError("nvcc not found: cannot build libmsda_b200.so")
    return cand


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(f.stat().st_mtime > built for f in [*_existing_sources(), *HEADERS])


def build_library(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Build the shared library if missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = _nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    env = dict(os.environ)

    def compile_one(src: pathlib.Path) -> pathlib.Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr)
        return obj

    sources = _existing_sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(sources)) as pool:
        objects = list(pool.map(compile_one, sources))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-o", str(tmp), *map(str, objects),
            "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    res = subprocess.run(link, capture_output=True, text=True, env=env)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB_PATH)  # atomic: a concurrent loader never sees a half-written file
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
