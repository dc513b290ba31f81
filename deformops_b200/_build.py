"""Compile the CUDA sources under ``csrc/`` into ``_lib/libmsda_b200.so`` for sm_100a.

Plain ``nvcc`` (cross-compiles without a GPU); the library depends on nothing but the
CUDA runtime, which is linked statically.  The reference's counterpart is its JIT/AOT
loader ``sources/deformops/core/build.py:1116-1296``; here there is exactly one local
build and no download path.
"""

from __future__ import annotations

import concurrent.futures
import contextlib
import fcntl
import os
import pathlib
import shutil
import subprocess

__all__ = ["FLOORS_PATH", "LIB_PATH", "SOURCES", "TORCH_BINDING_PATH", "build_floors_library",
           "build_library", "build_torch_binding", "is_stale"]

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB_PATH = LIB_DIR / "libmsda_b200.so"
SOURCES = ["msda_forward.cu", "msda_backward.cu", "msda_abi.cu", "msda_static_scratch.cu",
           "msda_f64.cu"]
HEADERS = [CSRC / "msda_common.cuh", PKG.parent / "include" / "msda_b200.h"]
#: bench-only microbenchmarks of the hardware floors (csrc/floors/bench_floors.cu); never
#: loaded by the package itself
FLOORS_PATH = LIB_DIR / "libmsda_b200_floors.so"
#: native dispatcher registration for Python-free processes (see csrc/torch_binding.cpp)
TORCH_BINDING_PATH = LIB_DIR / "libmsda_b200_torch.so"

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


@contextlib.contextmanager
def _build_lock():
    """Exclusive lock between processes that may build at the same time (one rank per GPU all
    import the package at once): whoever comes second waits, then finds the library fresh."""
    LIB_DIR.mkdir(exist_ok=True)
    with open(LIB_DIR / ".build.lock", "w") as handle:
        fcntl.flock(handle, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(handle, fcntl.LOCK_UN)


def build_library(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Build the shared library if missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB_PATH
    with _build_lock():
        # another process may have finished the build while this one waited for the lock
        if not force and not is_stale():
            return LIB_PATH
        return _build_library_locked(verbose)


def _build_library_locked(verbose: bool) -> pathlib.Path:
    nvcc = _nvcc()
    # objects go to a directory of this process's own, the link to a name of its own: nothing a
    # concurrent loader could pick up half-written
    obj_dir = LIB_DIR / f"obj.{os.getpid()}"
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
    try:
        with concurrent.futures.ThreadPoolExecutor(max_workers=len(sources)) as pool:
            objects = list(pool.map(compile_one, sources))
        tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
        link = [nvcc, "-shared", "-o", str(tmp), *map(str, objects),
                "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        res = subprocess.run(link, capture_output=True, text=True, env=env)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, LIB_PATH)  # atomic: a concurrent loader never sees a half-written file
    finally:
        shutil.rmtree(obj_dir, ignore_errors=True)
    return LIB_PATH


def build_floors_library(force: bool = False) -> pathlib.Path:
    """Compile ``csrc/floors/bench_floors.cu`` into ``_lib/libmsda_b200_floors.so`` (one nvcc
    call; the benchmark loads it, the operator library never does)."""
    src = CSRC / "floors" / "bench_floors.cu"
    if not force and FLOORS_PATH.exists() and FLOORS_PATH.stat().st_mtime > src.stat().st_mtime:
        return FLOORS_PATH
    with _build_lock():
        if not force and FLOORS_PATH.exists() and FLOORS_PATH.stat().st_mtime > src.stat().st_mtime:
            return FLOORS_PATH
        tmp = FLOORS_PATH.with_suffix(f".so.tmp{os.getpid()}")
        res = subprocess.run([_nvcc(), *NVCC_FLAGS, "-shared", str(src), "-o", str(tmp)],
                             capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, FLOORS_PATH)
    return FLOORS_PATH


def build_torch_binding(force: bool = False) -> pathlib.Path:
    """Compile ``csrc/torch_binding.cpp`` against the installed torch into
    ``_lib/libmsda_b200_torch.so`` (links ``libmsda_b200.so`` next to it).  Needs a host C++
    compiler and the torch headers; the Python package itself never loads the result."""
    src = CSRC / "torch_binding.cpp"
    build_library()
    if (not force and TORCH_BINDING_PATH.exists()
            and TORCH_BINDING_PATH.stat().st_mtime > max(src.stat().st_mtime,
                                                         LIB_PATH.stat().st_mtime)):
        return TORCH_BINDING_PATH
    import torch
    from torch.utils import cpp_extension

    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no host C++ compiler found: cannot build the torch binding")
    torch_lib = pathlib.Path(torch.__file__).parent / "lib"
    tmp = TORCH_BINDING_PATH.with_suffix(".so.tmp")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", str(src),
           *[f"-I{p}" for p in cpp_extension.include_paths("cuda")],
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-o", str(tmp), f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
           "-lc10_cuda", f"-L{LIB_DIR}", "-lmsda_b200", "-Wl,-rpath,$ORIGIN",
           f"-Wl,-rpath,{torch_lib}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the torch binding failed:\n{res.stderr[-4000:]}")
    os.replace(tmp, TORCH_BINDING_PATH)
    return TORCH_BINDING_PATH


if __name__ == "__main__":
    import sys

    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_floors_library(force="--force" in sys.argv))
    if "--torch-binding" in sys.argv:
        print(build_torch_binding(force="--force" in sys.argv))
