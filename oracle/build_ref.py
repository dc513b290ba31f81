"""TEST INFRASTRUCTURE - compile the REFERENCE's own CUDA kernels into ``oracle/_ref/``.

The reference's MSDA kernels are a handful of headers plus one 25-line translation unit per
configuration; they compile with a single ``nvcc`` call against the torch headers, without
the reference's build system.  Sources are read where they lie in the reference checkout and
are never copied; only the resulting ``.so`` files (git-ignored) are written, under
``oracle/_ref/``:

    msda_fp32acc.so       the reference's production configuration (float32 accumulation)
    msda_half2atomic.so   its native 16-bit-atomics configuration

Flags follow ``sources/deformops/core/configs.py:48-66`` (``--use_fast_math``, C++20, the
half-operator undefines; ``-DDEFORMOPS_NO_FP64`` as in its ahead-of-time build for the
16-bit configuration only, so that the production one also runs in float64).  The
libraries are used by ``oracle/ref_cuda.py`` as the GPU-side parity oracle and speed bar.

``stage_package`` additionally places the reference's Python package, unmodified, under
``oracle/_ref/py/deformops`` (git-ignored like everything in ``oracle/_ref``), so that the
machine that runs the GPU tests can import it: the tests that drive these kernels through the
reference's own registry, layer and Hugging Face replacements, and the benchmark's reference
arm (the reference's eager CPU path and its Triton kernels), need the real package.

The reference checkout is found through ``--reference``, the environment variable
``DEFORMOPS_REFERENCE``, or a directory ``reference`` next to this repository.

    python oracle/build_ref.py [--reference /path/to/reference]
"""

from __future__ import annotations

import argparse
import os
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref"
PACKAGE_DIR = OUT / "py"


def default_reference() -> "pathlib.Path | None":
    """The reference checkout: ``$DEFORMOPS_REFERENCE`` or ``../reference`` beside the repo."""
    env = os.environ.get("DEFORMOPS_REFERENCE")
    for cand in ([pathlib.Path(env)] if env else []) + [HERE.parent.parent / "reference"]:
        if (cand / "sources" / "deformops").is_dir():
            return cand
    return None


def stage_package(reference: pathlib.Path) -> pathlib.Path:
    """Copy ``sources/deformops`` of the checkout to ``oracle/_ref/py/deformops`` (replacing an
    older copy) and return the directory to put on ``sys.path``."""
    src = reference / "sources" / "deformops"
    if not src.is_dir():
        raise FileNotFoundError(src)
    dst = PACKAGE_DIR / "deformops"
    if dst.exists():
        shutil.rmtree(dst)
    PACKAGE_DIR.mkdir(parents=True, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    # the package reads its version from the checkout's VERSION file, two directories above
    # itself, when it is not an installed distribution
    version = reference / "VERSION"
    if version.is_file():
        shutil.copyfile(version, PACKAGE_DIR.parent / "VERSION")
    return PACKAGE_DIR


def staged_package() -> "pathlib.Path | None":
    """``oracle/_ref/py`` if the reference package has been staged there, else None."""
    return PACKAGE_DIR if (PACKAGE_DIR / "deformops" / "__init__.py").exists() else None

UNITS = {
    "msda_fp32acc": "sources/deformops/backends/cuda/msda_fp32acc.cu",
    "msda_half2atomic": "sources/deformops/backends/cuda/experimental/msda_half2atomic.cu",
}
#: the production configuration is built WITH double precision (the float64 parity test runs
#: the reference's kernels in float64); the 16-bit-atomics one never sees float64
NO_FP64 = {"msda_half2atomic": ["-DDEFORMOPS_NO_FP64"]}


def build(reference: pathlib.Path, force: bool = False) -> list[pathlib.Path]:
    import torch
    from torch.utils import cpp_extension

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    include = reference / "sources/deformops/backends/cuda/include"
    torch_lib = pathlib.Path(torch.__file__).parent / "lib"
    OUT.mkdir(exist_ok=True)
    built = []
    for name, rel in UNITS.items():
        src = reference / rel
        target = OUT / f"{name}.so"
        if not src.exists():
            raise FileNotFoundError(src)
        if target.exists() and not force and target.stat().st_mtime > src.stat().st_mtime:
            built.append(target)
            continue
        cmd = [
            nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++20",
            "--use_fast_math", "-DUSE_CUDA", "-DTORCH_TARGET_VERSION=0x020B000000000000",
            *NO_FP64.get(name, []), "-U__CUDA_NO_HALF_OPERATORS__",
            "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
            "-Xcompiler", "-fPIC", "-shared", f"-I{include}",
            *[f"-I{p}" for p in cpp_extension.include_paths("cuda")],
            str(src), "-o", str(target),
            f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10",
            "-Xlinker", f"-rpath={torch_lib}",
        ]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stderr[-4000:]}")
        built.append(target)
    return built


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    ref = pathlib.Path(args.reference) if args.reference else default_reference()
    if ref is None or not ref.exists():
        print("no reference checkout (--reference / DEFORMOPS_REFERENCE): nothing built",
              file=sys.stderr)
        return
    for path in build(ref, args.force):
        print(f"{path}  {path.stat().st_size / 1e6:.1f} MB")
    print(f"staged {stage_package(ref) / 'deformops'}")


if __name__ == "__main__":
    main()
