"""The boundary is usable from plain C: the header is valid C99 / C++11 and a C program can
load the library, read its version and get a status code plus message back (no GPU needed:
argument errors are detected before any CUDA call)."""

from __future__ import annotations

import pathlib
import shutil
import subprocess

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "msda_b200.h"

C_PROGRAM = r"""
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>
#include "msda_b200.h"

typedef int (*version_fn)(void);
typedef const char *(*error_fn)(void);
typedef int (*forward_fn)(const void *, const int64_t *, const int64_t *, const float *,
                          const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t,
                          int64_t, int64_t, int, int, int, void *);
typedef int64_t (*scratch_fn)(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int);

int main(int argc, char **argv) {
    void *lib = dlopen(argv[1], RTLD_NOW);
    if (!lib) { fprintf(stderr, "%s\n", dlerror()); return 2; }
    version_fn version = (version_fn)dlsym(lib, "msda_b200_abi_version");
    error_fn last_error = (error_fn)dlsym(lib, "msda_b200_last_error");
    forward_fn forward = (forward_fn)dlsym(lib, "msda_b200_forward");
    scratch_fn scratch = (scratch_fn)dlsym(lib, "msda_b200_backward_scratch_bytes");
    if (!version || !last_error || !forward || !scratch) return 3;
    if (version() != MSDA_B200_ABI_VERSION) return 4;
    if (scratch(4, 21504, 8, 32, 21504, 3, 4, MSDA_B200_BF16) != 256 + 2 * 4LL * (21504 * 8 * 32 + 3 * 344064)) return 5;
    if (scratch(4, 21504, 8, 32, 21504, 3, 4, MSDA_B200_F32) != 0) return 6;
    /* dtype 9 does not exist: refused before anything touches the GPU */
    int st = forward(0, 0, 0, 0, 0, 0, 1, 1, 1, 8, 1, 1, 1, 9, 0, 0, 0);
    if (st != MSDA_B200_INVALID_ARGUMENT) return 7;
    if (strstr(last_error(), "dtype") == 0) return 8;
    /* head dimension that is not a multiple of the 16-byte vector */
    st = forward(0, 0, 0, 0, 0, 0, 1, 1, 1, 7, 1, 1, 1, MSDA_B200_BF16, 0, 0, 0);
    if (st != MSDA_B200_UNSUPPORTED) return 9;
    printf("abi %d ok\n", version());
    return 0;
}
"""


@pytest.mark.parametrize("compiler,flags", [
    ("gcc", ["-std=c99", "-pedantic", "-x", "c"]),
    ("g++", ["-std=c++11", "-x", "c++"]),
])
def test_header_is_valid_c_and_cxx(compiler, flags):
    if shutil.which(compiler) is None:
        pytest.skip(f"{compiler} not installed")
    done = subprocess.run([compiler, *flags, "-Wall", "-Wextra", "-Werror", "-fsyntax-only",
                           str(HEADER)], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr


def test_c_program_calls_the_library(tmp_path):
    if shutil.which("gcc") is None:
        pytest.skip("gcc not installed")
    from deformops_b200._build import LIB_PATH, build_library

    build_library()
    src = tmp_path / "caller.c"
    src.write_text(C_PROGRAM)
    exe = tmp_path / "caller"
    done = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{HEADER.parent}", str(src),
                           "-o", str(exe), "-ldl"], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    run = subprocess.run([str(exe), str(LIB_PATH)], capture_output=True, text=True)
    assert run.returncode == 0 and "ok" in run.stdout, (run.returncode, run.stderr)


def test_native_torch_binding_defines_the_same_schemas(tmp_path):
    """``libmsda_b200_torch.so`` loaded into a process that never imports the package defines
    the four private operators with exactly the schemas ``ops.py`` defines."""
    import subprocess
    import sys

    if shutil.which("g++") is None:
        pytest.skip("g++ not installed")
    from deformops_b200._build import build_torch_binding
    from deformops_b200.ops import _BACKWARD_SCHEMA, _FORWARD_SCHEMA, PRIVATE_OPS

    binding = build_torch_binding()
    script = (
        "import sys, torch\n"
        f"torch.ops.load_library(r'{binding}')\n"
        f"for name in {PRIVATE_OPS!r}:\n"
        "    print(name, '|', str(getattr(torch.ops.deformops_b200, name).default._schema))\n"
        "assert 'deformops_b200' not in sys.modules\n")
    done = subprocess.run([sys.executable, "-c", script], cwd=tmp_path, capture_output=True,
                          text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    seen = dict(line.split(" | ") for line in done.stdout.strip().splitlines())
    for name in PRIVATE_OPS:
        want = _FORWARD_SCHEMA if name.endswith("forward") else _BACKWARD_SCHEMA
        assert seen[name] == f"deformops_b200::{name}{want}", (seen[name], want)
