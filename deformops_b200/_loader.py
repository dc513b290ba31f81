"""Loads ``libmsda_b200.so`` (the C ABI of ``include/msda_b200.h``) through ctypes.

Plays the role of the reference's kernel-library loader
(``lazy_extension`` / ``define_library``, ``sources/deformops/core/build.py:75-137``
and ``:1116-1296``) reduced to what this build needs: one local library, loaded once
per process under a lock, a failed load is not memoised, and a forked child gets a fresh
lock.  There is no CPU path behind it: if the library cannot be loaded the call fails
with :class:`KernelUnavailableError`.
"""

from __future__ import annotations

import ctypes
import os
import threading

from ._build import LIB_PATH, build_library, is_stale
from .core.errors import KernelBuildError, KernelUnavailableError

__all__ = ["ABI_VERSION", "Shim", "library_path", "load_library", "loaded"]

ABI_VERSION = 5

_lock = threading.Lock()
_shim: "Shim | None" = None


def _reset_lock_in_child() -> None:
    global _lock
    _lock = threading.Lock()


os.register_at_fork(after_in_child=_reset_lock_in_child)

_i64, _vp, _int = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int


class Shim:
    """Typed handles on the exported functions of the library."""

    #: every symbol ``include/msda_b200.h`` declares
    SYMBOLS = ("msda_b200_abi_version", "msda_b200_last_error", "msda_b200_forward",
               "msda_b200_backward", "msda_b200_backward_scratch_bytes",
               "msda_b200_forward_offsets", "msda_b200_backward_offsets",
               "msda_b200_backward_static_scratch", "msda_b200_launch_geometry")

    def __init__(self, path: str):
        self.path = path
        self.lib = ctypes.CDLL(path)
        missing = [s for s in self.SYMBOLS if not hasattr(self.lib, s)]
        if missing:
            raise KernelUnavailableError(f"{path} does not export {missing}")
        self.lib.msda_b200_abi_version.restype = _int
        self.lib.msda_b200_abi_version.argtypes = []
        self.lib.msda_b200_last_error.restype = ctypes.c_char_p
        self.lib.msda_b200_last_error.argtypes = []
        self.forward = self.lib.msda_b200_forward
        self.forward.restype = _int
        self.forward.argtypes = [_vp] * 6 + [_i64] * 7 + [_int, _int, _int, _vp]
        self.backward = self.lib.msda_b200_backward
        self.backward.restype = _int
        self.backward.argtypes = ([_vp] * 10 + [_i64, _i64] + [_i64] * 7
                                  + [_int, _int, _int, _int, _vp])
        self.scratch_bytes = self.lib.msda_b200_backward_scratch_bytes
        self.scratch_bytes.restype = _i64
        self.scratch_bytes.argtypes = [_i64] * 7 + [_int]
        self.forward_offsets = self.lib.msda_b200_forward_offsets
        self.forward_offsets.restype = _int
        self.forward_offsets.argtypes = ([_vp] * 4 + [_int, _vp, _int, _vp, _vp] + [_i64] * 7
                                         + [_int, _int, _int, _vp])
        self.backward_offsets = self.lib.msda_b200_backward_offsets
        self.backward_offsets.restype = _int
        self.backward_offsets.argtypes = ([_vp] * 4 + [_int, _vp, _int] + [_vp] * 6
                                          + [_i64, _i64] + [_i64] * 7
                                          + [_int, _int, _int, _int, _vp])
        self.backward_static_scratch = self.lib.msda_b200_backward_static_scratch
        self.backward_static_scratch.restype = _int
        self.backward_static_scratch.argtypes = ([_vp] * 9 + [_i64] + [_i64] * 7
                                                 + [_int, _int, _int, _vp])
        self.launch_geometry = self.lib.msda_b200_launch_geometry
        self.launch_geometry.restype = _int
        self.launch_geometry.argtypes = [_i64] * 6 + [_int, _int, ctypes.POINTER(_i64),
                                         ctypes.POINTER(_int), ctypes.POINTER(_i64),
                                         ctypes.POINTER(_i64)]
        got = self.lib.msda_b200_abi_version()
        if got != ABI_VERSION:
            raise KernelUnavailableError(
                f"{path} has ABI version {got}, this package needs {ABI_VERSION}: rebuild it")

    def last_error(self) -> str:
        return self.lib.msda_b200_last_error().decode("utf-8", "replace")


def library_path() -> str:
    return os.environ.get("DEFORMOPS_B200_LIBRARY", str(LIB_PATH))


def loaded() -> bool:
    return _shim is not None


def load_library(*, compile: "bool | None" = None) -> Shim:
    """Load the kernel library once per process and return its :class:`Shim`.

    ``compile`` (default: environment ``DEFORMOPS_B200_COMPILE``, on unless it is ``0``)
    allows building the library with ``nvcc`` when it is missing or older than its sources.
    """
    global _shim
    if _shim is not None:
        return _shim
    with _lock:
        if _shim is not None:
            return _shim
        path = library_path()
        if compile is None:
            compile = os.environ.get("DEFORMOPS_B200_COMPILE", "1") != "0"
        if path == str(LIB_PATH) and compile and is_stale():
            try:
                build_library()
            except Exception as exc:  # noqa: BLE001 - surfaced as a typed error
                if not LIB_PATH.exists():
                    raise KernelBuildError(f"cannot build {LIB_PATH}: {exc}") from exc
        if not os.path.exists(path):
            raise KernelUnavailableError(
                f"kernel library {path} is missing; build it with "
                "`python -m deformops_b200._build` (needs nvcc). There is no CPU path.")
        try:
            _shim = Shim(path)
        except OSError as exc:
            raise KernelUnavailableError(f"cannot load {path}: {exc}") from exc
        return _shim
