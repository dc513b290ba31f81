"""TEST INFRASTRUCTURE - Python face of the C oracle in ``msda_oracle.c``.

Loads ``oracle/_build/libmsda_oracle.so`` (built by ``make -C oracle``, which
:func:`build` runs on demand) and exposes forward/backward on numpy arrays or
torch CPU tensors.  The arithmetic follows the reference files cited at the top
of ``msda_oracle_body.inc``.  Only tests, the smoke check and the benchmark's
CPU-baseline leg may import this module; the product path never does.
"""

from __future__ import annotations

import ctypes
import pathlib
import subprocess
import threading

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libmsda_oracle.so"
_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


def build(force: bool = False) -> pathlib.Path:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    sources = [_HERE / "msda_oracle.c", _HERE / "msda_oracle_body.inc"]
    stale = not _LIB_PATH.exists() or any(
        s.stat().st_mtime > _LIB_PATH.stat().st_mtime for s in sources
    )
    if force or stale:
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, capture_output=True)
    return _LIB_PATH


def _load() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            lib = ctypes.CDLL(str(build()))
            i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
            for suffix in ("f32", "f64"):
                fwd = getattr(lib, f"msda_oracle_forward_{suffix}")
                fwd.restype = None
                fwd.argtypes = [vp] * 6 + [i64] * 7 + [ci]
                bwd = getattr(lib, f"msda_oracle_backward_{suffix}")
                bwd.restype = None
                bwd.argtypes = [vp] * 9 + [i64] * 7 + [ci]
            lib.msda_oracle_max_points.restype = ci
            _lib = lib
    return _lib


def _as_np(x, dtype) -> np.ndarray:
    if hasattr(x, "detach"):  # torch tensor
        x = x.detach().cpu()
        if x.dtype.is_floating_point and x.dtype.itemsize < 4:
            x = x.float()  # bf16/fp16 -> fp32 is exact
        x = x.numpy()
    return np.ascontiguousarray(x, dtype=dtype)


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def _dims(value, loc):
    B, S, G, D = value.shape
    _, Q, _, L, K, two = loc.shape
    if two != 2:
        raise ValueError("sampling_locations must end in an (x, y) pair")
    return B, S, G, D, Q, L, K


def forward(value, spatial_shapes, level_start_index, loc, attn, *, softmax=False,
            precision="f64") -> np.ndarray:
    """Oracle forward; returns ``(B, Q, G*D)`` as float32 or float64 numpy."""
    lib = _load()
    real = np.float64 if precision == "f64" else np.float32
    value, loc, attn = _as_np(value, real), _as_np(loc, real), _as_np(attn, real)
    shapes = _as_np(spatial_shapes, np.int64)
    starts = _as_np(level_start_index, np.int64)
    B, S, G, D, Q, L, K = _dims(value, loc)
    if L * K > lib.msda_oracle_max_points():
        raise ValueError("L*K exceeds the oracle's softmax scratch")
    attn = attn.reshape(B, Q, G, L * K)
    out = np.empty((B, Q, G * D), dtype=real)
    fn = getattr(lib, f"msda_oracle_forward_{precision}")
    fn(_ptr(value), _ptr(shapes), _ptr(starts), _ptr(loc), _ptr(attn), _ptr(out),
       B, S, G, D, Q, L, K, int(bool(softmax)))
    return out


def backward(value, spatial_shapes, level_start_index, loc, attn, grad_out, *,
             softmax=False, precision="f64"):
    """Oracle backward; returns ``(grad_value, grad_loc, grad_attn)``.

    ``grad_attn`` has the shape of the ``attn`` argument (4-D or 5-D).
    """
    lib = _load()
    real = np.float64 if precision == "f64" else np.float32
    value, loc, attn = _as_np(value, real), _as_np(loc, real), _as_np(attn, real)
    grad_out = _as_np(grad_out, real)
    shapes = _as_np(spatial_shapes, np.int64)
    starts = _as_np(level_start_index, np.int64)
    B, S, G, D, Q, L, K = _dims(value, loc)
    if L * K > lib.msda_oracle_max_points():
        raise ValueError("L*K exceeds the oracle's softmax scratch")
    attn_shape = attn.shape
    attn = attn.reshape(B, Q, G, L * K)
    grad_value = np.empty_like(value)
    grad_loc = np.empty_like(loc)
    grad_attn = np.empty_like(attn)
    fn = getattr(lib, f"msda_oracle_backward_{precision}")
    fn(_ptr(value), _ptr(shapes), _ptr(starts), _ptr(loc), _ptr(attn), _ptr(grad_out),
       _ptr(grad_value), _ptr(grad_loc), _ptr(grad_attn), B, S, G, D, Q, L, K,
       int(bool(softmax)))
    return grad_value, grad_loc, grad_attn.reshape(attn_shape)
