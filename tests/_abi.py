"""Test helper: call ``libmsda_b200.so`` through its C ABI with torch-allocated CUDA buffers."""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from deformops_b200._loader import load_library
from deformops_b200.ops import DTYPE_CODES


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def dev(x, dtype=None, device="cuda"):
    t = torch.as_tensor(np.ascontiguousarray(x)) if isinstance(x, np.ndarray) else x
    if dtype is not None and t.is_floating_point():
        t = t.to(dtype)
    return t.to(device).contiguous()


def dims(value, loc):
    B, S, G, D = value.shape
    _, Q, _, L, K, _ = loc.shape
    return B, S, G, D, Q, L, K


def abi_forward(value, shapes, starts, loc, attn, *, softmax=False, stream=None):
    shim = load_library()
    B, S, G, D, Q, L, K = dims(value, loc)
    out = torch.full((B, Q, G * D), float("nan"), dtype=value.dtype, device=value.device)
    s = torch.cuda.current_stream().cuda_stream if stream is None else stream
    st = shim.forward(_p(value), _p(shapes), _p(starts), _p(loc), _p(attn), _p(out), B, S, G, D,
                      Q, L, K, DTYPE_CODES[value.dtype], int(softmax), value.device.index,
                      ctypes.c_void_p(s))
    assert st == 0, shim.last_error()
    return out


def abi_backward(value, shapes, starts, loc, attn, grad_out, *, softmax=False, zero=True,
                 scratch=True, scratch_adds=0):
    """``scratch=True`` hands the call the scratch the product path uses for 16-bit dtypes
    (scaled float16 accumulation); ``scratch=False`` adds straight into grad_value in its own
    type.  ``scratch_adds`` is accepted by the ABI and has no effect."""
    shim = load_library()
    B, S, G, D, Q, L, K = dims(value, loc)
    # poison the outputs: the call must overwrite every element
    grad_value = torch.full_like(value, float("nan")) if zero else torch.zeros_like(value)
    grad_loc = torch.full_like(loc, float("nan"))
    grad_attn = torch.full_like(attn, float("nan"))
    nbytes = shim.scratch_bytes(B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype]) if (scratch and zero) else 0
    # poisoned as well (0xFFFF is a NaN in both 16-bit types): the call must clear what it uses
    buf = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=value.device) if nbytes else None
    s = torch.cuda.current_stream().cuda_stream
    st = shim.backward(_p(value), _p(shapes), _p(starts), _p(loc), _p(attn), _p(grad_out),
                       _p(grad_value), _p(grad_loc), _p(grad_attn), _p(buf), nbytes, scratch_adds,
                       B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype], int(softmax), int(zero),
                       value.device.index, ctypes.c_void_p(s))
    assert st == 0, shim.last_error()
    return grad_value, grad_loc, grad_attn


def abi_forward_offsets(value, shapes, starts, ref, offsets, attn, *, softmax=False):
    shim = load_library()
    B, S, G, D, Q, L, K = dims(value, offsets)
    out = torch.full((B, Q, G * D), float("nan"), dtype=value.dtype, device=value.device)
    s = torch.cuda.current_stream().cuda_stream
    st = shim.forward_offsets(_p(value), _p(shapes), _p(starts), _p(ref), ref.shape[-1],
                              _p(offsets), DTYPE_CODES[offsets.dtype], _p(attn), _p(out), B, S, G,
                              D, Q, L, K, DTYPE_CODES[value.dtype], int(softmax),
                              value.device.index, ctypes.c_void_p(s))
    assert st == 0, shim.last_error()
    return out


def abi_backward_offsets(value, shapes, starts, ref, offsets, attn, grad_out, *, softmax=False):
    shim = load_library()
    B, S, G, D, Q, L, K = dims(value, offsets)
    grad_value = torch.full_like(value, float("nan"))
    grad_offsets = torch.full_like(offsets, float("nan"))
    grad_attn = torch.full_like(attn, float("nan"))
    nbytes = shim.scratch_bytes(B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype])
    buf = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=value.device) if nbytes else None
    s = torch.cuda.current_stream().cuda_stream
    st = shim.backward_offsets(_p(value), _p(shapes), _p(starts), _p(ref), ref.shape[-1],
                               _p(offsets), DTYPE_CODES[offsets.dtype], _p(attn), _p(grad_out),
                               _p(grad_value), _p(grad_offsets), _p(grad_attn), _p(buf), nbytes, 0,
                               B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype], int(softmax), 1,
                               value.device.index, ctypes.c_void_p(s))
    assert st == 0, shim.last_error()
    return grad_value, grad_offsets, grad_attn


def to_np(t):
    return t.detach().float().cpu().numpy().astype(np.float64)
