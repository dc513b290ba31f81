"""The allocation-free backward entry point, ``msda_b200_backward_static_scratch``.

It exists for hosts that cannot hand the library a scratch buffer when they call it - a
serving or training runtime that split up all device memory at start-up and forbids
``cudaMalloc`` afterwards, a plugin running inside another framework's step, a C program with
no caching allocator - and keeps the float16 image it accumulates grad_value in inside a fixed
32 MiB array of the library instead.  The test calls it through the C ABI twice in a row, with
different inputs, and checks both results against the ordinary entry point (caller-owned
scratch) and against the float64 CPU oracle: the second call must not see anything the first
one left in the shared array.  This file is collected
last so that a failure here cannot hide the other tests in a run that stops at the first one.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from tests._abi import abi_backward, dev, dims, to_np

pytestmark = pytest.mark.gpu

# max|a-b| / max|b| of grad_value, against the sibling entry point and against the oracle: the
# 16-bit bar of the parity tests.  The two entry points run the same kernels and differ only
# by the order of the float16 additions.
TOL_GRAD_VALUE = {torch.float16: 1e-2, torch.bfloat16: 1e-2}

SCRATCH_ADDS = 0   # accepted by the ABI, no effect


def _static_backward(value, shapes, starts, loc, attn, grad_out, *, softmax=False):
    from deformops_b200._loader import load_library
    from deformops_b200.ops import DTYPE_CODES

    shim = load_library()
    B, S, G, D, Q, L, K = dims(value, loc)
    grad_value = torch.full_like(value, float("nan"))
    grad_loc = torch.full_like(loc, float("nan"))
    grad_attn = torch.full_like(attn, float("nan"))
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    status = shim.backward_static_scratch(
        p(value), p(shapes), p(starts), p(loc), p(attn), p(grad_out), p(grad_value), p(grad_loc),
        p(grad_attn), SCRATCH_ADDS, B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype], int(softmax),
        value.device.index, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return status, shim.last_error(), (grad_value, grad_loc, grad_attn)


def _workload(first_sample, dtype):
    from deformops_b200.workloads import make_workload

    # 2 x 5376 x 8 x 32 = 2.75 M elements, 5.5 MB of the 32 MiB array
    w = make_workload("cfg1_m2f_512_bf16", batch=2, first_sample=first_sample)
    return (dev(w.value, dtype), dev(w.spatial_shapes), dev(w.level_start_index),
            dev(w.sampling_locations, torch.float32), dev(w.attention_weights, dtype),
            dev(w.grad_output, dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_two_calls_in_a_row_match_the_caller_scratch_entry_point(dtype):
    for call, first_sample in enumerate((0, 40)):          # different inputs each call
        args = _workload(first_sample, dtype)
        status, message, (gv, gl, ga) = _static_backward(*args)
        assert status == 0, message
        e_gv, e_gl, e_ga = abi_backward(*args, scratch_adds=SCRATCH_ADDS)   # caller-owned scratch
        torch.cuda.synchronize()
        assert torch.equal(gl, e_gl), f"grad_loc differs on call {call}"
        assert torch.equal(ga, e_ga), f"grad_attn differs on call {call}"
        assert torch.isfinite(gv).all()
        err = (gv.float() - e_gv.float()).abs().max() / e_gv.float().abs().max()
        assert err.item() <= TOL_GRAD_VALUE[dtype], f"grad_value off by {err.item():.3e} on call {call}"
        # and against the truth: float64 oracle on the same (rounded) inputs
        from oracle import msda_oracle

        v, shapes, starts, loc, attn, go = args
        o_gv, _, _ = msda_oracle.backward(v.cpu(), shapes.cpu(), starts.cpu(), loc.cpu(),
                                          attn.cpu(), go.cpu())
        o_err = np.abs(to_np(gv) - o_gv).max() / np.abs(o_gv).max()
        assert o_err <= TOL_GRAD_VALUE[dtype], f"grad_value {o_err:.3e} off the oracle on call {call}"


def test_float32_needs_no_scratch_and_softmax_works():
    args = _workload(3, torch.float32)
    status, message, (gv, gl, ga) = _static_backward(*args, softmax=True)
    assert status == 0, message
    e_gv, e_gl, e_ga = abi_backward(*args, softmax=True, scratch_adds=SCRATCH_ADDS)
    torch.cuda.synchronize()
    assert torch.equal(gl, e_gl) and torch.equal(ga, e_ga)
    torch.testing.assert_close(gv, e_gv, rtol=1e-4, atol=1e-5)


def test_shapes_beyond_the_built_in_array_are_refused():
    from deformops_b200.workloads import make_workload

    w = make_workload("cfg2_m2f_1024_bf16", batch=4)       # 4 x 21504 x 256 = 22 M elements
    args = (dev(w.value), dev(w.spatial_shapes), dev(w.level_start_index),
            dev(w.sampling_locations), dev(w.attention_weights), dev(w.grad_output))
    status, message, _ = _static_backward(*args)
    assert status == -2
    assert "exceed the built-in scratch" in message.replace("\n", " ") and "msda_b200_backward" in message
