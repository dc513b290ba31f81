"""float64 on the GPU: the configuration ``torch.autograd.gradcheck`` needs.

The reference's CUDA operator takes float64 values with float64 locations
(``sources/deformops/backends/cuda/include/msda_launch.cuh:54-61``) and its tests differentiate
it numerically.  Here the float64 kernels are compared with the float64 outputs the reference
produced for the fixtures (to 1e-12) and then put through ``gradcheck`` themselves.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests._abi import abi_backward, abi_forward, dev
from tests._golden import FULL_CASES, METHODS, attn_for, load, rel_err

pytestmark = pytest.mark.gpu


def _np(t):
    """float64 all the way (the shared helper goes through float32)."""
    return t.detach().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("method", METHODS)
@pytest.mark.parametrize("name", FULL_CASES)
def test_float64_matches_reference_fixtures(name, method):
    """Fixtures hold the reference's float64 results; no channel padding is needed here
    (any head size), so ``boundary`` runs with its single channel."""
    c = load(name)
    sm = method == "softmax"
    f64 = torch.float64
    v, a, go = dev(c["value"], f64), dev(attn_for(c, method), f64), dev(c["grad_out"], f64)
    l = dev(c["loc"], f64)
    sh, st = dev(c["spatial_shapes"]), dev(c["level_start_index"])
    out = abi_forward(v, sh, st, l, a, softmax=sm)
    gv, gl, ga = abi_backward(v, sh, st, l, a, go, softmax=sm)
    torch.cuda.synchronize()
    assert gl.dtype == f64 and out.dtype == f64
    for got, key in ((out, "out_eager"), (gv, "grad_value"), (gl, "grad_loc"), (ga, "grad_attn")):
        assert rel_err(_np(got), c[f"{method}_{key}"]) <= 1e-12, (name, method, key)


def _small(seed=0, B=1, Q=5, G=2, D=3, K=2, levels=((4, 5), (2, 3))):
    g = torch.Generator().manual_seed(seed)
    shapes = torch.tensor(levels, dtype=torch.int64)
    sizes = shapes[:, 0] * shapes[:, 1]
    starts = torch.cumsum(sizes, 0) - sizes
    S, L = int(sizes.sum()), len(levels)
    value = torch.randn((B, S, G, D), generator=g, dtype=torch.float64)
    # keep pixels away from integers: the location gradient jumps there
    loc = torch.rand((B, Q, G, L, K, 2), generator=g, dtype=torch.float64) * 0.9 + 0.05
    wh = shapes.flip(-1).to(torch.float64)[None, None, None, :, None, :]
    pix = loc * wh - 0.5
    loc = torch.where((pix - pix.round()).abs() < 0.05, loc + 0.1 / wh, loc)
    attn = torch.randn((B, Q, G, L * K), generator=g, dtype=torch.float64)
    return [t.cuda() for t in (value, shapes, starts, loc, attn)]


@pytest.mark.parametrize("method", METHODS)
def test_gradcheck(method):
    from deformops_b200 import msda

    value, shapes, starts, loc, attn = _small()
    value.requires_grad_()
    loc.requires_grad_()
    attn.requires_grad_()
    fn = lambda v, l, a: msda(v, shapes, starts, l, a, method=method)  # noqa: E731
    assert torch.autograd.gradcheck(fn, (value, loc, attn), eps=1e-6, atol=1e-7, rtol=1e-5,
                                    nondet_tol=1e-12)


def test_float64_and_float32_agree():
    from deformops_b200 import msda

    value, shapes, starts, loc, attn = _small(3, B=2, Q=40, G=4, D=8, K=4)
    out64 = msda(value, shapes, starts, loc, attn, softmax=True)
    out32 = msda(value.float(), shapes, starts, loc.float(), attn.float(), softmax=True)
    assert out64.dtype == torch.float64
    assert rel_err(_np(out32), _np(out64)) <= 1e-5


def test_offsets_functional_takes_float64_through_the_location_kernels():
    from deformops_b200 import msda_from_offsets

    value, shapes, starts, loc, attn = _small(4)
    B, Q, G, L, K, _ = loc.shape
    ref = torch.rand((B, Q, L, 2), dtype=torch.float64, device="cuda")
    wh = shapes.flip(-1).to(torch.float64)[None, None, None, :, None, :]
    offsets = ((loc - ref[:, :, None, :, None, :]) * wh).requires_grad_()
    out = msda_from_offsets(value, shapes, starts, ref, offsets, attn)
    assert out.dtype == torch.float64
    (g,) = torch.autograd.grad(out.sum(), [offsets])
    assert g.dtype == torch.float64 and torch.isfinite(g).all()


def test_float64_rejected_by_the_fused_entry_points():
    import ctypes

    from deformops_b200._loader import load_library

    shim = load_library()
    z = ctypes.c_void_p(0)
    st = shim.forward_offsets(z, z, z, z, 2, z, 0, z, z, 1, 1, 1, 1, 1, 1, 1, 3, 0, 0, z)
    assert st == -2 and "float64" in shim.last_error()
