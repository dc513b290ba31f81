"""GPU parity of the entry points that fuse the layer's location arithmetic
(``msda_b200_forward_offsets`` / ``msda_b200_backward_offsets`` and the ops above them).

The expectation is built the way the reference's layers compute it
(``sources/deformops/nn/msda.py:222-239``): locations in torch float32 from reference points and
offsets, then the pinned oracle on those locations, then the chain rule back to the offsets.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import msda_oracle as orc
from tests._abi import (abi_backward, abi_backward_offsets, abi_forward, abi_forward_offsets, dev,
                        to_np)
from tests._golden import rel_err
from tests.test_gpu_parity import _stable_points

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (1e-5, 1e-4), torch.float16: (1e-2, 1e-2), torch.bfloat16: (1e-2, 2e-2)}
LEVELS = [(12, 17), (6, 9), (3, 5)]


def _case(seed, coords, *, B=2, Q=75, G=4, D=16, K=4, levels=LEVELS):
    rng = np.random.default_rng(seed)
    shapes = np.asarray(levels, dtype=np.int64)
    starts = np.concatenate([[0], np.cumsum(shapes[:, 0] * shapes[:, 1])[:-1]]).astype(np.int64)
    S, L = int((shapes[:, 0] * shapes[:, 1]).sum()), len(levels)
    value = rng.standard_normal((B, S, G, D)).astype(np.float32)
    attn = rng.standard_normal((B, Q, G, L * K)).astype(np.float32)
    grad_out = rng.standard_normal((B, Q, G * D)).astype(np.float32)
    if coords == 2:
        ref = rng.uniform(-0.05, 1.05, (B, Q, L, 2)).astype(np.float32)
        offsets = (rng.standard_normal((B, Q, G, L, K, 2)) * 2.5).astype(np.float32)  # pixels
    else:
        ref = np.concatenate([rng.uniform(0.0, 1.0, (B, Q, L, 2)),
                              rng.uniform(0.05, 0.7, (B, Q, L, 2))], -1).astype(np.float32)
        offsets = (rng.standard_normal((B, Q, G, L, K, 2)) * K).astype(np.float32)
    return value, shapes, starts, ref, offsets, attn, grad_out


def _torch_locations(ref, offsets, shapes):
    """float32 torch arithmetic of the layer, on the CPU; also d(location)/d(offset)."""
    ref = torch.as_tensor(ref)[:, :, None, :, None, :]
    K = offsets.shape[4]
    if ref.shape[-1] == 2:
        wh = torch.as_tensor(shapes).flip(-1).to(torch.float32)[None, None, None, :, None, :]
        return ref + offsets / wh, (1.0 / wh.double()).expand(offsets.shape)
    return (ref[..., :2] + offsets / K * ref[..., 2:] * 0.5,
            (ref[..., 2:].double() * 0.5 / K).expand(offsets.shape))


@pytest.mark.parametrize("method", ["linear", "softmax"])
@pytest.mark.parametrize("coords", [2, 4])
@pytest.mark.parametrize("dtype,offsets16", [(torch.float32, False), (torch.float16, False),
                                             (torch.float16, True), (torch.bfloat16, False),
                                             (torch.bfloat16, True)])
def test_fused_offsets_match_oracle_on_torch_locations(dtype, offsets16, coords, method):
    value, shapes, starts, ref, offsets, attn, grad_out = _case(11 + coords, coords)
    sm = method == "softmax"
    v, a, go = dev(value, dtype), dev(attn, dtype), dev(grad_out, dtype)
    off = dev(offsets, dtype if offsets16 else torch.float32)
    r, sh, st = dev(ref, torch.float32), dev(shapes), dev(starts)

    out = abi_forward_offsets(v, sh, st, r, off, a, softmax=sm)
    gv, goff, ga = abi_backward_offsets(v, sh, st, r, off, a, go, softmax=sm)
    torch.cuda.synchronize()
    assert goff.dtype == off.dtype and goff.shape == off.shape

    loc, dloc = _torch_locations(ref, off.cpu().float(), shapes)
    args = (v.cpu(), shapes, starts, loc, a.cpu())
    e_out = orc.forward(*args, softmax=sm, precision="f64")
    e_gv, e_gl, e_ga = orc.backward(*args, go.cpu(), softmax=sm, precision="f64")
    e_goff = np.asarray(e_gl) * dloc.numpy()
    keep = _stable_points(to_np(loc), shapes)[..., None]

    tol_out, tol_grad = TOL[dtype]
    errs = {"out": rel_err(to_np(out), e_out), "grad_value": rel_err(to_np(gv), e_gv),
            "grad_offsets": rel_err(to_np(goff) * keep, e_goff * keep),
            "grad_attn": rel_err(to_np(ga), e_ga)}
    assert errs["out"] <= tol_out, errs
    assert errs["grad_value"] <= tol_grad, errs
    assert errs["grad_offsets"] <= (tol_grad if not offsets16 else 1e-2), errs
    assert errs["grad_attn"] <= tol_grad, errs
    for t in (out, gv, goff, ga):
        assert torch.isfinite(t).all()


@pytest.mark.parametrize("coords", [2, 4])
def test_fused_forward_is_bit_identical_to_the_location_entry(coords):
    """The kernel forms ``ref + offset / (W, H)`` with IEEE float32 division and addition, the
    same bits torch produces; out, grad_value and grad_attn of the two entry points then agree
    exactly in float32 (same kernel, same locations)."""
    value, shapes, starts, ref, offsets, attn, grad_out = _case(5, coords)
    v, a, go = (dev(x, torch.float32) for x in (value, attn, grad_out))
    off, r, sh, st = dev(offsets, torch.float32), dev(ref, torch.float32), dev(shapes), dev(starts)
    loc, _ = _torch_locations(ref, torch.as_tensor(offsets), shapes)
    l = dev(loc.contiguous(), torch.float32)

    out_f = abi_forward_offsets(v, sh, st, r, off, a, softmax=True)
    out_l = abi_forward(v, sh, st, l, a, softmax=True)
    assert torch.equal(out_f, out_l)
    gv_f, goff, ga_f = abi_backward_offsets(v, sh, st, r, off, a, go, softmax=True)
    gv_l, gl, ga_l = abi_backward(v, sh, st, l, a, go, softmax=True)
    assert torch.equal(ga_f, ga_l)
    # float32 reductions land in nondeterministic order
    assert rel_err(to_np(gv_f), to_np(gv_l)) <= 1e-6
    _, dloc = _torch_locations(ref, torch.as_tensor(offsets), shapes)
    assert rel_err(to_np(goff), to_np(gl) * dloc.numpy()) <= 1e-6


def test_entry_points_reject_bad_reference_points():
    from deformops_b200._loader import load_library
    shim = load_library()
    value, shapes, starts, ref, offsets, attn, _ = _case(1, 2, B=1, Q=8)
    v, a = dev(value, torch.float16), dev(attn, torch.float16)
    off, r, sh, st = dev(offsets, torch.float32), dev(ref, torch.float32), dev(shapes), dev(starts)
    out = torch.empty((1, 8, 4 * 16), dtype=torch.float16, device="cuda")
    import ctypes
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    common = (1, v.shape[1], 4, 16, 8, 3, 4, 1, 0, 0, ctypes.c_void_p(0))
    assert shim.forward_offsets(p(v), p(sh), p(st), p(r), 3, p(off), 0, p(a), p(out),
                                *common) == -1
    assert "coordinates" in shim.last_error()
    assert shim.forward_offsets(p(v), p(sh), p(st), p(r), 2, p(off), 2, p(a), p(out),
                                *common) == -1          # bf16 offsets with f16 values
    assert "offsets must be" in shim.last_error()
    assert shim.forward_offsets(p(v), p(sh), p(st), None, 2, p(off), 0, p(a), p(out),
                                *common) == -1
    assert "reference_points" in shim.last_error()


# ---- the operator and the functional above the ABI ----------------------------------------

def _tensors(coords, dtype, offsets16=False, **kw):
    value, shapes, starts, ref, offsets, attn, grad_out = _case(21, coords, **kw)
    return (dev(value, dtype).requires_grad_(), dev(shapes), dev(starts),
            dev(ref, torch.float32), dev(offsets, dtype if offsets16 else torch.float32)
            .requires_grad_(), dev(attn, dtype).requires_grad_(), dev(grad_out, dtype))


@pytest.mark.parametrize("coords", [2, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_functional_matches_the_unfused_route(dtype, coords):
    from deformops_b200 import msda, msda_from_offsets
    from deformops_b200.registry import locations_from_offsets

    v, sh, st, r, off, a, go = _tensors(coords, dtype)
    if coords == 2:
        r.requires_grad_()
    out = msda_from_offsets(v, sh, st, r, off, a, softmax=True)
    grads = torch.autograd.grad(out, [v, off, a] + ([r] if coords == 2 else []), go)

    v2, off2, a2, r2 = (t.detach().clone().requires_grad_() for t in (v, off, a, r))
    out2 = msda(v2, sh, st, locations_from_offsets(r2, off2, sh), a2, softmax=True)
    grads2 = torch.autograd.grad(out2, [v2, off2, a2] + ([r2] if coords == 2 else []), go)

    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_err(to_np(out), to_np(out2)) <= tol
    for g, g2 in zip(grads, grads2):
        assert g.shape == g2.shape and g.dtype == g2.dtype
        assert rel_err(to_np(g), to_np(g2)) <= (1e-4 if dtype == torch.float32 else 2e-2)


def test_boxes_that_need_a_gradient_take_the_unfused_route():
    from deformops_b200 import msda_from_offsets
    v, sh, st, r, off, a, go = _tensors(4, torch.float32)
    r.requires_grad_()
    out = msda_from_offsets(v, sh, st, r, off, a)
    (g_ref,) = torch.autograd.grad(out, [r], go)
    assert g_ref.shape == r.shape and torch.isfinite(g_ref).all() and g_ref.abs().sum() > 0


def test_offsets_in_the_value_dtype_keep_their_dtype():
    from deformops_b200 import msda_from_offsets
    v, sh, st, r, off, a, go = _tensors(2, torch.bfloat16, offsets16=True)
    out = msda_from_offsets(v, sh, st, r, off, a, softmax=True)
    (g_off,) = torch.autograd.grad(out, [off], go)
    assert g_off.dtype == torch.bfloat16 and torch.isfinite(g_off).all()


def test_offsets_op_passes_opcheck():
    v, sh, st, r, off, a, _ = _tensors(2, torch.float32, B=1, Q=9, G=2, D=8, K=2)
    torch.library.opcheck(torch.ops.deformops_b200.msda_offsets_forward.default,
                          (v, sh, st, r, off, a, True))


def test_functional_argument_errors():
    from deformops_b200 import msda_from_offsets
    v, sh, st, r, off, a, _ = _tensors(2, torch.float32, B=1, Q=9)
    with pytest.raises(ValueError, match="reference points must be"):
        msda_from_offsets(v, sh, st, r[..., :1], off, a)
    with pytest.raises(ValueError, match="do not match offsets"):
        msda_from_offsets(v, sh, st, r[:, :5], off, a)
    out = msda_from_offsets(v, sh, st, r[:, :0], off[:, :0], a[:, :0])
    assert out.shape == (1, 0, v.shape[2] * v.shape[3])


@pytest.mark.parametrize("coords", [2, 4])
def test_fused_offsets_with_odd_points_heads_and_ragged_levels(coords):
    """K = 3 (``offset / K`` is not a power-of-two scale), 3 heads, levels down to 1 x 2."""
    value, shapes, starts, ref, offsets, attn, grad_out = _case(
        31, coords, B=3, Q=41, G=3, D=8, K=3, levels=[(7, 5), (3, 4), (1, 2)])
    v, a, go = (dev(x, torch.float32) for x in (value, attn, grad_out))
    off, r, sh, st = dev(offsets, torch.float32), dev(ref, torch.float32), dev(shapes), dev(starts)
    out = abi_forward_offsets(v, sh, st, r, off, a, softmax=True)
    gv, goff, ga = abi_backward_offsets(v, sh, st, r, off, a, go, softmax=True)
    loc, dloc = _torch_locations(ref, torch.as_tensor(offsets), shapes)
    args = (value, shapes, starts, loc, attn)
    e_out = orc.forward(*args, softmax=True, precision="f64")
    e_gv, e_gl, e_ga = orc.backward(*args, grad_out, softmax=True, precision="f64")
    keep = _stable_points(to_np(loc), shapes)[..., None]
    assert rel_err(to_np(out), e_out) <= 1e-5
    assert rel_err(to_np(gv), e_gv) <= 1e-4 and rel_err(to_np(ga), e_ga) <= 1e-4
    assert rel_err(to_np(goff) * keep, np.asarray(e_gl) * dloc.numpy() * keep) <= 1e-4
