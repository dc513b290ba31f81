"""The C oracle against fixtures produced by the reference library itself (CPU only)."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import msda_oracle as orc
from tests._golden import FULL_CASES, METHODS, attn_for, load, load_cfg0, rel_err


def _run(case, method, precision):
    sm = method == "softmax"
    args = (case["value"], case["spatial_shapes"], case["level_start_index"], case["loc"],
            attn_for(case, method))
    out = orc.forward(*args, softmax=sm, precision=precision)
    grads = orc.backward(*args, case["grad_out"], softmax=sm, precision=precision)
    return out, grads


@pytest.mark.parametrize("method", METHODS)
@pytest.mark.parametrize("name", FULL_CASES)
def test_oracle_f64_matches_reference(name, method):
    case = load(name)
    out, (gv, gl, ga) = _run(case, method, "f64")
    tol = 1e-12
    assert rel_err(out, case[f"{method}_out_eager"]) < tol
    # the reference's grid_sample definition agrees with its eager backend to ~1e-6 only
    # because grid_sample maps coordinates differently in floating point
    assert rel_err(out, case[f"{method}_out_gridsample"]) < 1e-5
    assert rel_err(gv, case[f"{method}_grad_value"]) < tol
    assert rel_err(gl, case[f"{method}_grad_loc"]) < tol
    assert rel_err(ga, case[f"{method}_grad_attn"]) < tol


@pytest.mark.parametrize("method", METHODS)
@pytest.mark.parametrize("name", FULL_CASES)
def test_oracle_f32_matches_reference(name, method):
    case = load(name)
    out, (gv, gl, ga) = _run(case, method, "f32")
    assert rel_err(out, case[f"{method}_out_eager"]) < 1e-5
    assert rel_err(gv, case[f"{method}_grad_value"]) < 1e-5
    assert rel_err(gl, case[f"{method}_grad_loc"]) < 1e-4
    assert rel_err(ga, case[f"{method}_grad_attn"]) < 1e-4


def test_boundary_known_answers():
    """value[s] = s on a 4x4 map: spot values that follow from the pixel table by hand."""
    case = load("boundary")
    out = orc.forward(case["value"], case["spatial_shapes"], case["level_start_index"],
                      case["loc"][:, :, :, :, :1], np.ones((1, 1, 1, 1)), precision="f64")
    # first location (0, 0) -> pixel (-0.5, -0.5): only corner (0,0) is inside, weight 0.25
    assert out.reshape(-1)[0] == 0.0  # value at pixel 0 is 0
    coords = [0.0, 0.125, 0.375, 0.5, 1.0, -0.125, 1.25]
    expected = {
        (0.125, 0.125): 0.0,    # pixel (0,0)
        (0.375, 0.125): 1.0,    # pixel x=1, y=0
        (0.375, 0.375): 5.0,    # pixel (1,1) -> s = 1*4 + 1
        (0.5, 0.5): 7.5,        # centre of pixels 5,6,9,10
        (1.0, 1.0): 15 * 0.25,  # pixel (3.5,3.5): only corner 15 inside, weight 0.25
        (-0.125, 0.5): 0.0,     # pixel x = -1: kept, but its only inside corners have weight 0
        (1.25, 0.5): 0.0,       # pixel x = 4.5: skipped
    }
    for i, (cx, cy) in enumerate((cx, cy) for cx in coords for cy in coords):
        if (cx, cy) in expected:
            got = orc.forward(case["value"], case["spatial_shapes"], case["level_start_index"],
                              case["loc"][:, :, :, :, i:i + 1], np.ones((1, 1, 1, 1)),
                              precision="f64").item()
            assert got == pytest.approx(expected[(cx, cy)], abs=1e-12), (cx, cy)


def test_all_outside_is_exactly_zero():
    case = load("all_outside")
    for method in METHODS:
        out, (gv, gl, ga) = _run(case, method, "f32")
        assert not out.any() and not gv.any() and not gl.any() and not ga.any()


@pytest.mark.parametrize("method", METHODS)
def test_oracle_cfg0_matches_reference(method):
    w, gold = load_cfg0()
    sm = method == "softmax"
    attn = w.attention_logits if sm else w.attention_weights
    args = (w.value, w.spatial_shapes, w.level_start_index, w.sampling_locations, attn)
    out = orc.forward(*args, softmax=sm, precision="f64")
    gv, gl, ga = orc.backward(*args, w.grad_output, softmax=sm, precision="f64")
    stride = int(gold["row_stride"])
    for key, arr in (("out_eager", out), ("grad_value", gv), ("grad_loc", gl), ("grad_attn", ga)):
        rows = arr.reshape(arr.shape[0], arr.shape[1], -1)[:, ::stride]
        assert rel_err(rows, gold[f"{method}_{key}_rows"]) < 1e-12, key
        assert float(arr.sum()) == pytest.approx(float(gold[f"{method}_{key}_sum"]), rel=1e-9, abs=1e-7)
        assert float(np.abs(arr).sum()) == pytest.approx(float(gold[f"{method}_{key}_abssum"]), rel=1e-10)


@pytest.mark.parametrize("method", METHODS)
@pytest.mark.parametrize("name", ["boundary", "small_b", "small_c", "ragged", "all_outside"])
def test_eager_port_matches_reference(name, method):
    """The torch restatement of the reference's eager path (timed as the CPU baseline)."""
    import torch

    from oracle.msda_eager_port import eager_forward_backward

    case = load(name)
    t = {k: torch.from_numpy(case[k]).double() for k in ("value", "loc", "grad_out")}
    attn = torch.from_numpy(attn_for(case, method)).double()
    out, gv, gl, ga = eager_forward_backward(
        t["value"], torch.from_numpy(case["spatial_shapes"]),
        torch.from_numpy(case["level_start_index"]), t["loc"], attn, t["grad_out"],
        softmax=method == "softmax")
    assert rel_err(out.numpy(), case[f"{method}_out_eager"]) < 1e-12
    assert rel_err(gv.numpy(), case[f"{method}_grad_value"]) < 1e-12
    assert rel_err(gl.numpy(), case[f"{method}_grad_loc"]) < 1e-12
    assert rel_err(ga.numpy(), case[f"{method}_grad_attn"]) < 1e-12
