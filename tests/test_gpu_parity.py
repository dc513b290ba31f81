"""GPU parity: the sm_100a kernels, called through the C ABI, against the pinned oracle and
the golden fixtures made by the reference.

Tolerances (metric of the reference's own tests, ``max|a-b| / max|b|``):
  float32   output 1e-5, gradients 1e-4
  bf16/fp16 1e-2 of the float32-accurate result computed from the same (rounded) inputs;
            ``grad_value`` is summed with 16-bit atomics in nondeterministic order.
"""

from __future__ import annotations

import json
import os
import pathlib

import numpy as np
import pytest
import torch

from oracle import msda_oracle as orc
from tests._abi import abi_backward, abi_forward, dev, to_np
from tests._golden import FULL_CASES, METHODS, attn_for, load, load_cfg0, rel_err

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (1e-5, 1e-4), torch.float16: (1e-2, 1e-2), torch.bfloat16: (1e-2, 1e-2)}
DTYPES = [torch.float32, torch.float16, torch.bfloat16]
#: set DEFORMOPS_B200_PARITY_LOG to a file to collect the measured errors of every case
_LOG = os.environ.get("DEFORMOPS_B200_PARITY_LOG")


def _record(name, dtype, method, errs):
    if not _LOG:
        return
    try:
        pathlib.Path(_LOG).parent.mkdir(parents=True, exist_ok=True)
        with open(_LOG, "a") as fh:
            fh.write(json.dumps({"case": name, "dtype": str(dtype), "method": method,
                                 **{k: float(v) for k, v in errs.items()}}) + "\n")
    except OSError:
        pass


def _stable_points(loc, shapes):
    """Mask of sample points whose pixel coordinates are not within 1e-4 of an integer.

    The location gradient is one-sided at integer pixels, so a float32 rounding of
    ``loc * size - 0.5`` (fused or not) that lands on the other side of an integer flips it;
    output, grad_value and grad_attn are continuous there and are compared everywhere.  Exact
    integer pixels are pinned separately by the ``ragged`` and ``boundary`` fixtures."""
    loc = np.asarray(loc, dtype=np.float64)
    hw = np.asarray(shapes, dtype=np.float64).reshape(1, 1, 1, -1, 1, 2)
    pix = loc * hw[..., ::-1] - 0.5
    near = np.abs(pix - np.round(pix)) < 1e-4
    exact = pix == np.round(pix)
    return ~(near & ~exact).any(-1)


def run_case(name, value, shapes, starts, loc, attn, grad_out, dtype, method, expected=None,
             tol=None):
    """Run fwd+bwd through the ABI at ``dtype``; compare with ``expected`` or the f64 oracle
    evaluated on the inputs as the kernel sees them (rounded to ``dtype``)."""
    sm = method == "softmax"
    v, a, go = dev(value, dtype), dev(attn, dtype), dev(grad_out, dtype)
    l = dev(loc, torch.float32)
    sh, st = dev(shapes), dev(starts)
    out = abi_forward(v, sh, st, l, a, softmax=sm)
    gv, gl, ga = abi_backward(v, sh, st, l, a, go, softmax=sm)
    torch.cuda.synchronize()
    if expected is None:
        args = (v.cpu(), shapes, starts, l.cpu(), a.cpu())
        e_out = orc.forward(*args, softmax=sm, precision="f64")
        e_gv, e_gl, e_ga = orc.backward(*args, go.cpu(), softmax=sm, precision="f64")
    else:
        e_out, e_gv, e_gl, e_ga = expected
    keep = _stable_points(to_np(l), shapes)[..., None]
    errs = {"out": rel_err(to_np(out), e_out), "grad_value": rel_err(to_np(gv), e_gv),
            "grad_loc": rel_err(to_np(gl) * keep, np.asarray(e_gl) * keep),
            "grad_attn": rel_err(to_np(ga), e_ga)}
    _record(name, dtype, method, errs)
    tol_out, tol_grad = tol or TOL[dtype]
    assert errs["out"] <= tol_out, errs
    assert errs["grad_value"] <= tol_grad, errs
    assert errs["grad_loc"] <= tol_grad, errs
    assert errs["grad_attn"] <= tol_grad, errs
    for t in (out, gv, gl, ga):
        assert torch.isfinite(t).all()
    return out, gv, gl, ga


@pytest.mark.parametrize("method", METHODS)
@pytest.mark.parametrize("name", FULL_CASES)
def test_fp32_matches_reference_fixtures(name, method):
    """float32 kernels against outputs the reference itself produced (fixtures)."""
    c = load(name)
    expected = tuple(c[f"{method}_{k}"] for k in ("out_eager", "grad_value", "grad_loc", "grad_attn"))
    value, grad_out = c["value"], c["grad_out"]
    D = value.shape[3]
    if D % 4:
        # the kernels move 16-byte channel vectors: replicate the channel 4x.  Every channel
        # then equals the fixture's; location / weight gradients sum over channels (x4).
        B, S, G, _ = value.shape
        value = np.repeat(value, 4, axis=3)
        grad_out = np.repeat(grad_out.reshape(B, -1, G, D), 4, axis=3).reshape(B, -1, G * D * 4)
        e_out, e_gv, e_gl, e_ga = expected
        expected = (np.repeat(e_out.reshape(B, -1, G, D), 4, axis=3).reshape(B, -1, G * D * 4),
                    np.repeat(e_gv, 4, axis=3), e_gl * 4, e_ga * 4)
    run_case(name, value, c["spatial_shapes"], c["level_start_index"], c["loc"],
             attn_for(c, method), grad_out, torch.float32, method, expected)


@pytest.mark.parametrize("method", METHODS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("name", ["small_b", "small_c", "k8_d64", "ragged"])
def test_16bit_matches_oracle_on_fixture_inputs(name, dtype, method):
    c = load(name)
    # Small fixtures: a handful of elements decide the max-norm metric and the order of the
    # 16-bit additions changes from run to run (measured over 30 runs: grad_value up to 7.4e-3,
    # typically 5e-3..7e-3), so the gradients get the reference's own 16-bit tolerance of 2e-2
    # (tests/deformops/test_experimental_parity.py:58); the full-size configurations below,
    # whose error barely moves between runs, keep 1e-2.
    run_case(name, c["value"], c["spatial_shapes"], c["level_start_index"], c["loc"],
             attn_for(c, method), c["grad_out"], dtype, method, tol=(1e-2, 2e-2))


@pytest.mark.parametrize("method", METHODS)
def test_cfg0_fp32_matches_reference_fixture(method):
    w, gold = load_cfg0()
    sm = method == "softmax"
    attn = w.attention_logits if sm else w.attention_weights
    v, l, a, go = (dev(t) for t in (w.value, w.sampling_locations, attn, w.grad_output))
    sh, st = dev(w.spatial_shapes), dev(w.level_start_index)
    out = abi_forward(v, sh, st, l, a, softmax=sm)
    gv, gl, ga = abi_backward(v, sh, st, l, a, go, softmax=sm)
    stride = int(gold["row_stride"])
    for key, t, tol in (("out_eager", out, 1e-5), ("grad_value", gv, 1e-4),
                        ("grad_loc", gl, 1e-4), ("grad_attn", ga, 1e-4)):
        arr = to_np(t)
        rows = arr.reshape(arr.shape[0], arr.shape[1], -1)[:, ::stride]
        assert rel_err(rows, gold[f"{method}_{key}_rows"]) <= tol, key
        assert np.abs(arr).sum() == pytest.approx(float(gold[f"{method}_{key}_abssum"]), rel=1e-4)


def _workload_case(name, method, dtype=None, batch=None):
    from deformops_b200.workloads import CONFIGS, make_workload

    w = make_workload(name, batch=batch)
    dtype = dtype or CONFIGS[name]["dtype"]
    attn = w.attention_logits if method == "softmax" else w.attention_weights
    return run_case(name, w.value, w.spatial_shapes, w.level_start_index, w.sampling_locations,
                    attn, w.grad_output, dtype, method)


@pytest.mark.parametrize("name,method", [
    ("cfg0_cpu_fp32", "linear"), ("cfg1_m2f_512_bf16", "linear"), ("cfg2_m2f_1024_bf16", "linear"),
    ("cfg2_m2f_1024_bf16", "softmax"), ("cfg3_detr_enc_fp16", "linear"),
    ("cfg3_detr_enc_fp32", "linear"), ("cfg3_detr_dec_fp16", "linear"),
    ("cfg3_detr_dec_fp16", "softmax"),
])
def test_baseline_configs_full_size(name, method):
    """Every benchmark configuration at its full size against the oracle."""
    _workload_case(name, method)


def test_full_size_adjoint_identities():
    """Size-independent properties at the headline size (float32): the operator is linear in
    value and in the weights, so <grad_out, out> = <value, grad_value> = <attn, grad_attn>."""
    from deformops_b200.workloads import make_workload

    w = make_workload("cfg2_m2f_1024_bf16", batch=2)
    v, l, a, go = (dev(t, torch.float32) for t in
                   (w.value, w.sampling_locations, w.attention_weights, w.grad_output))
    sh, st = dev(w.spatial_shapes), dev(w.level_start_index)
    out = abi_forward(v, sh, st, l, a)
    gv, gl, ga = abi_backward(v, sh, st, l, a, go)
    lhs = (go.double() * out.double()).sum().item()
    assert (v.double() * gv.double()).sum().item() == pytest.approx(lhs, rel=1e-5)
    assert (a.double() * ga.double()).sum().item() == pytest.approx(lhs, rel=1e-5)
    # exact linearity under a power-of-two scale of value
    out2 = abi_forward(v * 2, sh, st, l, a)
    assert torch.equal(out2, out * 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [
    # B, G, D, levels, K, Q
    (1, 1, 8, [(5, 7)], 1, 3),
    (2, 3, 16, [(6, 5), (3, 4)], 3, 37),          # odd heads, odd points, ragged tile
    (1, 8, 32, [(9, 9), (5, 5), (3, 3), (2, 2)], 4, 100),
    (2, 2, 128, [(8, 6)], 4, 19),                  # wide head: 16 or 32 lanes per slot
    (1, 5, 24, [(7, 7), (4, 4)], 2, 11),           # D not a power of two
    (3, 16, 16, [(4, 4), (2, 2), (1, 1)], 8, 65),
    (1, 4, 64, [(3, 3)] * 5, 4, 9),
    (1, 2, 256, [(5, 4), (2, 3)], 2, 7),           # float32: 64 vectors, two channel passes per lane
    (2, 1, 512, [(4, 4)], 3, 5),                   # 16-bit: 64 vectors as well
])
def test_shape_envelope(shape, dtype):
    B, G, D, levels, K, Q = shape
    if dtype != torch.float32 and D % 8:
        pytest.skip("16-bit kernels need D % 8 == 0")
    g = torch.Generator().manual_seed(1234)
    L, S = len(levels), sum(h * w for h, w in levels)
    shapes = torch.tensor(levels, dtype=torch.int64)
    starts = torch.cumsum(shapes[:, 0] * shapes[:, 1], 0) - shapes[:, 0] * shapes[:, 1]
    value = torch.randn(B, S, G, D, generator=g)
    loc = torch.rand(B, Q, G, L, K, 2, generator=g) * 1.3 - 0.15
    logits = torch.randn(B, Q, G, L * K, generator=g)
    grad_out = torch.randn(B, Q, G * D, generator=g)
    for method in METHODS:
        attn = logits if method == "softmax" else logits.softmax(-1)
        # tiny levels: a handful of elements decide the max-norm metric, so 16-bit runs get the
        # reference's own 16-bit tolerance (2e-2, tests/deformops/test_experimental_parity.py:58)
        tol = None if dtype == torch.float32 else (1e-2, 2e-2)
        run_case(f"envelope{shape}", value, shapes, starts, loc, attn, grad_out, dtype, method,
                 tol=tol)


def test_far_outside_gives_exact_zeros():
    c = load("all_outside")
    for method in METHODS:
        out, gv, gl, ga = run_case("all_outside", c["value"], c["spatial_shapes"],
                                   c["level_start_index"], c["loc"], attn_for(c, method),
                                   c["grad_out"], torch.float32, method)
        for t in (out, gv, gl, ga):
            assert not t.any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_non_finite_locations_are_skipped(dtype):
    """inf / NaN locations fail the pixel-range test: nothing is read or written for them,
    grad_value stays finite and every other query is unaffected."""
    c = load("small_b")
    loc = c["loc"].copy()
    loc[0, 0, 0, 0, 0] = [np.inf, 0.5]
    loc[0, 1, 1, 1, 1] = [0.5, -np.inf]
    loc[1, 2, 2, 2, 2] = [np.nan, np.nan]
    loc[1, 3] = np.inf
    run_case("non_finite", c["value"], c["spatial_shapes"], c["level_start_index"], loc,
             c["attn_linear"], c["grad_out"], dtype, "linear")


def test_empty_batch_and_zero_queries():
    c = load("small_b")
    sh, st = dev(c["spatial_shapes"]), dev(c["level_start_index"])
    v = dev(c["value"])
    G, L, K = v.shape[2], sh.shape[0], c["loc"].shape[4]
    loc0 = torch.empty(v.shape[0], 0, G, L, K, 2, device="cuda")
    attn0 = torch.empty(v.shape[0], 0, G, L * K, device="cuda")
    out = abi_forward(v, sh, st, loc0, attn0)
    assert out.shape == (v.shape[0], 0, G * v.shape[3])
    gv, gl, ga = abi_backward(v, sh, st, loc0, attn0, out)
    assert not gv.any() and gl.numel() == 0 and ga.numel() == 0
    vb = v[:0]
    out = abi_forward(vb, sh, st, loc0[:0], attn0[:0])
    assert out.numel() == 0


def test_accumulate_into_caller_buffer():
    """zero_grad_value = 0 adds into the buffer the caller prepared."""
    c = load("small_c")
    args = [dev(c[k]) for k in ("value", "spatial_shapes", "level_start_index", "loc",
                                "attn_linear", "grad_out")]
    gv1, _, _ = abi_backward(*args)
    gv2, _, _ = abi_backward(*args, zero=False)
    torch.testing.assert_close(gv1, gv2, rtol=1e-5, atol=1e-6)


def test_deterministic_outputs():
    """out, grad_loc and grad_attn have a fixed summation order: bit-identical across runs."""
    from deformops_b200.workloads import make_workload

    w = make_workload("cfg1_m2f_512_bf16", batch=2)
    v, l, a, go = (dev(t) for t in (w.value, w.sampling_locations, w.attention_weights, w.grad_output))
    sh, st = dev(w.spatial_shapes), dev(w.level_start_index)
    ref = None
    for _ in range(3):
        out = abi_forward(v, sh, st, l, a)
        _, gl, ga = abi_backward(v, sh, st, l, a, go)
        cur = (out.clone(), gl.clone(), ga.clone())
        if ref is not None:
            assert all(torch.equal(x, y) for x, y in zip(ref, cur))
        ref = cur


def test_bad_arguments_return_status_not_crash():
    import ctypes

    from deformops_b200._loader import load_library

    shim = load_library()
    null = ctypes.c_void_p(0)
    st = shim.forward(null, null, null, null, null, null, 1, 4, 1, 8, 1, 1, 1, 2, 0, 0, null)
    assert st == -1 and "null" in shim.last_error()
    st = shim.forward(null, null, null, null, null, null, 1, 4, 1, 12, 1, 1, 1, 2, 0, 0, null)
    assert st == -2 and "multiple of 8" in shim.last_error()
    st = shim.forward(null, null, null, null, null, null, 1, 4, 1, 8, 1, 99, 1, 2, 0, 0, null)
    assert st == -2
    st = shim.forward(null, null, null, null, null, null, 1, 4, 1, 8, 1, 1, 1, 7, 0, 0, null)
    assert st == -1


def _random_shape_case():
    """Hypothesis strategy over the operator's envelope, in the spirit of the reference's
    property tests (``tests/deformops/test_msda_cuda.py:30-71``): ragged level pyramids down to
    1x1, 1..8 points, 1..5 levels, odd head counts, head sizes from one to many 16-byte vectors,
    locations reaching outside [0, 1]."""
    from hypothesis import strategies as st

    level = st.tuples(st.integers(1, 11), st.integers(1, 11))
    return st.fixed_dictionaries({
        "B": st.integers(1, 3), "G": st.integers(1, 9),
        "D": st.sampled_from([4, 8, 12, 16, 32, 40, 64, 128]),
        "levels": st.lists(level, min_size=1, max_size=5),
        "K": st.integers(1, 8), "Q": st.integers(1, 70),
        "spread": st.sampled_from([1.0, 1.3, 3.0]),
        "softmax": st.booleans(), "seed": st.integers(0, 2**31 - 1),
    })


def test_random_envelope_float32_property():
    from hypothesis import HealthCheck, given, settings

    @settings(max_examples=120, deadline=None, derandomize=True,
              suppress_health_check=list(HealthCheck))
    @given(_random_shape_case())
    def check(s):
        g = torch.Generator().manual_seed(s["seed"])
        levels = s["levels"]
        L, S = len(levels), sum(h * w for h, w in levels)
        B, G, D, K, Q = s["B"], s["G"], s["D"], s["K"], s["Q"]
        shapes = torch.tensor(levels, dtype=torch.int64)
        sizes = shapes[:, 0] * shapes[:, 1]
        starts = torch.cumsum(sizes, 0) - sizes
        value = torch.randn(B, S, G, D, generator=g)
        loc = (torch.rand(B, Q, G, L, K, 2, generator=g) - 0.5) * s["spread"] + 0.5
        logits = torch.randn(B, Q, G, L * K, generator=g)
        grad_out = torch.randn(B, Q, G * D, generator=g)
        method = "softmax" if s["softmax"] else "linear"
        attn = logits if s["softmax"] else logits.softmax(-1)
        run_case(f"property{(B, G, D, levels, K, Q)}", value, shapes, starts, loc, attn,
                 grad_out, torch.float32, method)

    check()
