"""GPU checks modelled on the reference's robustness tests: bias of the 16-bit ``grad_value``
sums, ``-inf`` logits, odd batch sizes, concurrent streams and host threads."""

from __future__ import annotations

import threading

import numpy as np
import pytest
import torch

from oracle import msda_oracle as orc
from tests._abi import abi_backward, abi_forward, dev, to_np
from tests._golden import rel_err

pytestmark = pytest.mark.gpu


def _case(seed, B, Q, G, D, K, levels, spread=1.2):
    g = torch.Generator().manual_seed(seed)
    shapes = torch.tensor(levels, dtype=torch.int64)
    sizes = shapes[:, 0] * shapes[:, 1]
    starts = torch.cumsum(sizes, 0) - sizes
    S, L = int(sizes.sum()), len(levels)
    value = torch.randn(B, S, G, D, generator=g)
    loc = (torch.rand(B, Q, G, L, K, 2, generator=g) - 0.5) * spread + 0.5
    logits = torch.randn(B, Q, G, L * K, generator=g)
    grad_out = torch.randn(B, Q, G * D, generator=g)
    return value, shapes, starts, loc, logits, grad_out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_16bit_grad_value_has_no_directional_bias(dtype):
    """The rounding error of the 16-bit sums must not lean along the true gradient (it would
    act as a learning-rate change): |cos(mean error, truth)| < 0.05 over four runs, the
    reference's criterion and shape (``tests/deformops/test_msda_bias.py:78-109``: Q=1024,
    levels 48/24/12)."""
    value, shapes, starts, loc, logits, grad_out = _case(
        7, 2, 1024, 8, 32, 4, [(48, 48), (24, 24), (12, 12)], spread=1.0)
    attn = logits.softmax(-1)
    v, a, go = dev(value, dtype), dev(attn, dtype), dev(grad_out, dtype)
    l, sh, st = dev(loc, torch.float32), dev(shapes), dev(starts)
    truth, _, _ = orc.backward(v.cpu(), shapes, starts, l.cpu(), a.cpu(), go.cpu(), precision="f64")
    runs = [to_np(abi_backward(v, sh, st, l, a, go)[0]) for _ in range(4)]
    mean_err = (np.mean(runs, axis=0) - truth).ravel()
    t = np.asarray(truth).ravel()
    cos = float(mean_err @ t / (np.linalg.norm(mean_err) * np.linalg.norm(t) + 1e-30))
    assert abs(cos) < 0.05, cos


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_with_minus_infinity_logits_and_wide_locations(dtype):
    """A masked-out point (``-inf`` logit) gets probability zero, nothing becomes NaN, and
    locations far outside the image only drop out (reference:
    ``tests/deformops/test_msda_softmax_before_softmax_gpu.py:79-126``)."""
    value, shapes, starts, loc, logits, grad_out = _case(
        3, 2, 60, 4, 32, 4, [(9, 11), (5, 6), (3, 3)], spread=4.0)
    logits[:, ::3, :, 5] = float("-inf")
    logits[0, 1, 0, :-1] = float("-inf")          # a pair with a single live point
    v, a, go = dev(value, dtype), dev(logits, dtype), dev(grad_out, dtype)
    l, sh, st = dev(loc, torch.float32), dev(shapes), dev(starts)
    out = abi_forward(v, sh, st, l, a, softmax=True)
    gv, gl, ga = abi_backward(v, sh, st, l, a, go, softmax=True)
    for t in (out, gv, gl, ga):
        assert torch.isfinite(t).all()
    args = (v.cpu(), shapes, starts, l.cpu(), a.cpu())
    e_out = orc.forward(*args, softmax=True, precision="f64")
    e_gv, e_gl, e_ga = orc.backward(*args, go.cpu(), softmax=True, precision="f64")
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert rel_err(to_np(out), e_out) <= tol
    assert rel_err(to_np(gv), e_gv) <= tol
    assert rel_err(to_np(ga), e_ga) <= tol
    assert (to_np(ga)[:, ::3, :, 5] == 0).all()    # no gradient into a masked logit


@pytest.mark.parametrize("batch", [7, 70, 96])
def test_odd_batch_sizes(batch):
    """Batches that do not divide any internal tile (the reference splits them at
    ``chunk_step``, ``tests/deformops/test_release_hardening.py:280-301``; here one launch)."""
    value, shapes, starts, loc, logits, grad_out = _case(
        batch, batch, 13, 2, 16, 4, [(6, 7), (3, 4)])
    attn = logits.softmax(-1)
    v, a, go = (dev(x, torch.float32) for x in (value, attn, grad_out))
    l, sh, st = dev(loc, torch.float32), dev(shapes), dev(starts)
    out = abi_forward(v, sh, st, l, a)
    gv, gl, ga = abi_backward(v, sh, st, l, a, go)
    args = (value, shapes, starts, loc, attn)
    assert rel_err(to_np(out), orc.forward(*args, precision="f64")) <= 1e-5
    e_gv, e_gl, e_ga = orc.backward(*args, grad_out, precision="f64")
    assert rel_err(to_np(gv), e_gv) <= 1e-4 and rel_err(to_np(ga), e_ga) <= 1e-4


def test_concurrent_streams_and_host_threads():
    """Calls from several host threads on their own streams (the autograd engine calls the
    backward from another thread): every result equals the single-threaded one."""
    from deformops_b200.registry import msda

    value, shapes, starts, loc, logits, grad_out = _case(
        11, 2, 500, 8, 32, 4, [(20, 20), (10, 10), (5, 5)])
    v, a, go = (dev(x, torch.float32) for x in (value, logits, grad_out))
    l, sh, st = dev(loc, torch.float32), dev(shapes), dev(starts)

    def step():
        vv, ll, aa = (t.detach().clone().requires_grad_() for t in (v, l, a))
        out = msda(vv, sh, st, ll, aa, softmax=True)
        grads = torch.autograd.grad(out, [vv, ll, aa], go)
        return out, grads

    want_out, want = step()
    torch.cuda.synchronize()
    results, errors = {}, []

    def worker(i):
        try:
            with torch.cuda.stream(torch.cuda.Stream()):
                for _ in range(5):
                    results[i] = step()
                torch.cuda.current_stream().synchronize()
        except Exception as exc:  # noqa: BLE001 - reported through the assertion below
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors, errors
    for out, grads in results.values():
        assert torch.equal(out, want_out)
        assert torch.equal(grads[1], want[1]) and torch.equal(grads[2], want[2])
        assert rel_err(to_np(grads[0]), to_np(want[0])) <= 1e-6


def test_malformed_level_tables_are_skipped_not_dereferenced():
    """Levels that do not lie inside the value tensor (too large, negative start, zero size,
    running past the end) act as empty levels: their points contribute nothing and get zero
    gradients.  The buffers here are allocated far larger than the size handed to the library,
    so the addresses such a table describes are inside the allocation either way; the test
    reads the behaviour off the results."""
    import ctypes

    from deformops_b200._loader import load_library

    shim = load_library()
    G, D, K, Q, S, rows = 2, 8, 2, 9, 16, 256
    g = torch.Generator().manual_seed(5)
    shapes = torch.tensor([[8, 8], [2, 4], [0, 5], [3, 3], [3, 3]], dtype=torch.int64)
    starts = torch.tensor([0, 4, 1, -4, 14], dtype=torch.int64)       # only level 1 fits S = 16
    L = shapes.shape[0]
    value = torch.randn(1, rows, G, D, generator=g)
    loc = torch.rand(1, Q, G, L, K, 2, generator=g)
    attn = torch.rand(1, Q, G, L * K, generator=g)
    grad_out = torch.randn(1, Q, G * D, generator=g)
    v, l, a, go = (dev(t, torch.float32) for t in (value, loc, attn, grad_out))
    sh, st = dev(shapes), dev(starts)
    out = torch.full((1, Q, G * D), float("nan"), device="cuda")
    gv = torch.full((1, rows, G, D), float("nan"), device="cuda")
    gl, ga = torch.full_like(l, float("nan")), torch.full_like(a, float("nan"))
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    z = ctypes.c_void_p(0)
    assert shim.forward(p(v), p(sh), p(st), p(l), p(a), p(out), 1, S, G, D, Q, L, K, 0, 0, 0, z) == 0
    assert shim.backward(p(v), p(sh), p(st), p(l), p(a), p(go), p(gv), p(gl), p(ga), None, 0, 0,
                         1, S, G, D, Q, L, K, 0, 0, 1, 0, z) == 0
    torch.cuda.synchronize()
    # expectation: the one valid level alone, on a consistent table
    one = (value[:, :S], shapes[1:2], starts[1:2], loc[:, :, :, 1:2].contiguous(),
           attn.view(1, Q, G, L, K)[:, :, :, 1].contiguous())
    e_out = orc.forward(*one, precision="f64")
    e_gv, e_gl, e_ga = orc.backward(*one, grad_out, precision="f64")
    assert rel_err(to_np(out), e_out) <= 1e-5
    assert rel_err(to_np(gv[:, :S]), e_gv) <= 1e-4
    assert torch.isnan(gv[:, S:]).all()                       # nothing beyond S rows was touched
    gl5, ga5 = gl.cpu(), ga.cpu().view(1, Q, G, L, K)
    assert rel_err(gl5[:, :, :, 1:2].numpy().astype(np.float64), e_gl) <= 1e-4
    assert rel_err(ga5[:, :, :, 1].numpy().astype(np.float64), e_ga) <= 1e-4
    for bad in (0, 2, 3, 4):
        assert (gl5[:, :, :, bad] == 0).all() and (ga5[:, :, :, bad] == 0).all()


def test_empty_value_tensor_gives_zeros():
    from deformops_b200.registry import msda

    value = torch.zeros(2, 0, 4, 8, device="cuda", requires_grad=True)
    shapes = torch.tensor([[3, 3]], device="cuda")
    starts = torch.tensor([0], device="cuda")
    loc = torch.rand(2, 5, 4, 1, 2, 2, device="cuda", requires_grad=True)
    attn = torch.rand(2, 5, 4, 2, device="cuda", requires_grad=True)
    out = msda(value, shapes, starts, loc, attn)
    assert out.shape == (2, 5, 32) and (out == 0).all()
    out.sum().backward()
    assert (loc.grad == 0).all() and (attn.grad == 0).all() and value.grad.shape == value.shape


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_non_finite_values_at_a_border_stay_within_the_documented_difference(dtype):
    """Pins how ``inf`` stored in a border pixel behaves.  The forward gather does not skip the
    load of a corner that lies outside its level (the reference does, ``interpolate.cuh:24-67``):
    it reads the nearest pixel inside and multiplies by an exact zero.  Skipping would cost 12 %
    of the forward at the headline shape, so the difference is kept and bounded here:
      * where the reference's result is non-finite, so is ours;
      * where ours is finite it equals the reference's;
      * ours may be non-finite where the reference's is finite ONLY for a (query, head) that
        has a skipped point or a point with a corner outside its level - and that does happen
        in this case (``0 * inf``), which is the whole difference.
    The backward predicates its loads, so gradients never see it."""
    value, shapes, starts, loc, logits, grad_out = _case(
        11, 2, 200, 4, 32, 4, [(6, 7), (3, 4)], spread=2.5)
    # far-away points (skipped), points hugging the border from outside, points inside
    loc[:, ::5] = 1.7
    loc[:, 1::5, :, :, :, 0] = -0.04
    loc[:, 2::5] = loc[:, 2::5].clamp(0.2, 0.8)
    attn = logits.softmax(-1)
    v32 = value.clone()
    for (h, w), first in zip(shapes.tolist(), starts.tolist()):
        v32[:, first] = float("inf")                    # pixel (0, 0) of the level
        v32[:, first + h * w - 1] = float("-inf")       # its last pixel
    v, a = dev(v32, dtype), dev(attn, dtype)
    l, sh, st = dev(loc, torch.float32), dev(shapes), dev(starts)
    out = to_np(abi_forward(v, sh, st, l, a)).reshape(2, 200, 4, 32)
    want = orc.forward(v.cpu(), shapes, starts, l.cpu(), a.cpu(), precision="f64").reshape(2, 200, 4, 32)
    ours_ok, ref_ok = np.isfinite(out), np.isfinite(want)
    assert not (ours_ok & ~ref_ok).any()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    both = ours_ok & ref_ok
    assert both.any() and np.abs(out[both] - want[both]).max() <= tol * np.abs(want[both]).max()
    # (query, head) pairs in which some point is skipped or has a corner outside its level
    wh = shapes.flip(-1).to(torch.float64)[None, None, None, :, None, :]
    pix = loc.to(torch.float64) * wh - 0.5
    partial = ((pix < 0) | (pix > wh - 1)).any(-1).any(-1).any(-1).numpy()     # (B, Q, G)
    only_ours = (~ours_ok & ref_ok).any(-1)
    assert only_ours.any(), "the case no longer exercises the difference"
    assert not (only_ours & ~partial).any()


def test_levels_listed_out_of_order_bf16_with_scratch():
    """``level_start_index`` need not ascend: the same pyramid with its levels listed in a
    different order (same pixels, same memory) gives the same gradients - the scratch image is
    addressed per level, never by "the last level that starts before this row"."""
    value, shapes, starts, loc, logits, grad_out = _case(
        5, 2, 150, 8, 32, 4, [(12, 9), (6, 5), (3, 3)], spread=1.1)
    attn = logits.softmax(-1)
    perm = [2, 0, 1]
    L, K = 3, 4
    loc_p = loc[:, :, :, perm]
    attn_p = attn.view(2, 150, 8, L, K)[:, :, :, perm].reshape(2, 150, 8, L * K)
    dt = torch.bfloat16
    v, go = dev(value, dt), dev(grad_out, dt)
    base = abi_backward(v, dev(shapes), dev(starts), dev(loc, torch.float32), dev(attn, dt), go)
    other = abi_backward(v, dev(shapes[perm]), dev(starts[perm]), dev(loc_p, torch.float32),
                         dev(attn_p, dt), go)
    truth, _, _ = orc.backward(v.cpu(), shapes, starts, loc, dev(attn, dt).cpu(), go.cpu())
    for gv in (base[0], other[0]):
        assert rel_err(to_np(gv), truth) <= 1e-2
    # the location / weight gradients are the same numbers in permuted places
    assert torch.equal(other[1], base[1][:, :, :, perm])
    assert torch.equal(other[2].view(2, 150, 8, L, K), base[2].view(2, 150, 8, L, K)[:, :, :, perm])


@pytest.mark.parametrize("G,D", [(1, 8), (2, 24)])
def test_many_small_samples_with_replicated_levels(G, D):
    """Hundreds of samples of a tiny pyramid whose levels all need several accumulators: the
    pass that folds the replicas into grad_value then strides over whole samples between the
    vectors one thread handles, and its running (sample, position, column) must stay right."""
    B, Q, K = 600, 300, 4
    value, shapes, starts, loc, logits, grad_out = _case(11, B, Q, G, D, K, [(4, 4), (2, 2)], spread=1.1)
    attn = logits.softmax(-1)
    dt = torch.bfloat16
    v, a, go = dev(value, dt), dev(attn, dt), dev(grad_out, dt)
    gv, gl, ga = abi_backward(v, dev(shapes), dev(starts), dev(loc, torch.float32), a, go)
    t_gv, t_gl, t_ga = orc.backward(v.cpu(), shapes, starts, loc, a.cpu(), go.cpu())
    assert rel_err(to_np(gv), t_gv) <= 1e-2
    assert rel_err(to_np(gl), t_gl) <= 1e-2 and rel_err(to_np(ga), t_ga) <= 1e-2
    # sample by sample as well: an error confined to a few samples would vanish in the global norm
    g = to_np(gv).reshape(B, -1)
    t = np.asarray(t_gv).reshape(B, -1)
    worst = np.max(np.abs(g - t), axis=1) / (np.max(np.abs(t), axis=1) + 1e-30)
    assert worst.max() <= 2e-2, (int(worst.argmax()), float(worst.max()))


@pytest.mark.parametrize("dtype,exponent", [
    (torch.bfloat16, -14), (torch.bfloat16, 0), (torch.bfloat16, 12),
    # (float16 itself ends at 65504: at 2^12 the true grad_attn no longer fits the dtype)
    (torch.float16, -14), (torch.float16, 0), (torch.float16, 8)])
def test_grad_value_accuracy_does_not_depend_on_the_magnitude_of_grad_out(dtype, exponent):
    """The scaled float16 accumulation picks its power of two from the largest |grad_out| of the
    call, so a gradient thousands of times larger (loss scaling) or 2^14 times smaller neither
    overflows the float16 sums nor loses them to underflow: same relative error as at 1."""
    value, shapes, starts, loc, logits, grad_out = _case(
        9, 2, 1200, 8, 32, 4, [(20, 20), (10, 10), (5, 5)], spread=1.0)
    attn = logits.softmax(-1)
    scaled = grad_out * 2.0 ** exponent
    v, a, go = dev(value, dtype), dev(attn, dtype), dev(scaled, dtype)
    l, sh, st = dev(loc, torch.float32), dev(shapes), dev(starts)
    gv, gl, ga = abi_backward(v, sh, st, l, a, go)
    truth, t_gl, t_ga = orc.backward(v.cpu(), shapes, starts, l.cpu(), a.cpu(), go.cpu())
    assert torch.isfinite(gv).all()
    assert rel_err(to_np(gv), truth) <= 1e-2
    assert rel_err(to_np(ga), t_ga) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_degenerate_grad_out_zero_and_non_finite(dtype):
    """The power of two of the float16 accumulation comes from max|grad_out|: an all-zero
    gradient (nothing to scale by) must give exactly zero gradients, and an ``inf`` in grad_out
    (no finite scale exists) must neither fault nor leak into samples it does not belong to."""
    value, shapes, starts, loc, logits, grad_out = _case(
        13, 2, 300, 8, 32, 4, [(10, 10), (5, 5)], spread=1.0)
    attn = logits.softmax(-1)
    v, a = dev(value, dtype), dev(attn, dtype)
    l, sh, st = dev(loc, torch.float32), dev(shapes), dev(starts)
    gv, gl, ga = abi_backward(v, sh, st, l, a, dev(torch.zeros_like(grad_out), dtype))
    assert not gv.any() and not gl.any() and not ga.any()
    bad = grad_out.clone()
    bad[1, 7, 5] = float("inf")                              # one element of sample 1
    gv, gl, ga = abi_backward(v, sh, st, l, a, dev(bad, dtype))
    torch.cuda.synchronize()
    # sample 0 never sees that element: all of its gradients stay finite and accurate
    truth, t_gl, t_ga = orc.backward(v.cpu()[:1], shapes, starts, l.cpu()[:1], a.cpu()[:1],
                                     dev(grad_out, dtype).cpu()[:1])
    assert torch.isfinite(gv[0]).all() and torch.isfinite(gl[0]).all() and torch.isfinite(ga[0]).all()
    assert rel_err(to_np(gv[:1]), truth) <= 2e-2
    assert rel_err(to_np(ga[:1]), t_ga) <= 1e-2
    assert not torch.isfinite(gv[1]).all()                   # and sample 1 shows it
