"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE LIBRARY.

Run where the reference checkout is available (it is imported read-only):

    python tests/golden/make_golden.py --reference /path/to/reference/sources

For every case the inputs are built here, then the reference computes

* ``out_eager``  - its eager backend (``registry.msda(..., backend=Backend.EAGER)``),
* ``out_gridsample`` - its ``grid_sample`` based definition of correct
  (``backends/reference/msda.py``), linear cases only,
* ``grad_value / grad_loc / grad_attn`` - torch autograd through the eager backend
  with the stored ``grad_out``,

all in float64 on CPU, for ``method="linear"`` and ``method="softmax"``.  The
fixtures travel with the repository; the reference itself does not, so nothing
else in the test-suite imports it.

Cases
-----
boundary      the reference's own known-answer table: a 4x4 map with value[s] = s and
              the 7x7 grid of locations that hit pixel -1, -0.5, 0, 1, 1.5, 3.5, 4.5
              (tests/deformops/test_msda_eager.py:54-80 in the reference)
small_*       the shape list of tests/deformops/test_msda_eager.py:39-46, locations
              uniform in [-0.1, 1.1]
ragged        non-square levels (7,5),(4,6),(1,1), locations in [-0.3, 1.3], plus one
              exact integer pixel, one pixel-coordinate -1 and one fully outside query
all_outside   every location far outside: exact zeros everywhere
k8_d64        8 points per level, 64 channels per head
cfg0          batch 2, levels 32/16/8 squared, 8 heads x 32, 4 points: the seeded
              workload generator of deformops_b200.workloads; inputs are regenerated
              from the seed (an input checksum is stored), outputs are stored for
              every 31st row plus float64 checksums of the full tensors
"""

from __future__ import annotations

import argparse
import os
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

CFG0_STRIDE = 31


def tables(levels):
    shapes = torch.tensor(levels, dtype=torch.int64).reshape(-1, 2)
    sizes = shapes[:, 0] * shapes[:, 1]
    return shapes, torch.cumsum(sizes, 0) - sizes


def random_case(seed, B, G, D, levels, K, Q, lo=-0.1, hi=1.1):
    g = torch.Generator().manual_seed(seed)
    L = len(levels)
    S = sum(h * w for h, w in levels)
    value = torch.randn(B, S, G, D, generator=g)
    loc = torch.rand(B, Q, G, L, K, 2, generator=g) * (hi - lo) + lo
    attn = torch.randn(B, Q, G, L * K, generator=g)
    grad_out = torch.randn(B, Q, G * D, generator=g)
    return value, loc, attn, grad_out


def run_reference(value, shapes, starts, loc, attn_raw, grad_out, method):
    """Reference eager forward + autograd backward in float64; grid_sample forward."""
    from deformops.backends.reference.msda import reference as grid_reference
    from deformops.registry import Backend, msda

    v = value.double().requires_grad_(True)
    l = loc.double().requires_grad_(True)
    a = attn_raw.double().requires_grad_(True)
    out = msda(v, shapes, starts, l, a, backend=Backend.EAGER, method=method)
    out.backward(grad_out.double())
    res = {
        "out_eager": out.detach().numpy(),
        "grad_value": v.grad.numpy(),
        "grad_loc": l.grad.numpy(),
        "grad_attn": a.grad.numpy(),
    }
    L, K = loc.shape[3], loc.shape[4]
    probs = a.detach().softmax(-1) if method == "softmax" else a.detach()
    res["out_gridsample"] = grid_reference(
        v.detach(), shapes, l.detach(), probs.unflatten(-1, (L, K))
    ).numpy()
    return res


def save_case(name, levels, value, loc, attn_linear, attn_logits, grad_out, store_inputs=True,
              subsample=None):
    shapes, starts = tables(levels)
    payload = {"spatial_shapes": shapes.numpy(), "level_start_index": starts.numpy()}
    if store_inputs:
        payload.update(value=value.numpy(), loc=loc.numpy(), attn_linear=attn_linear.numpy(),
                       attn_logits=attn_logits.numpy(), grad_out=grad_out.numpy())
    for method, attn in (("linear", attn_linear), ("softmax", attn_logits)):
        res = run_reference(value, shapes, starts, loc, attn, grad_out, method)
        for key, arr in res.items():
            if subsample is None:
                payload[f"{method}_{key}"] = arr
            else:
                flat = arr.reshape(arr.shape[0], arr.shape[1], -1)
                payload[f"{method}_{key}_rows"] = flat[:, ::subsample].copy()
                payload[f"{method}_{key}_sum"] = np.array(arr.sum(dtype=np.float64))
                payload[f"{method}_{key}_abssum"] = np.array(np.abs(arr).sum(dtype=np.float64))
    return payload


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DEFORMOPS_REFERENCE_SOURCES"),
                    help="directory that holds the reference's `deformops` package (its "
                         "`sources/`); default $DEFORMOPS_REFERENCE_SOURCES")
    args = ap.parse_args()
    if not args.reference:
        ap.error("pass --reference or set DEFORMOPS_REFERENCE_SOURCES")
    sys.path.insert(0, args.reference)
    torch.set_num_threads(4)

    # --- boundary known-answer table -------------------------------------------------
    H = W = 4
    coords = [0.0, 0.125, 0.375, 0.5, 1.0, -0.125, 1.25]
    pts = torch.tensor([(cx, cy) for cx in coords for cy in coords], dtype=torch.float32)
    value = torch.arange(H * W, dtype=torch.float32).view(1, H * W, 1, 1)
    loc = pts.view(1, 1, 1, 1, len(pts), 2)
    ones = torch.ones(1, 1, 1, len(pts))
    g = torch.Generator().manual_seed(11)
    np.savez_compressed(HERE / "boundary.npz", **save_case(
        "boundary", [(H, W)], value, loc, ones, torch.randn(1, 1, 1, len(pts), generator=g),
        torch.ones(1, 1, 1)))

    # --- small shapes ----------------------------------------------------------------
    small = [
        ("small_a", 1, 1, 16, [(8, 8)], 4, 5),
        ("small_b", 2, 4, 32, [(8, 8), (4, 4), (2, 2)], 4, 12),
        ("small_c", 1, 8, 16, [(7, 5), (3, 3)], 8, 9),
        ("small_d", 3, 2, 16, [(1, 1)], 1, 4),
        ("k8_d64", 2, 2, 64, [(9, 6), (5, 3)], 8, 7),
    ]
    for i, (name, B, G, D, levels, K, Q) in enumerate(small):
        value, loc, logits, grad_out = random_case(100 + i, B, G, D, levels, K, Q)
        np.savez_compressed(HERE / f"{name}.npz", **save_case(
            name, levels, value, loc, logits.softmax(-1), logits, grad_out))

    # --- ragged levels with hand-placed special points --------------------------------
    levels = [(7, 5), (4, 6), (1, 1)]
    value, loc, logits, grad_out = random_case(200, 2, 3, 8, levels, 3, 6, lo=-0.3, hi=1.3)
    # exact in float32 and float64 alike (level 1 has height 4): the fixtures must not
    # depend on which side of a skip boundary a rounding error lands
    loc[0, 0, 0, 1, 0] = torch.tensor([0.3, 0.375])            # pixel row 1 exactly
    loc[0, 0, 0, 1, 1] = torch.tensor([0.7, -0.125])           # pixel row -1 exactly (kept)
    loc[0, 1, 1, 1, 0] = torch.tensor([0.4, 0.875])            # pixel row H - 1 (far edge)
    loc[1, 2] = 7.0                                            # whole query outside
    np.savez_compressed(HERE / "ragged.npz", **save_case(
        "ragged", levels, value, loc, logits.softmax(-1), logits, grad_out))

    # --- everything outside -----------------------------------------------------------
    levels = [(4, 4)]
    value, loc, logits, grad_out = random_case(300, 1, 2, 16, levels, 4, 6)
    loc = torch.full_like(loc, 5.0)
    np.savez_compressed(HERE / "all_outside.npz", **save_case(
        "all_outside", levels, value, loc, logits.softmax(-1), logits, grad_out))

    # --- configuration 0 from the workload generator ------------------------------------
    from deformops_b200.workloads import CONFIGS, make_workload

    w = make_workload("cfg0_cpu_fp32", seed=0)
    payload = save_case("cfg0", CONFIGS["cfg0_cpu_fp32"]["levels"], w.value, w.sampling_locations,
                        w.attention_weights, w.attention_logits, w.grad_output,
                        store_inputs=False, subsample=CFG0_STRIDE)
    payload["input_checksum"] = np.array([
        w.value.double().sum().item(), w.sampling_locations.double().sum().item(),
        w.attention_weights.double().abs().sum().item(), w.attention_logits.double().sum().item(),
        w.grad_output.double().sum().item()])
    payload["row_stride"] = np.array(CFG0_STRIDE)
    np.savez_compressed(HERE / "cfg0.npz", **payload)

    for f in sorted(HERE.glob("*.npz")):
        print(f"{f.name:20s} {f.stat().st_size / 1024:8.1f} KiB")


if __name__ == "__main__":
    main()
