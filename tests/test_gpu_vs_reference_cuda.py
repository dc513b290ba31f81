"""GPU parity against the REFERENCE'S OWN CUDA KERNELS on the same inputs, on the same GPU.

``oracle/_ref/*.so`` are the reference's kernels compiled from its sources by
``oracle/build_ref.py``; the tests are skipped when they have not been built.  Tolerances:
float32 output 1e-5 and gradients 1e-4 of the reference's float32 CUDA result; bf16 / f16
1e-2 of the reference's float32 result on the same (rounded) inputs.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import ref_cuda
from tests._abi import abi_backward, abi_forward, dev, to_np
from tests._golden import rel_err
from tests.test_gpu_parity import _stable_points

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref not built")]


def _inputs(name, dtype, batch=None):
    from deformops_b200.workloads import make_workload

    w = make_workload(name, batch=batch)
    t = dict(value=dev(w.value, dtype), loc=dev(w.sampling_locations, torch.float32),
             attn=dev(w.attention_weights, dtype), logits=dev(w.attention_logits, dtype),
             grad_out=dev(w.grad_output, dtype), shapes=dev(w.spatial_shapes),
             starts=dev(w.level_start_index))
    return w, t


def _compare(t, dtype, softmax, tol_out, tol_grad):
    attn = t["logits"] if softmax else t["attn"]
    args = (t["value"], t["shapes"], t["starts"], t["loc"], attn)
    out = abi_forward(*args, softmax=softmax)
    gv, gl, ga = abi_backward(*args, t["grad_out"], softmax=softmax)
    # the reference's float32 result on the inputs as the kernels see them
    f32 = [x.float() if x.is_floating_point() else x for x in args]
    r_out = ref_cuda.forward(*f32, softmax=softmax)
    r_gv, r_gl, r_ga = ref_cuda.backward(*f32, t["grad_out"].float(), softmax=softmax)
    keep = _stable_points(to_np(t["loc"]), to_np(t["shapes"]))[..., None]
    errs = {"out": rel_err(to_np(out), to_np(r_out)), "grad_value": rel_err(to_np(gv), to_np(r_gv)),
            "grad_loc": rel_err(to_np(gl) * keep, to_np(r_gl) * keep),
            "grad_attn": rel_err(to_np(ga), to_np(r_ga))}
    assert errs["out"] <= tol_out, errs
    assert max(errs["grad_value"], errs["grad_loc"], errs["grad_attn"]) <= tol_grad, errs
    return errs


@pytest.mark.parametrize("softmax", [False, True])
@pytest.mark.parametrize("name", ["cfg0_cpu_fp32", "cfg3_detr_enc_fp32"])
def test_fp32_against_reference_cuda(name, softmax):
    _, t = _inputs(name, torch.float32)
    _compare(t, torch.float32, softmax, 1e-5, 1e-4)


@pytest.mark.parametrize("name,dtype", [
    ("cfg1_m2f_512_bf16", torch.bfloat16), ("cfg2_m2f_1024_bf16", torch.bfloat16),
    ("cfg3_detr_enc_fp16", torch.float16), ("cfg3_detr_dec_fp16", torch.float16),
])
def test_16bit_against_reference_cuda_fp32_result(name, dtype):
    _, t = _inputs(name, dtype)
    _compare(t, dtype, False, 1e-2, 1e-2)


@pytest.mark.parametrize("batch", [16, 64])
def test_scaling_slices_against_reference_cuda(batch):
    """The slices a rank holds in the batch-sharded scaling sweep (global batch 64 over 8 ... 1
    GPUs: 8, 16, 32 or 64 samples of the headline shape per GPU), in one call each: the sample
    bases go past 2^31 bytes at these sizes and the scratch past a gigabyte.  Compared on the
    GPU (no host copies of the gigabyte tensors) with the reference's float32 CUDA result."""
    _, t = _inputs("cfg2_m2f_1024_bf16", torch.bfloat16, batch=batch)
    args = (t["value"], t["shapes"], t["starts"], t["loc"], t["attn"])
    out = abi_forward(*args)
    gv, gl, ga = abi_backward(*args, t["grad_out"])
    f32 = [x.float() if x.is_floating_point() else x for x in args]
    r_out = ref_cuda.forward(*f32)
    r_gv, r_gl, r_ga = ref_cuda.backward(*f32, t["grad_out"].float())

    def err(a, b):
        return float((a.double() - b.double()).abs().max() / b.double().abs().max())

    wh = torch.flip(t["shapes"], [-1]).double()[None, None, None, :, None, :]
    pix = t["loc"].double() * wh - 0.5
    keep = ((pix - pix.round()).abs() >= 1e-4).all(-1, keepdim=True)
    errs = {"out": err(out, r_out), "grad_value": err(gv, r_gv),
            "grad_loc": err(gl * keep, r_gl * keep), "grad_attn": err(ga, r_ga)}
    assert max(errs.values()) <= 1e-2, errs
    assert all(torch.isfinite(x).all() for x in (out, gv, gl, ga))


@pytest.mark.parametrize("softmax", [False, True])
def test_float64_against_reference_cuda_float64(softmax):
    """Both implementations in double precision on the same inputs: 1e-10 (the orders of the
    sums differ, nothing else)."""
    w, _ = _inputs("cfg0_cpu_fp32", torch.float64)
    f64 = torch.float64
    t = dict(value=dev(w.value, f64), loc=dev(w.sampling_locations, f64),
             attn=dev(w.attention_logits if softmax else w.attention_weights, f64),
             grad_out=dev(w.grad_output, f64), shapes=dev(w.spatial_shapes),
             starts=dev(w.level_start_index))
    args = (t["value"], t["shapes"], t["starts"], t["loc"], t["attn"])
    out = abi_forward(*args, softmax=softmax)
    gv, gl, ga = abi_backward(*args, t["grad_out"], softmax=softmax)
    r_out = ref_cuda.forward(*args, softmax=softmax)
    r_gv, r_gl, r_ga = ref_cuda.backward(*args, t["grad_out"], softmax=softmax)
    np64 = lambda x: x.detach().cpu().numpy().astype(np.float64)  # noqa: E731
    for mine, theirs in ((out, r_out), (gv, r_gv), (gl, r_gl), (ga, r_ga)):
        assert theirs.dtype == f64 or theirs.dtype == torch.float32
        assert rel_err(np64(mine), np64(theirs)) <= 1e-10
