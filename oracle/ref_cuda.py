"""TEST INFRASTRUCTURE - run the REFERENCE's own CUDA kernels (built by ``build_ref.py``).

The reference registers its kernels against operator schemas that its Python side defines
first (``sources/deformops/backends/cuda/_schema.py:18-71``); this module defines the same
schemas for the two configurations in ``oracle/_ref/`` and loads the libraries, so the
kernels can be called as ``torch.ops.deformops_cuda.<prefix>_{forward,backward}`` without
importing the reference package (which does not travel to the GPU box).

Operand preparation follows the reference's functional entry and autograd closure
(``_msda_bridge.py:232-259``, ``:411-448``): the production configuration ``msda_fp32acc``
upcasts value, locations, weights and grad_output to float32 for its backward and casts the
gradients back; ``msda_half2atomic`` keeps the 16-bit operands.  Only tests and the same-box
timing script use this module.
"""

from __future__ import annotations

import pathlib

import torch

_REF = pathlib.Path(__file__).resolve().parent / "_ref"
_NS = "deformops_cuda"
_FWD = ("(Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor loc, Tensor attn, "
        "int chunk_step, int K, int channels_per_thread, int threads_per_block) -> Tensor")
_BWD = ("(Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor loc, Tensor attn, "
        "Tensor grad_output, int chunk_step, int K, int channels_per_thread, "
        "int threads_per_block) -> (Tensor, Tensor, Tensor)")
PREFIXES = ("msda_fp32acc", "msda_half2atomic")
_loaded: set[str] = set()


def available(prefix: str = "msda_fp32acc") -> bool:
    return (_REF / f"{prefix}.so").exists()


def load(prefix: str) -> None:
    if prefix in _loaded:
        return
    if not available(prefix):
        raise FileNotFoundError(f"{_REF / (prefix + '.so')} missing: run oracle/build_ref.py "
                                "where the reference checkout is available")
    ns = getattr(torch.ops, _NS)
    for marker in ("", "_softmax"):
        for direction, schema in (("forward", _FWD), ("backward", _BWD)):
            name = f"{prefix}{marker}_{direction}"
            if not hasattr(ns, name):
                torch.library.define(f"{_NS}::{name}", schema)
    torch.ops.load_library(str(_REF / f"{prefix}.so"))
    _loaded.add(prefix)


def _op(prefix: str, softmax: bool, direction: str):
    load(prefix)
    return getattr(getattr(torch.ops, _NS), f"{prefix}{'_softmax' if softmax else ''}_{direction}")


def _loc_for(value, loc):
    """Locations as the reference's op wants them: float32, or float64 beside float64 values
    (``msda_launch.cuh:54-61``)."""
    return loc.to(torch.float64 if value.dtype == torch.float64 else torch.float32).contiguous()


def forward(value, shapes, starts, loc, attn, *, softmax=False, prefix="msda_fp32acc",
            chunk_step=128):
    K = loc.shape[4]
    with torch.autocast("cuda", enabled=False):
        return _op(prefix, softmax, "forward")(
            value.contiguous(), shapes.to(torch.int64), starts.to(torch.int64),
            _loc_for(value, loc), attn.contiguous().type_as(value), chunk_step, K, 0, 0)


def backward(value, shapes, starts, loc, attn, grad_out, *, softmax=False,
             prefix="msda_fp32acc", chunk_step=128):
    """Gradients ``(grad_value, grad_loc, grad_attn)`` in the dtypes of the inputs."""
    K = loc.shape[4]
    # the production configuration upcasts 16-bit operands to float32; float64 stays float64
    upcast = prefix == "msda_fp32acc" and value.dtype != torch.float64
    cast = (lambda t: t.float()) if upcast else (lambda t: t)
    with torch.autocast("cuda", enabled=False):
        gv, gl, ga = _op(prefix, softmax, "backward")(
            cast(value.contiguous()), shapes.to(torch.int64), starts.to(torch.int64),
            _loc_for(value, loc), cast(attn.contiguous()),
            cast(grad_out.contiguous()), chunk_step, K, 0, 0)
    return gv.type_as(value), gl.type_as(loc), ga.type_as(attn)
