"""Space-filling-curve query ordering: an optional locality pre-pass for unordered queries.

Encoder queries enumerate the pixels of the pyramid, so neighbouring queries already sample
neighbouring pixels.  Decoder-style queries have no such order; sorting them along a Morton or
Hilbert curve of their mean sampling location makes consecutive warps touch nearby pixels of
``value``.  The operator treats queries independently, so the permutation changes the order of
the work and of the ``grad_value`` reductions, never the result.

Plays the role of the reference's experiment ``sources/deformops/backends/cuda/experimental/
_query_order.py`` (host-side sort, gather, run, scatter back) as a backend object that wraps
the sm_100a backend: hand ``ReorderingBackend()`` to a layer or to ``run_msda`` as ``backend``.
"""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from .core.runtime import Method
from .registry.msda import CudaBackend, MSDABackend, MSDAContext

__all__ = ["Curve", "ReorderingBackend", "curve_index", "query_permutation"]

Curve = Literal["morton", "hilbert"]


def _quantise(coord: Tensor, bits: int) -> Tensor:
    """[0, 1] (clamped; NaN -> 0) to integers in [0, 2^bits)."""
    cells = (1 << bits) - 1
    return (torch.nan_to_num(coord.float(), nan=0.0).clamp(0.0, 1.0) * cells).round().to(torch.int64)


def _spread_bits(v: Tensor) -> Tensor:
    """Insert a zero bit above every bit of a 16-bit integer (abcd -> 0a0b0c0d)."""
    v = (v | (v << 8)) & 0x00FF00FF
    v = (v | (v << 4)) & 0x0F0F0F0F
    v = (v | (v << 2)) & 0x33333333
    v = (v | (v << 1)) & 0x55555555
    return v


def _hilbert(ix: Tensor, iy: Tensor, bits: int) -> Tensor:
    """Distance along the Hilbert curve of order ``bits`` (quadrant by quadrant from the top
    bit down, reflecting and transposing the lower bits as the curve turns)."""
    d = torch.zeros_like(ix)
    for level in range(bits - 1, -1, -1):
        side = 1 << level
        rx = (ix >> level) & 1
        ry = (iy >> level) & 1
        d = d + side * side * ((3 * rx) ^ ry)
        low_x, low_y = ix & (side - 1), iy & (side - 1)
        # lower quadrants are transposed; the lower-right one is reflected first
        reflect = (ry == 0) & (rx == 1)
        low_x2 = torch.where(reflect, side - 1 - low_x, low_x)
        low_y2 = torch.where(reflect, side - 1 - low_y, low_y)
        transpose = ry == 0
        ix = torch.where(transpose, low_y2, low_x2)
        iy = torch.where(transpose, low_x2, low_y2)
    return d


def curve_index(x: Tensor, y: Tensor, curve: Curve = "morton", bits: int = 10) -> Tensor:
    """Position of normalised points ``(x, y)`` on a space-filling curve (int64, any shape)."""
    if not 1 <= bits <= 16:
        raise ValueError(f"bits must be between 1 and 16, got {bits}")
    ix, iy = _quantise(x, bits), _quantise(y, bits)
    if curve == "morton":
        return _spread_bits(ix) | (_spread_bits(iy) << 1)
    if curve == "hilbert":
        return _hilbert(ix, iy, bits)
    raise ValueError(f"curve must be 'morton' or 'hilbert', got {curve!r}")


def query_permutation(sampling_locations: Tensor, curve: Curve = "morton", bits: int = 10) -> Tensor:
    """``(B, Q)`` permutation that sorts each sample's queries along the curve, keyed by the
    query's mean location over heads, levels and points of ``(B,Q,G,L,K,2)`` locations."""
    centre = sampling_locations.detach().float().mean(dim=(2, 3, 4))
    key = curve_index(centre[..., 0], centre[..., 1], curve, bits)
    return torch.argsort(key, dim=1, stable=True)


def _take(t: Tensor, perm: Tensor) -> Tensor:
    index = perm.view(*perm.shape, *([1] * (t.ndim - 2))).expand(*perm.shape, *t.shape[2:])
    return torch.gather(t, 1, index)


class ReorderingBackend(MSDABackend):
    """Sort the queries along a curve, run the wrapped backend, put the rows back."""

    def __init__(self, curve: Curve = "morton", inner: MSDABackend | None = None, bits: int = 10):
        if curve not in ("morton", "hilbert"):
            raise ValueError(f"curve must be 'morton' or 'hilbert', got {curve!r}")
        self.curve, self.bits = curve, bits
        self.inner = inner if inner is not None else CudaBackend()

    @property
    def name(self) -> str:
        return f"{self.inner.name}+{self.curve}"

    def supports(self, context: MSDAContext) -> bool:
        return self.inner.supports(context)

    def forward(self, value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor,
                sampling_locations: Tensor, attention_weights: Tensor, chunk_step: int,
                method: Method) -> Tensor:
        perm = query_permutation(sampling_locations, self.curve, self.bits)
        out = self.inner.forward(value, spatial_shapes, level_start_index,
                                 _take(sampling_locations, perm), _take(attention_weights, perm),
                                 chunk_step, method)
        inverse = torch.empty_like(perm)
        inverse.scatter_(1, perm, torch.arange(perm.shape[1], device=perm.device)
                         .expand_as(perm))
        return _take(out, inverse)
