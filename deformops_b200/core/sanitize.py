"""Structural checks on the operands of an MSDA call, run before any launch.

Same contract as ``check_msda_call`` in the reference
(``sources/deformops/core/sanitize.py:276-436``): every structural mismatch raises
``ValueError`` naming the first offending operand; only metadata is read, so the checks
never synchronise with the device.  The checks that read the level table back to the host
(positive sizes, exclusive prefix sum, coverage of ``value``) run only when the
environment variable ``DEFORMOPS_VALIDATE`` is set to a true value, because they do
synchronise.
"""

from __future__ import annotations

import os

import torch
from torch import Tensor

__all__ = ["check_msda_call", "value_checks_enabled"]


def value_checks_enabled() -> bool:
    return os.environ.get("DEFORMOPS_VALIDATE", "0").strip().lower() in {"1", "true", "yes", "on"}


def _need_rank(name: str, t: Tensor, ranks: tuple[int, ...], layout: str) -> None:
    if t.dim() not in ranks:
        want = " or ".join(str(r) for r in ranks)
        raise ValueError(
            f"{name} must have {want} dimensions {layout}, got {t.dim()} with shape {tuple(t.shape)}"
        )


def _need_size(name: str, t: Tensor, axis: int, size, why: str) -> None:
    if t.shape[axis] != size:
        raise ValueError(
            f"{name} has size {t.shape[axis]} on axis {axis} but {size} is required ({why}); "
            f"shape {tuple(t.shape)}"
        )


def check_msda_call(value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor,
                    sampling_locations: Tensor, attention_weights: Tensor) -> None:
    """Validate ``(B,S,G,D)``, ``(L,2)``, ``(L,)``, ``(B,Q,G,L,K,2)`` and ``(B,Q,G,L*K)`` / ``(B,Q,G,L,K)``."""
    _need_rank("value", value, (4,), "(B, S, G, D)")
    _need_rank("spatial_shapes", spatial_shapes, (2,), "(L, 2)")
    _need_rank("level_start_index", level_start_index, (1,), "(L,)")
    _need_rank("sampling_locations", sampling_locations, (6,), "(B, Q, G, L, K, 2)")
    _need_rank("attention_weights", attention_weights, (4, 5), "(B, Q, G, L * K) or (B, Q, G, L, K)")

    _need_size("spatial_shapes", spatial_shapes, 1, 2, "each row is (height, width)")
    _need_size("sampling_locations", sampling_locations, 5, 2, "each location is an (x, y) pair")

    B, _, G, _ = value.shape
    L = spatial_shapes.shape[0]
    _, Q, _, loc_levels, K, _ = sampling_locations.shape
    _need_size("level_start_index", level_start_index, 0, L, "one entry per level")
    _need_size("sampling_locations", sampling_locations, 0, B, "batch of value")
    _need_size("sampling_locations", sampling_locations, 2, G, "heads of value")
    _need_size("sampling_locations", sampling_locations, 3, L, "rows of spatial_shapes")
    _need_size("attention_weights", attention_weights, 0, B, "batch of value")
    _need_size("attention_weights", attention_weights, 1, Q, "queries of sampling_locations")
    _need_size("attention_weights", attention_weights, 2, G, "heads of value")
    if attention_weights.dim() == 4:
        _need_size("attention_weights", attention_weights, 3, loc_levels * K,
                   "levels x points of sampling_locations")
    else:
        _need_size("attention_weights", attention_weights, 3, loc_levels,
                   "levels of sampling_locations")
        _need_size("attention_weights", attention_weights, 4, K, "points of sampling_locations")

    for name, t in (("spatial_shapes", spatial_shapes), ("level_start_index", level_start_index)):
        if t.is_floating_point() or t.is_complex() or t.dtype == torch.bool:
            raise ValueError(f"{name} must be an integer tensor (it indexes value), got {t.dtype}")
    for name, t in (("value", value), ("attention_weights", attention_weights),
                    ("sampling_locations", sampling_locations)):
        if not t.is_floating_point():
            raise ValueError(f"{name} must be a floating-point tensor, got dtype {t.dtype}")
    # the kernels read the weights at the value's width; locations may differ (autocast)
    if attention_weights.dtype != value.dtype:
        raise ValueError(
            f"attention_weights has dtype {attention_weights.dtype} but value has {value.dtype}; "
            "mixed input dtypes are not supported: cast to a common dtype or use autocast"
        )
    devices = {
        "value": value.device, "spatial_shapes": spatial_shapes.device,
        "level_start_index": level_start_index.device,
        "sampling_locations": sampling_locations.device,
        "attention_weights": attention_weights.device,
    }
    if len(set(devices.values())) != 1:
        listing = ", ".join(f"{k} on {v}" for k, v in devices.items())
        raise ValueError(f"all operands must be on one device, got {listing}")

    if value_checks_enabled() and not _is_fake(spatial_shapes) and not _is_fake(level_start_index):
        _check_level_layout(value, spatial_shapes, level_start_index)


def _is_fake(t: Tensor) -> bool:
    return t.device.type == "meta" or type(t).__name__ in {"FakeTensor", "FunctionalTensor"}


def _check_level_layout(value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor) -> None:
    """The level table must tile ``value`` exactly; the kernels index from it unchecked."""
    shapes = spatial_shapes.detach().cpu().tolist()
    starts = level_start_index.detach().cpu().tolist()
    running, expected = 0, []
    for level, (h, w) in enumerate(shapes):
        if h <= 0 or w <= 0:
            raise ValueError(f"spatial_shapes row {level} is ({h}, {w}); sizes must be positive")
        expected.append(running)
        running += h * w
    if starts != expected:
        raise ValueError(
            f"level_start_index {starts} is not the exclusive prefix sum of the level sizes "
            f"{[h * w for h, w in shapes]}; expected {expected}"
        )
    if running != value.shape[1]:
        raise ValueError(
            f"spatial_shapes describes {running} positions but value has {value.shape[1]} on "
            "its spatial axis; the levels must tile the value tensor exactly"
        )
