"""``MultiScaleDeformAttn2d``: the deformable-attention layer on top of the sm_100a operator.

Same constructor, forward signature, parameter names and state-dict behaviour as the
reference layer (``sources/deformops/nn/msda.py:24-273``), so a checkpoint of either loads into
the other and a model can swap the class without further edits:

* four linears ``proj_offset`` (``G*L*K*2``), ``proj_weights`` (``G*L*K``), ``proj_value``,
  ``proj_output``; Deformable-DETR initialisation (zero offset weights, offset biases on a
  ring of ``G`` directions scaled by the point index, zero weight logits, Xavier projections);
* reference points ``(B, Q, L, 2)`` take offsets in pixels of each level, boxes
  ``(B, Q, L, 4)`` place samples at ``centre + offset / K * size / 2``;
* ``padding_mask`` zeroes projected value tokens before sampling;
* ``load_state_dict`` renames Deformable-DETR keys (``sampling_offsets``,
  ``attention_weights``, ``value_proj``, ``output_proj``) for metadata versions below 2.

The sampling itself is one call of :func:`deformops_b200.registry.msda_from_offsets` (default
``method="softmax"``: the logits are normalised and the offsets added to the reference points
inside the kernel; neither normalised weights nor a location tensor are materialised).
"""

from __future__ import annotations

import math
from typing import Any

import torch
from torch import Tensor, nn

from ..core.runtime import Method
from ..registry.msda import Backend, MSDABackend, msda, msda_from_offsets

__all__ = ["MultiScaleDeformAttn2d"]

_DETR_NAMES = {"sampling_offsets": "proj_offset", "attention_weights": "proj_weights",
               "value_proj": "proj_value", "output_proj": "proj_output"}


def _check_layer_sizes(dim: int, num_heads: int, num_levels: int, num_points: int) -> None:
    for name, v in (("dim", dim), ("num_heads", num_heads), ("num_levels", num_levels),
                    ("num_points", num_points)):
        if not isinstance(v, int) or v <= 0:
            raise ValueError(f"{name} must be a positive integer, got {v!r}")
    if dim % num_heads:
        raise ValueError(f"dim ({dim}) must be divisible by num_heads ({num_heads})")
    head = dim // num_heads
    if head & (head - 1):
        raise ValueError(f"dim // num_heads = {head} must be a power of two")


class MultiScaleDeformAttn2d(nn.Module):
    """Multi-scale deformable attention layer (Deformable DETR) running on the B200 kernels."""

    _version = 2

    def __init__(self, dim: int, dim_value: int | None = None, dim_output: int | None = None, *,
                 num_heads: int, num_levels: int, num_points: int = 4,
                 method: "Method | str" = Method.SOFTMAX,
                 backend: "Backend | MSDABackend | None" = None, chunk_step: int = 128):
        super().__init__()
        _check_layer_sizes(dim, num_heads, num_levels, num_points)
        self.dim, self.num_heads = dim, num_heads
        self.num_levels, self.num_points = num_levels, num_points
        self.method = Method(method)
        self.backend = backend
        self.chunk_step = chunk_step
        #: let the kernels do the location arithmetic (set False to build locations in torch)
        self.fuse_locations = True

        samples = num_heads * num_levels * num_points
        self.proj_offset = nn.Linear(dim, samples * 2)
        self.proj_weights = nn.Linear(dim, samples)
        self.proj_value = nn.Linear(dim_value or dim, dim)
        self.proj_output = nn.Linear(dim, dim_output or dim)
        self._register_load_state_dict_pre_hook(self._rename_detr_keys)
        self.reset_parameters()

    # -- checkpoints ---------------------------------------------------------------------
    def _rename_detr_keys(self, state_dict: dict[str, Tensor], prefix: str,
                          local_metadata: dict[str, Any], *_: Any, **__: Any) -> None:
        version = local_metadata.get("version", 1)
        if isinstance(version, int) and version >= self._version:
            return
        for old, new in _DETR_NAMES.items():
            for part in ("weight", "bias"):
                key = f"{prefix}{old}.{part}"
                if key in state_dict:
                    state_dict[f"{prefix}{new}.{part}"] = state_dict.pop(key)

    # -- initialisation ------------------------------------------------------------------
    @torch.no_grad()
    def reset_parameters(self) -> None:
        G, L, K = self.num_heads, self.num_levels, self.num_points
        angle = torch.arange(G, dtype=torch.float32) * (2.0 * math.pi / G)
        ring = torch.stack([angle.cos(), angle.sin()], dim=-1)
        ring = ring / ring.abs().amax(dim=-1, keepdim=True)          # on the unit square
        steps = torch.arange(1, K + 1, dtype=torch.float32).view(1, 1, K, 1)
        bias = ring.view(G, 1, 1, 2).expand(G, L, K, 2) * steps      # point k sits k+1 steps out
        self.proj_offset.weight.zero_()
        self.proj_offset.bias.copy_(bias.reshape(-1))
        self.proj_weights.weight.zero_()
        self.proj_weights.bias.zero_()
        for proj in (self.proj_value, self.proj_output):
            nn.init.xavier_uniform_(proj.weight)
            proj.bias.zero_()

    # -- forward -------------------------------------------------------------------------
    def sampling_locations(self, q: Tensor, p: Tensor, spatial_shapes: Tensor) -> Tensor:
        """``(B, Q, G, L, K, 2)`` normalised sample locations predicted from the queries."""
        B, Q, _ = q.shape
        offset = self.proj_offset(q).view(B, Q, self.num_heads, self.num_levels,
                                          self.num_points, 2)
        ref = p[:, :, None, :, None, :]
        if p.shape[-1] == 2:
            wh = spatial_shapes.flip(-1).to(offset.dtype)             # (L, 2) as (width, height)
            return ref + offset / wh[None, None, None, :, None, :]
        if p.shape[-1] == 4:
            return ref[..., :2] + offset / self.num_points * ref[..., 2:] * 0.5
        raise ValueError(f"reference points must end in 2 or 4 coordinates, got {p.shape[-1]}")

    def forward(self, q: Tensor, p: Tensor, v: Tensor, spatial_shapes: Tensor,
                level_start_index: Tensor, padding_mask: Tensor | None = None) -> Tensor:
        """``q (B,Q,dim)``, ``p (B,Q,L,2|4)``, ``v (B,N,dim_value)`` -> ``(B,Q,dim_output)``."""
        B, Q, _ = q.shape
        N = v.shape[1]
        value = self.proj_value(v)
        if padding_mask is not None:
            value = value.masked_fill(padding_mask[..., None], 0.0)
        value = value.view(B, N, self.num_heads, self.dim // self.num_heads)
        weights = self.proj_weights(q).view(B, Q, self.num_heads,
                                            self.num_levels * self.num_points)

        if isinstance(self.backend, MSDABackend):
            locations = self.sampling_locations(q, p, spatial_shapes)
            out = self.backend.forward(value, spatial_shapes, level_start_index, locations,
                                       weights, self.chunk_step, self.method)
        elif self.fuse_locations:
            # the kernels add the offsets to the reference points themselves; no location
            # tensor is built
            msda._only_cuda(self.backend)
            offset = self.proj_offset(q).view(B, Q, self.num_heads, self.num_levels,
                                              self.num_points, 2)
            out = msda_from_offsets(value, spatial_shapes, level_start_index, p, offset, weights,
                                    method=self.method)
        else:
            locations = self.sampling_locations(q, p, spatial_shapes)
            options: dict[str, Any] = {"method": self.method, "backend": self.backend}
            if self.backend is not None:
                options["chunk_step"] = self.chunk_step
            out = msda(value, spatial_shapes, level_start_index, locations, weights, **options)
        return self.proj_output(out)
