"""``run_msda``: the call third-party attention modules make once they have locations and weights.

Same keyword surface as the reference bridge (``sources/deformops/integrations/_ops.py:24-93``):
``level_start_index`` may be ``None`` (derived on the device from ``spatial_shapes``, no host
read), ``backend`` may be a ``Backend`` member, a backend object (called directly, without
operand checks) or ``None``, and ``method`` defaults to LINEAR because the Hugging Face
modules apply their softmax in torch before calling in
(``sources/deformops/integrations/transformers.py:188-231``).
"""

from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from ..core.runtime import Method
from ..registry.msda import Backend, MSDABackend, msda

__all__ = ["run_msda"]


def run_msda(value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor | None,
             sampling_locations: Tensor, attention_weights: Tensor, *, chunk_step: int,
             backend: "Backend | MSDABackend | None", method: "Method | str" = Method.LINEAR) -> Tensor:
    """``(B,S,G,D)`` value, ``(B,Q,G,L,K,2)`` locations, ``(B,Q,G,L*K)`` weights -> ``(B,Q,G*D)``."""
    if level_start_index is None:
        sizes = spatial_shapes[:, 0] * spatial_shapes[:, 1]
        level_start_index = torch.cumsum(sizes, 0) - sizes
    if isinstance(backend, MSDABackend):
        return backend.forward(value, spatial_shapes, level_start_index, sampling_locations,
                               attention_weights, chunk_step, Method(method))
    options: dict[str, Any] = {"method": method, "backend": backend}
    if backend is not None:
        options["chunk_step"] = chunk_step
    return msda(value, spatial_shapes, level_start_index, sampling_locations, attention_weights,
                **options)
