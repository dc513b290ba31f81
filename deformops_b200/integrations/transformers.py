"""Hugging Face multi-scale deformable attention on the sm_100a operator.

Drop-in subclasses of the two Hugging Face classes the reference replaces
(``sources/deformops/integrations/transformers.py:62-235``) plus ``patch(model)``:

* :class:`MultiScaleDeformableAttention` - Deformable DETR's parameter-free attention core
  (``forward(value, value_spatial_shapes, value_spatial_shapes_list, level_start_index,
  sampling_locations, attention_weights, im2col_step)``): weights arrive already softmaxed,
  so it runs the LINEAR operator.
* :class:`Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention` - the pixel-decoder
  attention with its projections.  The reference computes the softmax over the ``L*K``
  logits in torch and then calls the linear operator (``transformers.py:188-193``); here the
  raw logits go to the SOFTMAX operator, which normalises inside the kernel, so one
  elementwise pass over the weights disappears from forward and backward.  The normalised
  weights are only materialised when the caller asks for them (``output_attentions``).
  The location arithmetic (``reference_points + offsets / (W, H)``, ``transformers.py:195-218``)
  is fused the same way: offsets and reference points go to the kernel as they are and no
  location tensor is written or read back.

Parameters keep their Hugging Face names, so pretrained checkpoints load unchanged.
"""

from __future__ import annotations

from typing import Any

import torch
from torch import Tensor, nn

from ..core.runtime import Method
from ..registry.msda import (Backend, MSDABackend, locations_from_offsets, msda,
                             msda_from_offsets)
from ._ops import run_msda

try:
    import transformers.models.deformable_detr.modeling_deformable_detr as _hf_detr
    import transformers.models.mask2former.modeling_mask2former as _hf_m2f

    _HF_CORE = _hf_detr.MultiScaleDeformableAttention
    _HF_M2F = _hf_m2f.Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention
except (ImportError, AttributeError) as exc:  # pragma: no cover - optional dependency
    raise ImportError(
        "deformops_b200.integrations.transformers needs a transformers release that defines "
        "MultiScaleDeformableAttention and "
        f"Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention ({exc})") from exc

__all__ = ["Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention",
           "MultiScaleDeformableAttention", "patch"]


class MultiScaleDeformableAttention(_HF_CORE):
    """Parameter-free attention core: samples ``value`` with given locations and weights."""

    def __init__(self, *, backend: "Backend | MSDABackend | None" = None) -> None:
        super().__init__()
        self.backend = backend

    def forward(self, value: Tensor, value_spatial_shapes: Tensor,
                value_spatial_shapes_list: Any, level_start_index: Tensor | None,
                sampling_locations: Tensor, attention_weights: Tensor,
                im2col_step: int) -> Tensor:
        if value_spatial_shapes is None:
            value_spatial_shapes = torch.tensor(list(value_spatial_shapes_list), dtype=torch.int64,
                                                device=value.device)
        return run_msda(value, value_spatial_shapes, level_start_index, sampling_locations,
                        attention_weights, chunk_step=im2col_step, backend=self.backend,
                        method=Method.LINEAR)


class Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention(_HF_M2F):
    """Mask2Former pixel-decoder attention; projections and parameter names as upstream."""

    def __init__(self, embed_dim: int, num_heads: int, n_levels: int, n_points: int, *,
                 backend: "Backend | MSDABackend | None" = None) -> None:
        super().__init__(embed_dim, num_heads, n_levels, n_points)
        self.backend = backend

    def forward(self, hidden_states: Tensor, attention_mask: Tensor | None = None,
                encoder_hidden_states: Tensor | None = None, encoder_attention_mask: Any = None,
                position_embeddings: Tensor | None = None, reference_points: Tensor | None = None,
                spatial_shapes_list: Any = None, level_start_index: Tensor | None = None,
                output_attentions: bool = False, **_: Any):
        if position_embeddings is not None:
            hidden_states = hidden_states + position_embeddings
        B, Q, _ = hidden_states.shape
        S = encoder_hidden_states.shape[1]
        G, L, K = self.n_heads, self.n_levels, self.n_points
        shapes = torch.tensor([list(s) for s in spatial_shapes_list], dtype=torch.int64,
                              device=hidden_states.device)

        value = self.value_proj(encoder_hidden_states)
        if attention_mask is not None:
            value = value.masked_fill(attention_mask[..., None], 0.0)
        value = value.view(B, S, G, self.d_model // G)
        offsets = self.sampling_offsets(hidden_states).view(B, Q, G, L, K, 2)
        logits = self.attention_weights(hidden_states).view(B, Q, G, L * K)

        if reference_points.shape[-1] not in (2, 4):
            raise ValueError("Last dim of reference_points must be 2 or 4, but got "
                             f"{reference_points.shape[-1]}")
        if isinstance(self.backend, MSDABackend):
            locations = locations_from_offsets(reference_points, offsets, shapes)
            out = run_msda(value, shapes, level_start_index, locations, logits,
                           chunk_step=self.im2col_step, backend=self.backend,
                           method=Method.SOFTMAX)
        else:
            # softmax and `reference + offsets / (W, H)` both happen inside the kernel
            msda._only_cuda(self.backend)
            if level_start_index is None:
                sizes = shapes[:, 0] * shapes[:, 1]
                level_start_index = torch.cumsum(sizes, 0) - sizes
            out = msda_from_offsets(value, shapes, level_start_index, reference_points, offsets,
                                    logits, method=Method.SOFTMAX)
        weights = torch.softmax(logits, -1).view(B, Q, G, L, K) if output_attentions else None
        return self.output_proj(out), weights


def patch(model: nn.Module, *, backend: "Backend | MSDABackend | None" = None) -> nn.Module:
    """Replace every Hugging Face MSDA module inside ``model`` in place; returns ``model``.

    Modules with parameters are rebuilt with the same sizes and take over the original
    parameter tensors (no copy), so optimizers and checkpoints keep working.
    """

    def convert(module: nn.Module) -> nn.Module | None:
        if isinstance(module, (MultiScaleDeformableAttention,
                               Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention)):
            return None
        if isinstance(module, _HF_M2F):
            new = Mask2FormerPixelDecoderEncoderMultiscaleDeformableAttention(
                module.d_model, module.n_heads, module.n_levels, module.n_points, backend=backend)
            for name in ("sampling_offsets", "attention_weights", "value_proj", "output_proj"):
                setattr(new, name, getattr(module, name))
            new.im2col_step = module.im2col_step
            new.train(module.training)
            return new
        if isinstance(module, _HF_CORE):
            new = MultiScaleDeformableAttention(backend=backend)
            new.train(module.training)
            return new
        return None

    def visit(parent: nn.Module) -> None:
        for name, child in list(parent.named_children()):
            replacement = convert(child)
            if replacement is not None:
                setattr(parent, name, replacement)
            else:
                visit(child)

    visit(model)
    return model
