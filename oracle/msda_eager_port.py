"""TEST INFRASTRUCTURE - torch restatement of the reference's eager (pure PyTorch) MSDA.

The reference's CPU path is ``sources/deformops/backends/eager/msda_pytorch.py:23-112``:
pixel coordinates for every (query, head, level, point) at once, four clamped
advanced-index gathers that each materialise an ``[N, Q, M, L, P, D]`` tensor, two-sided
validity masks, a weighted sum, and torch autograd for the backward.  This module restates
that algorithm (same tensor shapes, same number of gathers) so the benchmark can time "the
reference's CPU implementation" on machines where the reference is not installed.  It is
checked against the fixtures the reference produced in ``tests/test_oracle_golden.py``.
Only tests and the benchmark's CPU-baseline leg import it.
"""

from __future__ import annotations

import torch
from torch import Tensor


def eager_forward(value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor,
                  loc: Tensor, attn: Tensor, *, softmax: bool = False) -> Tensor:
    """``(N,S,M,D)`` value, ``(N,Q,M,L,P,2)`` locations, ``(N,Q,M,L*P)`` weights -> ``(N,Q,M*D)``."""
    N, _, M, D = value.shape
    _, Q, _, L, P, _ = loc.shape
    if softmax:
        attn = torch.softmax(attn.reshape(N, Q, M, L * P), -1)
    attn = attn.reshape(N, Q, M, L, P)

    dt = value.dtype
    bshape = (1, 1, 1, L, 1)
    Hi = spatial_shapes[:, 0].long().view(bshape)
    Wi = spatial_shapes[:, 1].long().view(bshape)
    first = level_start_index.long().view(bshape)

    # pixel = loc * size - 0.5, two rounded operations (msda_pytorch.py:64-66)
    px = loc[..., 0] * Wi.to(dt) - 0.5
    py = loc[..., 1] * Hi.to(dt) - 0.5
    cx = px.floor()
    cy = py.floor()
    tx = px - cx
    ty = py - cy
    cx = cx.long()
    cy = cy.long()

    batch = torch.arange(N, device=value.device).view(N, 1, 1, 1, 1)
    head = torch.arange(M, device=value.device).view(1, 1, M, 1, 1)

    def corner(ix: Tensor, iy: Tensor, w: Tensor) -> Tensor:
        inside = (ix >= 0) & (ix < Wi) & (iy >= 0) & (iy < Hi)
        flat = first + iy.clamp(min=0).minimum(Hi - 1) * Wi + ix.clamp(min=0).minimum(Wi - 1)
        picked = value[batch, flat, head]                      # [N, Q, M, L, P, D]
        return picked * (w * inside.to(dt)).unsqueeze(-1)

    sampled = (corner(cx, cy, (1 - tx) * (1 - ty)) + corner(cx + 1, cy, tx * (1 - ty))
               + corner(cx, cy + 1, (1 - tx) * ty) + corner(cx + 1, cy + 1, tx * ty))
    out = (sampled * attn.unsqueeze(-1)).sum(dim=(3, 4))       # [N, Q, M, D]
    return out.reshape(N, Q, M * D)


def eager_forward_backward(value, spatial_shapes, level_start_index, loc, attn, grad_out, *,
                           softmax=False):
    """Forward plus torch-autograd backward; returns ``(out, grad_value, grad_loc, grad_attn)``."""
    v = value.detach().clone().requires_grad_(True)
    l = loc.detach().clone().requires_grad_(True)
    a = attn.detach().clone().requires_grad_(True)
    out = eager_forward(v, spatial_shapes, level_start_index, l, a, softmax=softmax)
    out.backward(grad_out)
    return out.detach(), v.grad, l.grad, a.grad
