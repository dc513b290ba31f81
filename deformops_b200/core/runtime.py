"""The aggregation-method enum and call-context helpers.

Mirrors ``sources/deformops/core/runtime.py:17-91`` of the reference: ``Method`` has the
string values ``"linear"`` and ``"softmax"`` and every ``method`` argument accepts the
member or its value; an explicit ``method`` wins over the ``softmax`` flag.
"""

from __future__ import annotations

import enum
import functools

import torch

__all__ = ["Method", "is_training_from", "resolve_method", "sm_version_for"]


class Method(enum.StrEnum):
    """How the per-point weights are normalised."""

    #: use the weights as given
    LINEAR = enum.auto()
    #: softmax jointly over the ``L * K`` points of each head, inside the kernel
    SOFTMAX = enum.auto()


def resolve_method(method: "str | Method | None", *, softmax: bool = False) -> Method:
    """An explicit ``method`` wins; otherwise ``softmax`` chooses; default is LINEAR."""
    if method is not None:
        return Method(method)
    return Method.SOFTMAX if softmax else Method.LINEAR


@functools.cache
def sm_version_for(device: torch.device) -> tuple[int, int]:
    """Compute capability of ``device``; ``(0, 0)`` off CUDA."""
    if device.type != "cuda" or not torch.cuda.is_available():
        return (0, 0)
    return torch.cuda.get_device_capability(device)


def is_training_from(*tensors: torch.Tensor) -> bool:
    """Whether a backward pass could run: grad mode on and an input that requires grad."""
    return torch.is_grad_enabled() and any(t.requires_grad for t in tensors)
