"""The MSDA functional, its call context and the single backend behind it.

Keeps the operator surface of the reference's ``deformops.registry.msda``
(``sources/deformops/registry/msda.py:40-146`` context and protocol, ``:274-356`` functional
signature, ``:366-412`` public ops) and of its CUDA functional entry
(``sources/deformops/backends/cuda/_msda_bridge.py:368-448``).  What is dropped on purpose
is the selection policy: there is one backend, the sm_100a kernels; no Triton, no eager, no
fallback.  ``backend`` is accepted so call sites need no edit: ``None`` and ``Backend.CUDA``
both run the kernels, any other member raises :class:`NoBackendError`.
"""

from __future__ import annotations

import abc
import dataclasses
import enum
from typing import Any, Protocol, runtime_checkable

import torch
from torch import Tensor

from .. import ops as _ops
from .._loader import load_library
from ..core.errors import NoBackendError
from ..core.runtime import Method, is_training_from, resolve_method, sm_version_for
from ..core.sanitize import check_msda_call

__all__ = [
    "Backend", "MSDABackend", "MSDAContext", "MSDAMethod", "apply_msda_method", "forward",
    "locations_from_offsets", "msda", "msda_from_offsets", "resolve_method", "supports_context",
]

MSDAMethod = Method


class Backend(enum.StrEnum):
    """Backend names of the reference (``registry/_dispatch.py:35-40``); only CUDA exists here."""

    CUDA = enum.auto()
    TRITON = enum.auto()
    EAGER = enum.auto()


@dataclasses.dataclass(frozen=True)
class MSDAContext:
    """What a backend needs to know to accept or refuse a call."""

    device: torch.device
    num_levels: int
    num_heads: int
    num_points: int
    dtype: torch.dtype
    sm_version: tuple[int, int]
    is_training: bool
    num_queries: int = dataclasses.field(compare=False)
    method: Method = Method.LINEAR
    #: channels per head; 0 when unknown
    head_dim: int = 0

    @classmethod
    def from_call(cls, value: Tensor, spatial_shapes: Tensor, sampling_locations: Tensor,
                  attention_weights: Tensor, method: Method) -> "MSDAContext":
        queries = sampling_locations.shape[1]
        return cls(
            device=value.device,
            num_levels=int(spatial_shapes.shape[0]),
            num_heads=int(value.shape[2]),
            num_points=int(sampling_locations.shape[4]),
            dtype=value.dtype,
            sm_version=sm_version_for(value.device),
            is_training=is_training_from(value, sampling_locations, attention_weights),
            num_queries=0 if isinstance(queries, torch.SymInt) else int(queries),
            method=method,
            head_dim=int(value.shape[3]),
        )


@runtime_checkable
class MSDABackend(Protocol):
    """Interface of a backend object handed to a layer (``registry/msda.py:91-146``)."""

    @property
    @abc.abstractmethod
    def name(self) -> str: ...

    @abc.abstractmethod
    def supports(self, context: MSDAContext) -> bool: ...

    @abc.abstractmethod
    def forward(self, value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor,
                sampling_locations: Tensor, attention_weights: Tensor, chunk_step: int,
                method: Method) -> Tensor: ...


#: channels per 16-byte vector; float64 runs on the simple gradcheck kernels (any head size)
_VECTOR = {torch.float32: 4, torch.float16: 8, torch.bfloat16: 8, torch.float64: 1}
_MAX_LEVELS = 16


def unsupported_reason(context: MSDAContext) -> str | None:
    """Why the kernels cannot take this call, or ``None`` if they can."""
    if context.device.type != "cuda":
        return f"tensors are on {context.device}; the kernels need a CUDA device (no CPU path)"
    if context.sm_version[0] != 10:
        return (f"device has compute capability {context.sm_version[0]}.{context.sm_version[1]}; "
                "the kernels are built for sm_100a only")
    if context.dtype not in _VECTOR:
        return f"dtype {context.dtype} is not float32, float16, bfloat16 or float64"
    if context.head_dim and context.head_dim % _VECTOR[context.dtype] != 0:
        return (f"head dimension {context.head_dim} is not a multiple of "
                f"{_VECTOR[context.dtype]} (16-byte channel vectors)")
    if not 1 <= context.num_levels <= _MAX_LEVELS:
        return f"{context.num_levels} levels; 1 to {_MAX_LEVELS} are supported"
    if context.num_points < 1:
        return "at least one point per level is required"
    return None


def supports_context(context: MSDAContext) -> bool:
    return unsupported_reason(context) is None


def apply_msda_method(attention_weights: Tensor, method: "str | Method") -> Tensor:
    """Normalise raw weights in torch (for callers that want the linear op afterwards)."""
    method = Method(method)
    if method is Method.LINEAR:
        return attention_weights
    if attention_weights.ndim == 5:
        return torch.softmax(attention_weights.flatten(-2), -1).unflatten(
            -1, attention_weights.shape[-2:])
    if attention_weights.ndim != 4:
        raise ValueError("attention weights must be (B, Q, G, L * K) or (B, Q, G, L, K); got "
                         f"{attention_weights.ndim} dimensions.")
    return torch.softmax(attention_weights, -1)


def forward(value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor,
            sampling_locations: Tensor, attention_weights: Tensor, chunk_step: int = 128, *,
            num_points: int | None = None, channels_per_thread: int = 0,
            threads_per_block: int = 0, softmax: bool = False) -> Tensor:
    """Differentiable MSDA on the sm_100a kernels, without structural operand checks.

    Makes operands kernel-ready the way the reference's functional entry does
    (``_msda_bridge.py:411-448``): contiguous tensors, int64 level tables (converted on the
    device, no host synchronisation), float32 locations (float64 for float64 values), weights
    in the value dtype, autocast
    disabled around the op; empty batch or zero queries return zeros without a launch.
    The weights may be ``(B,Q,G,L*K)`` or ``(B,Q,G,L,K)``; their gradient comes back in the
    shape and dtype given.
    """
    if value.device.type != "cuda":
        raise NoBackendError("deformops_b200 runs on CUDA tensors only; there is no CPU path")
    value = value.contiguous()
    spatial_shapes = spatial_shapes.to(torch.int64).contiguous()
    level_start_index = level_start_index.to(torch.int64).contiguous()
    sampling_locations = sampling_locations.contiguous()
    attention_weights = attention_weights.contiguous()

    B, _, G, D = value.shape
    Q = sampling_locations.shape[1]
    if Q == 0 or B == 0:
        return value.new_zeros((B, Q, G * D))
    if num_points is None:
        num_points = sampling_locations.shape[4]

    load_library()
    op = (torch.ops.deformops_b200.msda_softmax_forward if softmax
          else torch.ops.deformops_b200.msda_forward)
    with torch.autocast("cuda", enabled=False):
        result = op(value, spatial_shapes, level_start_index,
                    sampling_locations.to(torch.float64 if value.dtype == torch.float64
                                          else torch.float32),
                    attention_weights.type_as(value),
                    chunk_step, num_points, channels_per_thread, threads_per_block)
        return result.type_as(value)


class CudaBackend(MSDABackend):
    """The backend object a layer can hold (``MSDABackend`` protocol)."""

    @property
    def name(self) -> str:
        return "cuda_b200"

    def supports(self, context: MSDAContext) -> bool:
        return supports_context(context)

    def forward(self, value, spatial_shapes, level_start_index, sampling_locations,
                attention_weights, chunk_step, method) -> Tensor:
        return forward(value, spatial_shapes, level_start_index, sampling_locations,
                       attention_weights, chunk_step,
                       softmax=Method(method) is Method.SOFTMAX)


_CALL_OPTIONS = frozenset({"chunk_step", "num_points", "channels_per_thread", "threads_per_block",
                           "fp32acc"})


class _MSDA:
    """Callable with the reference's functional signature plus ``load`` / ``context_of``."""

    backend = CudaBackend()

    def load(self, backend: Backend | None = None, **_: Any) -> str:
        """Load the kernel library now (otherwise the first call does); returns its path."""
        self._only_cuda(backend)
        return load_library().path

    @staticmethod
    def _only_cuda(backend: Any) -> None:
        if backend is None:
            return
        if isinstance(backend, str) and not isinstance(backend, Backend):
            raise TypeError(f"backend must be a Backend member or None, got the string {backend!r}")
        if not isinstance(backend, Backend):
            raise TypeError(f"backend must be a Backend member or None, got {type(backend).__name__}")
        if backend is not Backend.CUDA:
            raise NoBackendError(
                f"backend {backend.value!r} is not part of this build: only the sm_100a CUDA "
                "kernels exist (no Triton, no eager, no fallback)")

    def context_of(self, value, spatial_shapes, level_start_index=None, sampling_locations=None,
                   attention_weights=None, *, method=None, softmax=False, **options) -> MSDAContext:
        if level_start_index is None or sampling_locations is None or attention_weights is None:
            raise TypeError("msda takes (values, spatial_shapes, level_start_index, "
                            "sampling_locations, attention_weights) positionally")
        unknown = set(options) - _CALL_OPTIONS
        if unknown:
            raise TypeError("msda got unexpected keyword argument(s): " + ", ".join(sorted(unknown)))
        check_msda_call(value, spatial_shapes, level_start_index, sampling_locations,
                        attention_weights)
        return MSDAContext.from_call(value, spatial_shapes, sampling_locations, attention_weights,
                                     resolve_method(method, softmax=softmax))

    def __call__(self, value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor = None,
                 sampling_locations: Tensor = None, attention_weights: Tensor = None, /, *,
                 method: "str | Method | None" = None, softmax: bool = False,
                 backend: Backend | None = None, **options: Any) -> Tensor:
        """Multi-scale deformable attention: ``(B,S,G,D)`` value sampled at
        ``(B,Q,G,L,K,2)`` locations with ``(B,Q,G,L*K)`` weights -> ``(B,Q,G*D)``.

        ``method="softmax"`` (or ``softmax=True``) normalises the weights over the ``L*K``
        points inside the kernel.  ``chunk_step`` and the launch-geometry keywords of the
        reference are accepted and ignored.  Raises ``TypeError`` for a string backend, a
        missing operand or an unknown keyword; ``ValueError`` for operands that disagree in
        rank, size, dtype or device; :class:`NoBackendError` when the kernels cannot take
        the call (the message says why).
        """
        self._only_cuda(backend)
        context = self.context_of(value, spatial_shapes, level_start_index, sampling_locations,
                                  attention_weights, method=method, softmax=softmax, **options)
        reason = unsupported_reason(context)
        if reason is not None:
            raise NoBackendError(f"msda cannot run this call: {reason}")
        use_softmax = context.method is Method.SOFTMAX
        if backend is None and not (set(options) - {"chunk_step"}):
            # like the reference's backend=None route (registry/msda.py:415-452): go through the
            # public operator, so that Dynamo and torch.export record `deformops_b200::msda`
            op = (torch.ops.deformops_b200.msda_softmax if use_softmax
                  else torch.ops.deformops_b200.msda)
            return op(value, spatial_shapes, level_start_index, sampling_locations,
                      attention_weights)
        return forward(value, spatial_shapes, level_start_index, sampling_locations,
                       attention_weights, options.get("chunk_step", 128),
                       num_points=options.get("num_points"), softmax=use_softmax)


msda = _MSDA()


def locations_from_offsets(reference_points: Tensor, offsets: Tensor,
                           spatial_shapes: Tensor) -> Tensor:
    """The layers' location arithmetic in torch (``sources/deformops/nn/msda.py:222-239``):
    ``(B,Q,L,2|4)`` reference points and ``(B,Q,G,L,K,2)`` offsets -> ``(B,Q,G,L,K,2)``."""
    ref = reference_points[:, :, None, :, None, :]
    if reference_points.shape[-1] == 2:
        wh = spatial_shapes.flip(-1).to(offsets.dtype)                # (L, 2) as (width, height)
        return ref + offsets / wh[None, None, None, :, None, :]
    if reference_points.shape[-1] == 4:
        return ref[..., :2] + offsets / offsets.shape[4] * ref[..., 2:] * 0.5
    raise ValueError("reference points must end in 2 or 4 coordinates, got "
                     f"{reference_points.shape[-1]}")


def msda_from_offsets(value: Tensor, spatial_shapes: Tensor, level_start_index: Tensor,
                      reference_points: Tensor, offsets: Tensor, attention_weights: Tensor, *,
                      method: "str | Method | None" = None, softmax: bool = False) -> Tensor:
    """MSDA straight from what a deformable-attention layer predicts.

    ``reference_points (B,Q,L,2|4)`` and ``offsets (B,Q,G,L,K,2)`` take the place of the
    sampling locations; the kernels compute ``ref + offsets / (W, H)`` (two coordinates) or
    ``ref.xy + offsets / K * ref.wh / 2`` (boxes) per point in float32, so the location
    tensor and its gradient are never materialised.  Offsets may stay in the value dtype
    (their gradient then comes back in it) or be float32.  Gradients flow to value, offsets
    and weights, and to two-coordinate reference points; boxes that require a gradient take
    the unfused route (locations in torch, then :data:`msda`).
    """
    resolved = resolve_method(method, softmax=softmax)
    if reference_points.ndim != 4 or reference_points.shape[-1] not in (2, 4):
        raise ValueError("reference points must be (B, Q, L, 2) or (B, Q, L, 4); got "
                         f"{tuple(reference_points.shape)}")
    if offsets.ndim == 6 and tuple(reference_points.shape[:3]) != (
            offsets.shape[0], offsets.shape[1], offsets.shape[3]):
        raise ValueError(f"reference points {tuple(reference_points.shape)} do not match offsets "
                         f"{tuple(offsets.shape)} in batch, queries or levels")
    check_msda_call(value, spatial_shapes, level_start_index, offsets, attention_weights)
    if reference_points.device != value.device:
        raise ValueError(f"reference points are on {reference_points.device}, value on "
                         f"{value.device}")
    context = MSDAContext.from_call(value, spatial_shapes, offsets, attention_weights, resolved)
    reason = unsupported_reason(context)
    if reason is not None:
        raise NoBackendError(f"msda cannot run this call: {reason}")
    needs_box_gradient = (reference_points.shape[-1] == 4 and reference_points.requires_grad
                          and torch.is_grad_enabled())
    if needs_box_gradient or value.dtype == torch.float64:
        # float64 (numerical differentiation) runs on the location kernels only
        work = torch.float64 if value.dtype == torch.float64 else torch.float32
        locations = locations_from_offsets(reference_points.to(work), offsets.to(work),
                                           spatial_shapes)
        return msda(value, spatial_shapes, level_start_index, locations, attention_weights,
                    method=resolved)

    B, _, G, D = value.shape
    Q = offsets.shape[1]
    if Q == 0 or B == 0:
        return value.new_zeros((B, Q, G * D))
    load_library()
    value = value.contiguous()
    if offsets.dtype != value.dtype:
        offsets = offsets.to(torch.float32)
    weights = attention_weights.contiguous()
    with torch.autocast("cuda", enabled=False):
        out = torch.ops.deformops_b200.msda_offsets_forward(
            value, spatial_shapes.to(torch.int64).contiguous(),
            level_start_index.to(torch.int64).contiguous(),
            reference_points.to(torch.float32).contiguous(), offsets.contiguous(),
            weights.flatten(-2).type_as(value) if weights.ndim == 5 else weights.type_as(value),
            resolved is Method.SOFTMAX)
        return out.type_as(value)


def _public_kernel(method: Method):
    """Kernel of the public operator for one aggregation method (CompositeImplicitAutograd)."""

    def kernel(value, spatial_shapes, level_start_index, sampling_locations, attention_weights):
        check_msda_call(value, spatial_shapes, level_start_index, sampling_locations,
                        attention_weights)
        return forward(value, spatial_shapes, level_start_index, sampling_locations,
                       attention_weights, softmax=method is Method.SOFTMAX)

    return kernel


_ops._define_public_ops()
