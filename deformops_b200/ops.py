"""``torch.library`` registration of the MSDA operators on top of the C-ABI shim.

Private ops (namespace ``deformops_b200``), same schemas as the reference's
``deformops_cuda::<prefix>_{forward,backward}`` (``sources/deformops/backends/cuda/_schema.py:18-29``):

    msda_forward / msda_softmax_forward
        (value, spatial_shapes, level_start_index, loc, attn,
         int chunk_step, int K, int channels_per_thread, int threads_per_block) -> Tensor
    msda_backward / msda_softmax_backward
        (…same five…, grad_output, int chunk_step, int K, int channels_per_thread,
         int threads_per_block) -> (Tensor, Tensor, Tensor)

``chunk_step``, ``channels_per_thread`` and ``threads_per_block`` are accepted for schema
compatibility and have no effect: the kernels take the whole batch in one launch and pick
their own geometry.  The CUDA implementations allocate outputs with torch and pass raw
pointers plus the current stream to ``libmsda_b200.so``; there is no other implementation
(a CPU tensor reaching these ops is an error).  Meta kernels and the autograd formula
follow ``sources/deformops/backends/cuda/_msda_bridge.py:146-299``.

``msda_offsets_forward`` / ``msda_offsets_backward`` have no counterpart in the reference: they
take reference points and predicted offsets instead of locations (see further down).

Public ops ``deformops_b200::msda`` and ``deformops_b200::msda_softmax`` take the five
tensors only (``sources/deformops/registry/msda.py:366-412``); they are
CompositeImplicitAutograd over the private ops and carry a vmap rule that folds the
mapped axis into the batch with the level tables shared
(``sources/deformops/registry/_vmap.py:19-82``).
"""

from __future__ import annotations

import ctypes
from typing import Any, Callable

import torch
from torch import Tensor
from torch.autograd.function import once_differentiable

from ._loader import load_library

__all__ = ["NAMESPACE", "OFFSETS_OPS", "PRIVATE_OPS", "PUBLIC_OPS", "DTYPE_CODES",
           "define_reference_op_names",
           "launch_counter"]

NAMESPACE = "deformops_b200"

_FORWARD_SCHEMA = (
    "(Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor loc, Tensor attn, "
    "int chunk_step, int K, int channels_per_thread, int threads_per_block) -> Tensor"
)
_BACKWARD_SCHEMA = (
    "(Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor loc, Tensor attn, "
    "Tensor grad_output, int chunk_step, int K, int channels_per_thread, "
    "int threads_per_block) -> (Tensor, Tensor, Tensor)"
)
_PUBLIC_SCHEMA = (
    "(Tensor value, Tensor spatial_shapes, Tensor level_start_index, "
    "Tensor sampling_locations, Tensor attention_weights) -> Tensor"
)

PRIVATE_OPS = ("msda_forward", "msda_backward", "msda_softmax_forward", "msda_softmax_backward")
PUBLIC_OPS = ("msda", "msda_softmax")

#: dtype codes of ``enum msda_b200_dtype``
DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.float64: 3}

_FORWARD_INPUTS = 9


class _LaunchCounter:
    """Counts launches issued through this module: forward 1 kernel; backward with the scaled
    float16 scratch 3 kernels (prepare, backward, finalize) and a 256-byte memset of the scratch
    header, else 1 kernel and 1 memset of grad_value."""

    def __init__(self) -> None:
        self.kernels = 0
        self.memsets = 0

    def reset(self) -> None:
        self.kernels = 0
        self.memsets = 0


launch_counter = _LaunchCounter()


def _ptr(t: Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _aligned(t: Tensor) -> Tensor:
    # torch allocations are 512-byte aligned; only an offset view can break 16-byte alignment
    return t if t.data_ptr() % 16 == 0 else t.clone(memory_format=torch.contiguous_format)


def _check_operands(value: Tensor, shapes: Tensor, starts: Tensor, loc: Tensor, attn: Tensor,
                    K: int) -> tuple[int, int, int, int, int, int, int]:
    """The private ops' preconditions (the reference's C++ TORCH_CHECKs raise RuntimeError too)."""
    if not value.is_cuda:
        raise RuntimeError("deformops_b200 kernels run on CUDA tensors only (there is no CPU path)")
    if value.dtype not in DTYPE_CODES:
        raise RuntimeError(f"unsupported value dtype {value.dtype}; use float32, float16, "
                           "bfloat16 or float64")
    # float64 values come with float64 locations (the gradcheck configuration)
    loc_dtype = torch.float64 if value.dtype == torch.float64 else torch.float32
    if loc.dtype != loc_dtype:
        raise RuntimeError(f"sampling locations must be {loc_dtype} for {value.dtype} values, "
                           f"got {loc.dtype}")
    if attn.dtype != value.dtype:
        raise RuntimeError(f"attention weights must have the value dtype {value.dtype}, got {attn.dtype}")
    if shapes.dtype != torch.int64 or starts.dtype != torch.int64:
        raise RuntimeError("spatial_shapes and level_start_index must be int64")
    for name, t in (("value", value), ("spatial_shapes", shapes), ("level_start_index", starts),
                    ("loc", loc), ("attn", attn)):
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
        if t.device != value.device:
            raise RuntimeError(f"{name} is on {t.device}, value on {value.device}")
    B, S, G, D = value.shape
    _, Q, _, L, K_loc, _ = loc.shape
    if K != K_loc:
        raise RuntimeError(f"K={K} does not match the locations' {K_loc} points per level")
    return B, S, G, D, Q, L, K


def _raise(shim, status: int, what: str) -> None:
    msg = f"{what} failed with status {status}: {shim.last_error()}"
    raise ValueError(msg) if status in (-1, -2) else RuntimeError(msg)


def _make_forward(softmax: bool) -> Callable[..., Tensor]:
    def forward_cuda(value, spatial_shapes, level_start_index, loc, attn, chunk_step, K,
                     channels_per_thread, threads_per_block):
        B, S, G, D, Q, L, K = _check_operands(value, spatial_shapes, level_start_index, loc, attn, K)
        out = torch.empty((B, Q, G * D), dtype=value.dtype, device=value.device)
        if B == 0 or Q == 0:
            return out
        shim = load_library()
        value, loc, attn = _aligned(value), _aligned(loc), _aligned(attn)
        stream = torch.cuda.current_stream(value.device).cuda_stream
        st = shim.forward(_ptr(value), _ptr(spatial_shapes), _ptr(level_start_index), _ptr(loc),
                          _ptr(attn), _ptr(out), B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype],
                          int(softmax), value.device.index, ctypes.c_void_p(stream))
        if st != 0:
            _raise(shim, st, "msda_b200_forward")
        launch_counter.kernels += 1
        return out

    return forward_cuda


def _make_backward(softmax: bool) -> Callable[..., tuple[Tensor, Tensor, Tensor]]:
    def backward_cuda(value, spatial_shapes, level_start_index, loc, attn, grad_output,
                      chunk_step, K, channels_per_thread, threads_per_block):
        B, S, G, D, Q, L, K = _check_operands(value, spatial_shapes, level_start_index, loc, attn, K)
        if grad_output.dtype != value.dtype or not grad_output.is_contiguous():
            raise RuntimeError("grad_output must be contiguous and have the value dtype")
        grad_value = torch.empty_like(value)
        grad_loc = torch.empty_like(loc)
        grad_attn = torch.empty_like(attn)
        if B == 0:
            return grad_value, grad_loc, grad_attn
        shim = load_library()
        value, loc, attn, grad_output = map(_aligned, (value, loc, attn, grad_output))
        stream = torch.cuda.current_stream(value.device).cuda_stream
        # scratch of a 16-bit backward (one float16 image of grad_value plus a header); comes
        # from torch's caching allocator, so steady-state calls reuse one block per stream
        nbytes = shim.scratch_bytes(B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype]) if Q > 0 else 0
        scratch = (torch.empty(nbytes, dtype=torch.uint8, device=value.device)
                   if nbytes else None)
        st = shim.backward(_ptr(value), _ptr(spatial_shapes), _ptr(level_start_index), _ptr(loc),
                           _ptr(attn), _ptr(grad_output), _ptr(grad_value), _ptr(grad_loc),
                           _ptr(grad_attn), _ptr(scratch) if nbytes else None, nbytes, 0,
                           B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype],
                           int(softmax), 1, value.device.index, ctypes.c_void_p(stream))
        if st != 0:
            _raise(shim, st, "msda_b200_backward")
        launch_counter.kernels += (3 if nbytes else 1) if Q > 0 else 0
        launch_counter.memsets += 1
        return grad_value, grad_loc, grad_attn

    return backward_cuda


# --- fake-tensor (meta) kernels: shapes and dtypes of the real outputs --------------------
def _forward_meta(value, spatial_shapes, level_start_index, loc, attn, chunk_step, K,
                  channels_per_thread, threads_per_block):
    B, _, G, D = value.shape
    return value.new_empty((B, loc.shape[1], G * D))


def _backward_meta(value, spatial_shapes, level_start_index, loc, attn, grad_output, chunk_step,
                   K, channels_per_thread, threads_per_block):
    return (value.new_empty(value.shape), loc.new_empty(loc.shape), attn.new_empty(attn.shape))


# --- autograd ---------------------------------------------------------------------------------
def _setup_context(ctx: Any, inputs: tuple[Any, ...], output: Tensor) -> None:
    if len(inputs) != _FORWARD_INPUTS:
        raise RuntimeError(f"msda setup_context received {len(inputs)} inputs, expected "
                           f"{_FORWARD_INPUTS}")
    # plain ints only: nothing here may specialise a trace on tensor sizes
    ctx.chunk_step = inputs[5]
    ctx.num_points = inputs[6]
    ctx.save_for_backward(*inputs[:5])


def _make_autograd_backward(backward_op: Callable[..., tuple[Tensor, Tensor, Tensor]]):
    @once_differentiable
    def backward(ctx: Any, grad_output: Tensor):
        value, shapes, starts, loc, attn = ctx.saved_tensors
        with torch.autocast("cuda", enabled=False):
            grad_value, grad_loc, grad_attn = backward_op(
                value, shapes, starts, loc, attn, grad_output.contiguous().type_as(value),
                ctx.chunk_step, ctx.num_points, 0, 0)
        grads: list[Tensor | None] = [None] * _FORWARD_INPUTS
        grads[0] = grad_value.type_as(value)
        grads[3] = grad_loc.type_as(loc)
        grads[4] = grad_attn.type_as(attn)
        return tuple(grads)

    return backward


def _define_private_ops() -> None:
    namespace = getattr(torch.ops, NAMESPACE)
    for marker, softmax in (("", False), ("_softmax", True)):
        fwd, bwd = f"msda{marker}_forward", f"msda{marker}_backward"
        if hasattr(namespace, fwd):  # survives importlib.reload
            continue
        torch.library.define(f"{NAMESPACE}::{fwd}", _FORWARD_SCHEMA)
        torch.library.define(f"{NAMESPACE}::{bwd}", _BACKWARD_SCHEMA)
        torch.library.impl(f"{NAMESPACE}::{fwd}", "CUDA")(_make_forward(softmax))
        torch.library.impl(f"{NAMESPACE}::{bwd}", "CUDA")(_make_backward(softmax))
        torch.library.register_fake(f"{NAMESPACE}::{fwd}")(_forward_meta)
        torch.library.register_fake(f"{NAMESPACE}::{bwd}")(_backward_meta)
        backward_op = getattr(getattr(torch.ops, NAMESPACE), bwd).default
        torch.library.register_autograd(
            f"{NAMESPACE}::{fwd}", _make_autograd_backward(backward_op),
            setup_context=_setup_context)


# --- ops with the layer's location arithmetic fused in -----------------------------------------
# No counterpart among the reference's operators: its layers compute
# ``reference_points + offsets / (W, H)`` (or the box form) in torch and hand the op a
# location tensor (``sources/deformops/nn/msda.py:222-239``).  These ops take the reference
# points and the predicted offsets instead; the kernels form each location in registers.
_OFFSETS_FORWARD_SCHEMA = (
    "(Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor reference_points, "
    "Tensor offsets, Tensor attn, bool softmax) -> Tensor"
)
_OFFSETS_BACKWARD_SCHEMA = (
    "(Tensor value, Tensor spatial_shapes, Tensor level_start_index, Tensor reference_points, "
    "Tensor offsets, Tensor attn, Tensor grad_output, bool softmax) -> (Tensor, Tensor, Tensor)"
)
OFFSETS_OPS = ("msda_offsets_forward", "msda_offsets_backward")


def _check_offsets_operands(value: Tensor, shapes: Tensor, starts: Tensor, ref: Tensor,
                            offsets: Tensor, attn: Tensor):
    if offsets.dtype != torch.float32 and offsets.dtype != value.dtype:
        raise RuntimeError(f"offsets must be float32 or the value dtype {value.dtype}, "
                           f"got {offsets.dtype}")
    if offsets.ndim != 6 or offsets.shape[-1] != 2:
        raise RuntimeError("offsets must be (B, Q, G, L, K, 2)")
    if not value.is_cuda:
        raise RuntimeError("deformops_b200 kernels run on CUDA tensors only (there is no CPU path)")
    if value.dtype not in DTYPE_CODES or value.dtype == torch.float64:
        raise RuntimeError(f"unsupported value dtype {value.dtype}; use float32, float16 or bfloat16")
    if attn.dtype != value.dtype:
        raise RuntimeError(f"attention weights must have the value dtype {value.dtype}, got {attn.dtype}")
    if shapes.dtype != torch.int64 or starts.dtype != torch.int64:
        raise RuntimeError("spatial_shapes and level_start_index must be int64")
    if ref.dtype != torch.float32:
        raise RuntimeError(f"reference points must be float32, got {ref.dtype}")
    for name, t in (("value", value), ("spatial_shapes", shapes), ("level_start_index", starts),
                    ("reference_points", ref), ("offsets", offsets), ("attn", attn)):
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
        if t.device != value.device:
            raise RuntimeError(f"{name} is on {t.device}, value on {value.device}")
    B, S, G, D = value.shape
    _, Q, _, L, K, _ = offsets.shape
    if ref.ndim != 4 or tuple(ref.shape[:3]) != (B, Q, L) or ref.shape[3] not in (2, 4):
        raise RuntimeError(f"reference points must be ({B}, {Q}, {L}, 2 or 4), got "
                           f"{tuple(ref.shape)}")
    return B, S, G, D, Q, L, K


def _offsets_forward_cuda(value, spatial_shapes, level_start_index, reference_points, offsets,
                          attn, softmax):
    B, S, G, D, Q, L, K = _check_offsets_operands(value, spatial_shapes, level_start_index,
                                                  reference_points, offsets, attn)
    out = torch.empty((B, Q, G * D), dtype=value.dtype, device=value.device)
    if B == 0 or Q == 0:
        return out
    shim = load_library()
    value, reference_points, offsets, attn = map(_aligned, (value, reference_points, offsets, attn))
    stream = torch.cuda.current_stream(value.device).cuda_stream
    st = shim.forward_offsets(_ptr(value), _ptr(spatial_shapes), _ptr(level_start_index),
                              _ptr(reference_points), reference_points.shape[3], _ptr(offsets),
                              DTYPE_CODES[offsets.dtype], _ptr(attn), _ptr(out), B, S, G, D, Q, L,
                              K, DTYPE_CODES[value.dtype], int(softmax), value.device.index,
                              ctypes.c_void_p(stream))
    if st != 0:
        _raise(shim, st, "msda_b200_forward_offsets")
    launch_counter.kernels += 1
    return out


def _offsets_backward_cuda(value, spatial_shapes, level_start_index, reference_points, offsets,
                           attn, grad_output, softmax):
    B, S, G, D, Q, L, K = _check_offsets_operands(value, spatial_shapes, level_start_index,
                                                  reference_points, offsets, attn)
    if grad_output.dtype != value.dtype or not grad_output.is_contiguous():
        raise RuntimeError("grad_output must be contiguous and have the value dtype")
    grad_value = torch.empty_like(value)
    grad_offsets = torch.empty_like(offsets)
    grad_attn = torch.empty_like(attn)
    if B == 0:
        return grad_value, grad_offsets, grad_attn
    shim = load_library()
    value, reference_points, offsets, attn, grad_output = map(
        _aligned, (value, reference_points, offsets, attn, grad_output))
    stream = torch.cuda.current_stream(value.device).cuda_stream
    nbytes = shim.scratch_bytes(B, S, G, D, Q, L, K, DTYPE_CODES[value.dtype]) if Q > 0 else 0
    scratch = (torch.empty(nbytes, dtype=torch.uint8, device=value.device)
               if nbytes else None)
    st = shim.backward_offsets(
        _ptr(value), _ptr(spatial_shapes), _ptr(level_start_index), _ptr(reference_points),
        reference_points.shape[3], _ptr(offsets), DTYPE_CODES[offsets.dtype], _ptr(attn),
        _ptr(grad_output), _ptr(grad_value), _ptr(grad_offsets), _ptr(grad_attn),
        _ptr(scratch) if nbytes else None, nbytes, 0, B, S, G, D, Q, L, K,
        DTYPE_CODES[value.dtype], int(softmax), 1, value.device.index, ctypes.c_void_p(stream))
    if st != 0:
        _raise(shim, st, "msda_b200_backward_offsets")
    launch_counter.kernels += (3 if nbytes else 1) if Q > 0 else 0
    launch_counter.memsets += 1
    return grad_value, grad_offsets, grad_attn


def _offsets_forward_meta(value, spatial_shapes, level_start_index, reference_points, offsets,
                          attn, softmax):
    B, _, G, D = value.shape
    return value.new_empty((B, offsets.shape[1], G * D))


def _offsets_backward_meta(value, spatial_shapes, level_start_index, reference_points, offsets,
                           attn, grad_output, softmax):
    return (value.new_empty(value.shape), offsets.new_empty(offsets.shape),
            attn.new_empty(attn.shape))


def _offsets_setup_context(ctx: Any, inputs: tuple[Any, ...], output: Tensor) -> None:
    ctx.softmax = inputs[6]
    ctx.save_for_backward(*inputs[:6])


def _make_offsets_autograd_backward(backward_op):
    @once_differentiable
    def backward(ctx: Any, grad_output: Tensor):
        value, shapes, starts, ref, offsets, attn = ctx.saved_tensors
        with torch.autocast("cuda", enabled=False):
            grad_value, grad_offsets, grad_attn = backward_op(
                value, shapes, starts, ref, offsets, attn,
                grad_output.contiguous().type_as(value), ctx.softmax)
        grad_ref = None
        if ctx.needs_input_grad[3]:
            if ref.shape[-1] != 2:
                raise RuntimeError(
                    "msda_offsets: no gradient is produced for 4-coordinate reference boxes; "
                    "compute the locations in torch and call msda for that case")
            # d(location)/d(reference) = 1 and location gradient = offset gradient * (W, H)
            wh = shapes.flip(-1).to(torch.float32)
            grad_ref = (grad_offsets.to(torch.float32)
                        * wh[None, None, None, :, None, :]).sum(dim=(2, 4))
        return grad_value, None, None, grad_ref, grad_offsets, grad_attn, None

    return backward


def _define_offsets_ops() -> None:
    namespace = getattr(torch.ops, NAMESPACE)
    fwd, bwd = OFFSETS_OPS
    if hasattr(namespace, fwd):
        return
    torch.library.define(f"{NAMESPACE}::{fwd}", _OFFSETS_FORWARD_SCHEMA)
    torch.library.define(f"{NAMESPACE}::{bwd}", _OFFSETS_BACKWARD_SCHEMA)
    torch.library.impl(f"{NAMESPACE}::{fwd}", "CUDA")(_offsets_forward_cuda)
    torch.library.impl(f"{NAMESPACE}::{bwd}", "CUDA")(_offsets_backward_cuda)
    torch.library.register_fake(f"{NAMESPACE}::{fwd}")(_offsets_forward_meta)
    torch.library.register_fake(f"{NAMESPACE}::{bwd}")(_offsets_backward_meta)
    backward_op = getattr(getattr(torch.ops, NAMESPACE), bwd).default
    torch.library.register_autograd(
        f"{NAMESPACE}::{fwd}", _make_offsets_autograd_backward(backward_op),
        setup_context=_offsets_setup_context)


# --- public ops -------------------------------------------------------------------------------
#: kept for the life of the process: a collected Library unregisters its operators
_PUBLIC_LIBRARY: "torch.library.Library | None" = None

_SHARED_ARGS = {1: "spatial_shapes", 2: "level_start_index"}


def _vmap_rule(op: Callable[..., Tensor]):
    """Fold the mapped axis into the batch, run the op once, unfold the result."""

    def rule(info: Any, in_dims: tuple[Any, ...], *args: Tensor):
        size = info.batch_size
        folded = []
        for index, (arg, dim) in enumerate(zip(args, in_dims)):
            if index in _SHARED_ARGS:
                if dim is not None:
                    raise ValueError(
                        f"{_SHARED_ARGS[index]} is shared by the whole batch and cannot be vmapped")
                folded.append(arg)
            elif dim is None:
                folded.append(arg.unsqueeze(0).expand(size, *arg.shape).flatten(0, 1))
            else:
                folded.append(arg.movedim(dim, 0).flatten(0, 1))
        out = op(*folded)
        return out.unflatten(0, (size, -1)), 0

    return rule


def _define_public_ops() -> None:
    global _PUBLIC_LIBRARY
    namespace = getattr(torch.ops, NAMESPACE)
    if hasattr(namespace, "msda"):
        return
    from .registry.msda import _public_kernel  # late: registry imports this module
    from .core.runtime import Method

    lib = torch.library.Library(NAMESPACE, "FRAGMENT")
    for name, method in (("msda", Method.LINEAR), ("msda_softmax", Method.SOFTMAX)):
        lib.define(name + _PUBLIC_SCHEMA)
        lib.impl(name, _public_kernel(method), "CompositeImplicitAutograd")
        op = getattr(getattr(torch.ops, NAMESPACE), name)
        torch.library.register_vmap(f"{NAMESPACE}::{name}", _vmap_rule(op), lib=lib)
    _PUBLIC_LIBRARY = lib


#: kept for the life of the process, like _PUBLIC_LIBRARY
_REFERENCE_NAMES_LIBRARY: "torch.library.Library | None" = None


def define_reference_op_names() -> bool:
    """Offer the public operators under the REFERENCE's names as well, ``deformops::msda`` and
    ``deformops::msda_softmax`` (same schema: ``sources/deformops/registry/msda.py:366-412``,
    ``registry/_public_ops.py:28-67``), so that a program exported or traced against the
    reference runs in a process that has this package but not the reference.

    Explicit, not done at import: the reference defines its operators idempotently by name
    (``_public_ops.py:58-60``), so whoever defines the names first keeps them.  Returns False,
    and changes nothing, when the names already exist (the reference is imported)."""
    global _REFERENCE_NAMES_LIBRARY
    if hasattr(torch.ops, "deformops") and hasattr(torch.ops.deformops, "msda"):
        return False
    _define_public_ops()
    from .core.runtime import Method
    from .registry.msda import _public_kernel

    lib = torch.library.Library("deformops", "FRAGMENT")
    for name, method in (("msda", Method.LINEAR), ("msda_softmax", Method.SOFTMAX)):
        lib.define(name + _PUBLIC_SCHEMA)
        lib.impl(name, _public_kernel(method), "CompositeImplicitAutograd")
        op = getattr(torch.ops.deformops, name)
        torch.library.register_vmap(f"deformops::{name}", _vmap_rule(op), lib=lib)
    _REFERENCE_NAMES_LIBRARY = lib
    return True


_define_private_ops()
_define_offsets_ops()
