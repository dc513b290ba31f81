"""Plug the sm_100a kernels into an installed reference library (``deformops``).

``register_into_deformops()`` performs the call a backend module of the reference makes at
import time, ``msda.register(Backend.CUDA, fn, supports=, load=)``
(``sources/deformops/registry/_dispatch.py:169-205``; adapter shape
``sources/deformops/backends/cuda/msda.py:14-45``), so that every caller of the reference -
``deformops.registry.msda(..., backend=Backend.CUDA)``, ``MultiScaleDeformAttn2d``, the
Hugging Face attention replacements - runs these kernels without an edit.  The reference is
optional: without it the function raises ``ImportError``.
"""

from __future__ import annotations

from typing import Any

from .._loader import load_library
from ..core.runtime import Method, resolve_method
from ..registry.msda import forward as _forward
from ..registry.msda import unsupported_reason

__all__ = ["msda_b200_adapter", "register_into_deformops", "supports"]


def msda_b200_adapter(value: Any, spatial_shapes: Any, level_start_index: Any,
                      sampling_locations: Any, attention_weights: Any, *, chunk_step: int = 128,
                      num_points: int | None = None, channels_per_thread: int = 0,
                      threads_per_block: int = 0, method: Any = None, softmax: bool = False,
                      **kwargs: Any) -> Any:
    """Adapter with the keyword surface of the reference's ``msda_cuda``; launch-geometry
    keywords are accepted and ignored."""
    method = getattr(method, "value", method)   # the reference's own Method enum -> its string
    use_softmax = resolve_method(method, softmax=softmax) is Method.SOFTMAX
    return _forward(value, spatial_shapes, level_start_index, sampling_locations,
                    attention_weights, chunk_step, num_points=num_points, softmax=use_softmax)


def supports(context: Any) -> bool:
    """``supports`` callback: reads the fields the reference's ``MSDAContext`` shares with ours."""
    return unsupported_reason(context) is None


def _load(*, download: Any = None, compile: Any = None) -> str:
    return load_library(compile=None if compile is None else bool(compile)).path


def register_into_deformops() -> Any:
    """Register the adapter as ``Backend.CUDA`` of ``deformops.registry.msda``; returns it.

    The reference imports its own backend adapters lazily, on the first dispatch
    (``_dispatch.py:216-246``), and each adapter registers itself at import.  Its CUDA adapter
    is therefore imported here first - a module is only executed once - so that this
    registration is the one that stays."""
    import importlib

    from deformops.registry import Backend as RefBackend  # type: ignore[import-not-found]
    from deformops.registry import msda as ref_msda  # type: ignore[import-not-found]

    try:
        importlib.import_module("deformops.backends.cuda.msda")
    except Exception:  # noqa: BLE001 - an adapter that cannot import registers nothing to replace
        pass
    ref_msda.register(RefBackend.CUDA, msda_b200_adapter, supports=supports, load=_load)
    return ref_msda
