"""Operator registry surface: the ``msda`` functional, ``Backend``, context and protocol.

Import-compatible with the names the reference exposes from ``deformops.registry``
(``sources/deformops/registry/__init__.py``) for the MSDA path.
"""

from ..core.runtime import Method
from .msda import (
    Backend,
    CudaBackend,
    MSDABackend,
    MSDAContext,
    MSDAMethod,
    apply_msda_method,
    forward,
    locations_from_offsets,
    msda,
    msda_from_offsets,
    resolve_method,
    supports_context,
    unsupported_reason,
)

__all__ = [
    "Backend", "CudaBackend", "MSDABackend", "MSDAContext", "MSDAMethod", "Method",
    "apply_msda_method", "forward", "locations_from_offsets", "msda", "msda_from_offsets",
    "resolve_method", "supports_context", "unsupported_reason",
]
