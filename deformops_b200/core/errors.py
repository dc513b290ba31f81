"""Exceptions raised when the kernel library or a backend cannot serve a call.

Same names and meaning as ``sources/deformops/core/errors.py:17-47`` in the reference,
so callers that catch them keep working.
"""

from __future__ import annotations

__all__ = ["KernelBuildError", "KernelUnavailableError", "NoBackendError"]


class KernelUnavailableError(RuntimeError):
    """The compiled kernel library could not be made available."""


class KernelBuildError(KernelUnavailableError):
    """Compiling the kernel library was attempted and failed."""


class NoBackendError(RuntimeError):
    """No backend can run an operator call (there is exactly one here: the sm_100a kernels)."""
