"""B200-native multi-scale deformable attention (MSDA) behind the deformops operator surface.

``from deformops_b200.registry import msda, Backend`` mirrors ``deformops.registry``;
``torch.ops.deformops_b200.msda`` / ``msda_softmax`` are the public custom ops.
"""

__version__ = "0.1.0"

from .core.errors import KernelBuildError, KernelUnavailableError, NoBackendError  # noqa: F401
from .core.runtime import Method  # noqa: F401
from .registry import Backend, MSDABackend, MSDAContext, msda, msda_from_offsets  # noqa: F401
