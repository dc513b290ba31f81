"""Layers built on the MSDA operator."""

from .msda import MultiScaleDeformAttn2d

__all__ = ["MultiScaleDeformAttn2d"]
