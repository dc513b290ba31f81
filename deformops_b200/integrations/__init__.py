"""Bridges for model code that carries its own projections (Hugging Face, mmcv style)."""

from ._ops import run_msda

__all__ = ["run_msda"]
