"""Checkpoint formats: safetensors IO, FP4 layouts, MMFP4 loader, trellis containers."""
from . import fp4, safetensors_io  # noqa: F401
