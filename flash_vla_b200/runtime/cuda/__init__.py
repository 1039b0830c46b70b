"""CUDA runtime helpers shared by targets (no model or hardware imports)."""
from .arena import ScratchPool

__all__ = ["ScratchPool"]
