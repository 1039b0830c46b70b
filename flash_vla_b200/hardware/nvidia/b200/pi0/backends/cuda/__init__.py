"""Hand-written sm_100a CUDA backend for the Pi0 call sites.

Exposes the registry contract of the reference's backends
(`.../h100/pi0/backends/__init__.py:10-14`): `ALL_WRAPPERS` and `FUSED_WRAPPERS`.
"""
from __future__ import annotations

from . import fused_wrappers, wrappers

ALL_WRAPPERS = dict(wrappers.ALL_WRAPPERS)
FUSED_WRAPPERS = dict(fused_wrappers.FUSED_WRAPPERS)

__all__ = ["ALL_WRAPPERS", "FUSED_WRAPPERS", "wrappers", "fused_wrappers"]
