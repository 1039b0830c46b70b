"""Backend registry of the B200 Pi0 target.

A backend is a module with two dicts of call-site wrappers sharing one signature per name:
`ALL_WRAPPERS` (every call site) and `FUSED_WRAPPERS` (overlays used when `fused=True`).
Same contract as the reference's registry (`.../h100/pi0/backends/__init__.py:10-40`); this
target registers one backend, "cuda".
"""
from __future__ import annotations

from types import SimpleNamespace

from . import cuda as _cuda

BACKENDS = {"cuda": _cuda}
DEFAULT_FUSED_OPS = tuple(sorted(_cuda.FUSED_WRAPPERS))

__all__ = ["BACKENDS", "DEFAULT_FUSED_OPS", "build_table"]


def build_table(backend: str = "cuda", fused: bool = True) -> SimpleNamespace:
    """All call sites of one backend, with its fused overlays applied when `fused`."""
    module = BACKENDS[backend]
    table = dict(module.ALL_WRAPPERS)
    if fused:
        table.update(module.FUSED_WRAPPERS)
    return SimpleNamespace(**table)
