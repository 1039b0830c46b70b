"""The operation table the B200 pipeline is written against.

`pipeline` calls operations by attribute on a table built once per engine, so the
implementation behind a call site is a lookup, not control flow, and two engines with
different tables can coexist. Same construction rules as the reference
(`.../h100/pi0/ops.py:21-52`): no plan -> one backend's wrappers with its fused overlays when
`fused`; with a plan -> per-op backend choice, preferring that backend's fused entry.
"""
from __future__ import annotations

from types import SimpleNamespace

from .backends import BACKENDS, build_table as _build_table


def op_table(fused: bool = True, backend: str = "cuda",
             plan: dict[str, str] | None = None) -> SimpleNamespace:
    """Build the table; `plan` maps op names to backend names and overrides `backend`."""
    if plan is None:
        return _build_table(backend, fused=fused)
    unknown = set(plan.values()) - set(BACKENDS)
    if unknown:
        raise KeyError(f"op_table: unknown backend(s) in plan: {sorted(unknown)}")
    table = {}
    for name in _op_names(backend):
        module = BACKENDS[plan.get(name, backend)]
        if fused and name in module.FUSED_WRAPPERS:
            table[name] = module.FUSED_WRAPPERS[name]
        elif name in module.ALL_WRAPPERS:
            table[name] = module.ALL_WRAPPERS[name]
    return SimpleNamespace(**table)


def _op_names(backend: str) -> list[str]:
    module = BACKENDS[backend]
    return sorted(set(module.ALL_WRAPPERS) | set(module.FUSED_WRAPPERS))


def op_names(fused: bool = True, backend: str = "cuda") -> list[str]:
    """Names present in the table, for reports."""
    return sorted(vars(op_table(fused, backend=backend)))
