"""Scratch memory that is safe to use inside a captured CUDA graph.

A captured graph replays fixed addresses, so nothing may be allocated while
capturing. Temporaries (split-K partial sums, flash-decoding partials, the
patchified image matrix, tile semaphores) are therefore requested by role and
shape during the warm-up passes, kept for the life of the engine, and the pool
is frozen before capture: a request that warm-up did not cover then raises
instead of allocating. Behaviour follows the reference's `ScratchPool`
(`src/flash_vla/runtime/cuda/arena.py:19-42`): buffers are zero-filled when
first created and are never freed by the pool.
"""
from __future__ import annotations

import torch


class ScratchPool:
    def __init__(self) -> None:
        self._slabs: dict[tuple, torch.Tensor] = {}
        self._frozen = False

    def get(self, role: str, shape, dtype, device) -> torch.Tensor:
        """The buffer registered for (role, shape, dtype, device); created zeroed on first use."""
        key = (role, tuple(int(s) for s in shape), dtype, str(device))
        slab = self._slabs.get(key)
        if slab is not None:
            return slab
        if self._frozen:
            raise RuntimeError(
                f"ScratchPool is frozen but {key} was requested: warm-up never touched this "
                "role/shape, so serving it now would allocate during graph capture.")
        slab = torch.zeros(key[1], dtype=dtype, device=device)
        self._slabs[key] = slab
        return slab

    def freeze(self) -> None:
        """Disallow new buffers from here on (call after warm-up, before capture)."""
        self._frozen = True

    @property
    def frozen(self) -> bool:
        return self._frozen

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._slabs.values())

    def __len__(self) -> int:
        return len(self._slabs)
