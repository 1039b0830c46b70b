"""Synthetic Pi0 checkpoints.

Same contract as the reference's `random_checkpoint`
(`src/flash_vla/models/pi0/weights.py:10-24`): one generator seeded once,
tensors drawn as fp32 normal samples in `weight_shapes` order, scaled, then
rounded to bf16. Because CPU and CUDA generators produce different streams
for the same seed, parity work always generates on the CPU and uploads.
"""
from __future__ import annotations

import math

import torch

from .spec import weight_shapes


def random_checkpoint(num_views: int = 3, chunk_size: int = 50, prompt_len: int = 256,
                      wscale: float = 0.05, seed: int = 0, device: str = "cuda",
                      only: tuple[str, ...] | None = None) -> dict:
    """Draw every checkpoint tensor from N(0, wscale^2) and round to bf16.

    `num_views` and `chunk_size` are accepted for call compatibility only; no
    tensor shape depends on them. `only`, an extension, keeps just the tensors
    whose names start with one of the given prefixes while still advancing the
    generator through the skipped ones, so a decoder-only test sees exactly the
    decoder weights of the full checkpoint without holding 5.4 GB.
    """
    del num_views, chunk_size
    gen = torch.Generator(device=device).manual_seed(seed)
    shapes = weight_shapes(prompt_len)
    # One fp32 staging buffer, sized for the largest tensor and reused for every draw (the stream of
    # samples is the same as with a fresh tensor per draw; the 2.4 GB allocations are what is saved).
    staging = torch.empty(max(math.prod(s) for s in shapes.values()), dtype=torch.float32, device=device)
    out = {}
    for name, shape in shapes.items():
        count = math.prod(shape)
        sample = staging[:count].view(shape) if count else torch.empty(shape, dtype=torch.float32, device=device)
        if count:
            torch.randn(shape, dtype=torch.float32, device=device, generator=gen, out=sample)
        if only is None or name.startswith(only):
            out[name] = (sample * wscale).to(torch.bfloat16)
    return out
