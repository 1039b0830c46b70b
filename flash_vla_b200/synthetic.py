"""Seeded synthetic inputs for benchmarks and parity tests (no dataset is used anywhere).

Everything is drawn on the CPU, because CPU and CUDA generators give different streams for
one seed, and rounded to bf16, because the engine's input buffers are bf16. Counterpart of the
reference's `benchmarks/synthetic.py:21-73` and the input recipe of
`eval/correctness/pi0/openpi_parity.py:39-44`.
"""
from __future__ import annotations

import torch

bf16 = torch.bfloat16
VOCAB = 257152


def bench_inputs(seed: int = 0, num_views: int = 3, chunk_size: int = 50):
    """(images, state, noise): pixels ~ U[-1, 1], state and noise ~ N(0, 1), one generator, in
    this order; fp32 tensors holding bf16-representable values."""
    g = torch.Generator().manual_seed(seed)
    images = torch.rand((num_views, 224, 224, 3), generator=g) * 2.0 - 1.0
    state = torch.randn((32,), generator=g)
    noise = torch.randn((chunk_size, 32), generator=g)
    return [t.to(bf16).float() for t in (images, state, noise)]


def prompt_embeds(prompt_len: int, seed: int = 3):
    """(ids, rows): token ids ~ U{0..VOCAB-1} and the embedding rows they select, rows ~
    N(0, 0.02^2) in bf16. Only the gathered rows are materialised; a full VOCAB x 2048 table
    would be 1 GB and the unselected rows never matter."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, VOCAB, (prompt_len,), generator=g)
    rows = (torch.randn(prompt_len, 2048, generator=g) * 0.02).to(bf16)
    return ids, rows


def decoder_step_inputs(kv_scale: float, seed: int = 1, prefix: int = 768, chunk_size: int = 50):
    """Inputs of the "one decoder diffusion step" configuration: prefix K/V (18, prefix, 256)
    ~ N(0, kv_scale^2), state (32,), noise (chunk, 32); bf16 tensors."""
    g = torch.Generator().manual_seed(seed)
    K = (torch.randn(18, prefix, 256, generator=g) * kv_scale).to(bf16)
    V = (torch.randn(18, prefix, 256, generator=g) * kv_scale).to(bf16)
    state = torch.randn(32, generator=g).to(bf16)
    noise = torch.randn(chunk_size, 32, generator=g).to(bf16)
    return K, V, state, noise
