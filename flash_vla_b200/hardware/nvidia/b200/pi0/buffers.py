"""Static buffer plan of the B200 Pi0 target.

Every activation the forward pass touches lives at a fixed address so the pass can be
captured once and replayed. The plan keeps the reference's 22 buffers with their names,
shapes and bf16 dtype (`.../h100/pi0/buffers.py:26-64`) and adds what the B200 kernels need:

  * `vision_attn`, `encoder_attn`: outputs of the two attention ops that the reference
    computes with torch and therefore allocates inside its graph.
  * `decoder_x` is fp32 instead of bf16: the action expert's residual stream reaches |x| ~ 10,
    where a bf16 ulp is 2^-4, and 36 in-place residual adds per step would each round it. The
    GEMMs that read it take a bf16 copy of the normalised rows; the adds stay exact in fp32.
  * `decoder_x_bf16`: bf16 shadow of `decoder_x`, refreshed by every op that writes `decoder_x`
    (the engine registers the pair with the backend), so the QKV and gate/up GEMMs fetch their
    activation operand by TMA instead of converting fp32 rows inside the kernel.
  * `diffusion_noise_f32`: fp32 master copy of the action chunk. The ten Euler updates
    accumulate here so that each step adds its update without first rounding the running
    value to bf16; `diffusion_noise` (bf16) is refreshed from it at the end of the pass.

RoPE tables: row r holds interleaved (cos, sin) of (offset + r) * 10000^(-2p/256), rounded
to bf16 (`buffers.py:15-23`); the decoder's positions continue after the prefix.
"""
from __future__ import annotations

import torch

from flash_vla_b200.models.pi0.spec import (DECODER_DIM, DECODER_FFN, DECODER_HEADS, ENCODER_DIM,
                                           ENCODER_FFN, ENCODER_LAYERS, HEAD_DIM, ROPE_THETA,
                                           VISION_DIM, VISION_FFN, VISION_TOKENS, ACTION_DIM)


def rope_table(seq_len: int, offset: int, head_dim: int, device) -> torch.Tensor:
    """(seq_len, head_dim) bf16 table of interleaved cos/sin for positions offset..offset+seq_len-1."""
    position = (torch.arange(seq_len, device=device) + offset)[:, None]
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim
    phase = position * (1.0 / (ROPE_THETA ** exponent))[None, :]
    table = torch.stack((torch.cos(phase).to(torch.bfloat16), torch.sin(phase).to(torch.bfloat16)), dim=-1)
    return table.reshape(seq_len, head_dim)


def _prefix_plan(add, num_views: int, S: int, cache: int, episodes: int) -> None:
    """Buffers of SigLIP and the prefix encoder for `episodes` sequences of S tokens laid end to end."""
    E = episodes
    add("observation_images_normalized", E * num_views, 224, 224, 3)
    for name, width in (("vision_x", VISION_DIM), ("vision_x_norm", VISION_DIM),
                        ("vision_QKV", 3 * VISION_DIM), ("vision_attn", VISION_DIM),
                        ("vision_hidden", VISION_FFN)):
        add(name, E * num_views, VISION_TOKENS, width)
    add("encoder_rope_weights", S, HEAD_DIM)
    add("encoder_x", E * S, ENCODER_DIM)
    add("encoder_x_norm", E * S, ENCODER_DIM)
    if E == 1:
        add("encoder_K", ENCODER_LAYERS, cache, HEAD_DIM)
        add("encoder_V", ENCODER_LAYERS, cache, HEAD_DIM)
    else:
        add("encoder_K", E, ENCODER_LAYERS, cache, HEAD_DIM)
        add("encoder_V", E, ENCODER_LAYERS, cache, HEAD_DIM)
    add("encoder_Q", E * S * DECODER_HEADS, HEAD_DIM)
    add("encoder_attn", E * S, DECODER_HEADS * HEAD_DIM)
    add("encoder_hidden", E * S, ENCODER_FFN)


def _decoder_plan(add, chunk_size: int, cache: int) -> None:
    D = chunk_size + 1
    add("observation_state_normalized", ACTION_DIM)
    add("diffusion_noise", chunk_size, ACTION_DIM)
    add("diffusion_noise_f32", chunk_size, ACTION_DIM, dtype=torch.float32)
    add("decoder_rope_weights", D, HEAD_DIM)
    add("decoder_x", D, DECODER_DIM, dtype=torch.float32)
    add("decoder_x_bf16", D, DECODER_DIM)
    add("decoder_x_buf", chunk_size, DECODER_DIM)
    add("decoder_state_buf", 1, DECODER_DIM)
    add("decoder_norm_factor_buf", D)
    add("decoder_q_buf", D * DECODER_HEADS, HEAD_DIM)
    add("decoder_attn_buf", D * DECODER_HEADS, cache)
    add("decoder_hidden", D, DECODER_FFN)


def _materialise(plan, device):
    return {name: torch.zeros(shape, dtype=dtype, device=device) for name, (shape, dtype) in plan.items()}


def allocate_batched_decoder_buffers(chunk_size: int, episodes: int, encoder_seq_len: int, device: str):
    """Decoder buffers of the throughput profile when the action-expert decoder, too, runs once over all
    episodes' rows (M = episodes x (chunk + 1)): the residual stream, Q, the FFN hidden state and the noise
    hold the episodes end to end; K / V stay in the per-episode caches. `decoder_mlp_out` and
    `decoder_x_rows` are staging rows for the two places where an op's contiguous (episodes x chunk) rows
    meet the (episodes, chunk + 1) layout of the residual stream."""
    E, D = episodes, chunk_size + 1
    plan: dict[str, tuple[tuple[int, ...], torch.dtype]] = {}

    def add(name, *shape, dtype=torch.bfloat16):
        plan[name] = (shape, dtype)

    add("observation_state_normalized", E, ACTION_DIM)
    add("diffusion_noise", E, chunk_size, ACTION_DIM)
    add("diffusion_noise_f32", E * chunk_size, ACTION_DIM, dtype=torch.float32)
    add("decoder_rope_weights", D, HEAD_DIM)
    add("decoder_x", E * D, DECODER_DIM, dtype=torch.float32)
    add("decoder_x_buf", E * chunk_size, DECODER_DIM)
    add("decoder_mlp_out", E * chunk_size, DECODER_DIM, dtype=torch.float32)
    add("decoder_x_rows", E * chunk_size, DECODER_DIM, dtype=torch.float32)
    add("decoder_state_buf", E, DECODER_DIM)
    add("decoder_norm_factor_buf", E * D)
    add("decoder_q_buf", E * D * DECODER_HEADS, HEAD_DIM)
    add("decoder_hidden", E * D, DECODER_FFN)
    b = _materialise(plan, device)
    b["decoder_rope_weights"].copy_(rope_table(D, encoder_seq_len, HEAD_DIM, device))
    return b


def allocate_batched_buffers(num_views: int, chunk_size: int, prompt_len: int, episodes: int, device: str):
    """Buffer plan of the throughput profile: `episodes` independent episodes whose SigLIP tower and prefix
    encoder run as ONE pass over all episodes' tokens (M = episodes x S rows, so every vision and prefix
    weight is streamed once for the whole batch) while each episode keeps its own KV cache and decoder
    buffers. Returns (prefix, [decoder buffers per episode], S): `prefix` holds the batched tensors;
    every per-episode dict also carries views `encoder_K` / `encoder_V` (18, S + D, 256) of its own cache
    and `observation_images_normalized` of its own views, so the decoder ops see the single-episode layout."""
    S = num_views * VISION_TOKENS + prompt_len
    D = chunk_size + 1
    cache = S + D
    plan: dict[str, tuple[tuple[int, ...], torch.dtype]] = {}

    def add(name, *shape, dtype=torch.bfloat16):
        plan[name] = (shape, dtype)

    _prefix_plan(add, num_views, S, cache, episodes)
    prefix = _materialise(plan, device)
    prefix["encoder_rope_weights"].copy_(rope_table(S, 0, HEAD_DIM, device))
    per_episode = []
    for e in range(episodes):
        plan.clear()
        _decoder_plan(add, chunk_size, cache)
        b = _materialise(plan, device)
        b["decoder_rope_weights"].copy_(rope_table(D, S, HEAD_DIM, device))
        b["encoder_K"], b["encoder_V"] = prefix["encoder_K"][e], prefix["encoder_V"][e]
        b["observation_images_normalized"] = prefix["observation_images_normalized"][e * num_views:(e + 1) * num_views]
        per_episode.append(b)
    return prefix, per_episode, S


def allocate_static_buffers(num_views: int, chunk_size: int, prompt_len: int,
                            device: str) -> tuple[dict[str, torch.Tensor], int]:
    """Allocate every persistent buffer and fill the two RoPE tables. Returns (buffers, S)."""
    S = num_views * VISION_TOKENS + prompt_len          # prefix length
    D = chunk_size + 1                                   # state token + action chunk
    cache = S + D

    plan: dict[str, tuple[tuple[int, ...], torch.dtype]] = {}

    def add(name, *shape, dtype=torch.bfloat16):
        plan[name] = (shape, dtype)

    add("observation_images_normalized", num_views, 224, 224, 3)
    add("observation_state_normalized", ACTION_DIM)
    add("diffusion_noise", chunk_size, ACTION_DIM)
    add("diffusion_noise_f32", chunk_size, ACTION_DIM, dtype=torch.float32)
    for name, width in (("vision_x", VISION_DIM), ("vision_x_norm", VISION_DIM),
                        ("vision_QKV", 3 * VISION_DIM), ("vision_attn", VISION_DIM),
                        ("vision_hidden", VISION_FFN)):
        add(name, num_views, VISION_TOKENS, width)
    add("encoder_rope_weights", S, HEAD_DIM)
    add("encoder_x", S, ENCODER_DIM)
    add("encoder_x_norm", S, ENCODER_DIM)
    add("encoder_K", ENCODER_LAYERS, cache, HEAD_DIM)
    add("encoder_V", ENCODER_LAYERS, cache, HEAD_DIM)
    add("encoder_Q", S * DECODER_HEADS, HEAD_DIM)
    add("encoder_attn", S, DECODER_HEADS * HEAD_DIM)
    add("encoder_hidden", S, ENCODER_FFN)
    add("decoder_rope_weights", D, HEAD_DIM)
    add("decoder_x", D, DECODER_DIM, dtype=torch.float32)
    add("decoder_x_bf16", D, DECODER_DIM)
    add("decoder_x_buf", chunk_size, DECODER_DIM)
    add("decoder_state_buf", 1, DECODER_DIM)
    add("decoder_norm_factor_buf", D)
    add("decoder_q_buf", D * DECODER_HEADS, HEAD_DIM)
    add("decoder_attn_buf", D * DECODER_HEADS, cache)
    add("decoder_hidden", D, DECODER_FFN)

    buffers = {name: torch.zeros(shape, dtype=dtype, device=device)
               for name, (shape, dtype) in plan.items()}
    buffers["encoder_rope_weights"].copy_(rope_table(S, 0, HEAD_DIM, device))
    buffers["decoder_rope_weights"].copy_(rope_table(D, S, HEAD_DIM, device))
    return buffers, S
