"""OpenPI (PyTorch) Pi0 state dict -> the packed checkpoint this target consumes.

Behaviour follows the reference's adapter, `eval/baselines/openpi.py:75-126` (helpers) and
`:129-313` (`target_checkpoint`): same 38 output tensors, same arithmetic, same rounding (every
product is formed in fp32 and rounded to bf16 once, per layer, before stacking). It is written as
a table of recipes rather than one dict literal, and it takes a plain `state_dict` (or anything
with `.state_dict()`), so it runs without the `openpi` package: the only thing the reference
imports from `openpi` inside the conversion is `create_sinusoidal_pos_embedding`
(`openpi.py:280`), restated below from its published definition.

What the conversion does:
  * linear weights are transposed to (in, out);
  * Gemma RMSNorm scales `(1 + w)` are folded into the rows of the projection that follows the
    norm (QKV, gate, up; the final decoder norm into the action output projection);
  * Q and K columns are permuted per head from OpenPI's half-split RoPE layout
    `[x_0 .. x_{d/2-1} | x_{d/2} .. x_{d-1}]` to adjacent pairs `[x_0, x_{d/2}, x_1, x_{d/2+1}, ...]`,
    the layout the QKV epilogue rotates;
  * Q, K, V are concatenated along the output axis;
  * the action/time input MLP is folded for the ten fixed timesteps 1.0, 0.9, ..., 0.1 into one
    (32, 1024) matrix and ten bias rows; the Euler step dt = -0.1 is folded into the output
    projection, so one decoder step is `noise += b + rms(x) @ W`.
"""
from __future__ import annotations

import math
from typing import Callable, Mapping

import torch

from .spec import DECODER_DIM, DECODER_HEADS, DIFFUSION_STEPS, ENCODER_DIM, ENCODER_LAYERS, VISION_LAYERS, weight_shapes

_PALI = "paligemma_with_expert.paligemma.model"
VISION_ROOT = f"{_PALI}.vision_tower.vision_model"
PROJECTOR_ROOT = f"{_PALI}.multi_modal_projector.linear"
ENCODER_ROOT = f"{_PALI}.language_model"
DECODER_ROOT = "paligemma_with_expert.gemma_expert.model"

EULER_DT = -0.1


def sinusoidal_time_embedding(times: torch.Tensor, dimension: int, min_period: float, max_period: float) -> torch.Tensor:
    """[sin(2 pi t / p_j) | cos(2 pi t / p_j)], periods p_j log-spaced from `min_period` to `max_period`
    over `dimension / 2` entries. Restates `openpi.models_pytorch.pi0_pytorch.create_sinusoidal_pos_embedding`
    (the reference calls it at `eval/baselines/openpi.py:280-287`); computed in float64 as OpenPI does on
    non-MPS devices. The `openpi` package is not a dependency of the reference and is absent here, so
    this one function is not pinned against it."""
    if dimension % 2:
        raise ValueError("sinusoidal_time_embedding: dimension must be even")
    fraction = torch.linspace(0.0, 1.0, dimension // 2, dtype=torch.float64, device=times.device)
    period = min_period * (max_period / min_period) ** fraction
    phase = (2.0 * math.pi / period)[None, :] * times.to(torch.float64)[:, None]
    return torch.cat([torch.sin(phase), torch.cos(phase)], dim=1)


def adjacent_pair_columns(weight: torch.Tensor, heads: int) -> torch.Tensor:
    """Permute the output columns of a (in, heads * d) projection, per head, from half-split to
    adjacent-pair RoPE order: new column 2p is old column p, new column 2p + 1 is old column d/2 + p
    (`eval/baselines/openpi.py:101-109`)."""
    rows, cols = weight.shape
    d = cols // heads
    return weight.view(rows, heads, 2, d // 2).transpose(2, 3).reshape(rows, cols)


class _Source:
    """fp32 views of an OpenPI state dict with the reference's error for a missing name."""

    def __init__(self, state: Mapping[str, torch.Tensor]):
        self.state = state

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self.state:
            raise KeyError(f"OpenPI checkpoint is missing {name!r}")
        return self.state[name].detach().float()

    def linear(self, module: str) -> torch.Tensor:
        """`module.weight` as (in, out)."""
        return self.tensor(f"{module}.weight").T

    def folded(self, module: str, norm_weight: str) -> torch.Tensor:
        """(in, out) weight with the preceding RMSNorm scale (1 + w) multiplied into its rows."""
        # multiplied in the stored (out, in) layout, transposed as a view: the same fp32 products as scaling the rows of
        # the (in, out) view, without a strided pass over the fp32 data
        return (self.tensor(f"{module}.weight") * (1.0 + self.tensor(norm_weight))[None, :]).T

    def packed_qkv(self, root: str, layer: int) -> torch.Tensor:
        attn = f"{root}.layers.{layer}.self_attn"
        norm = f"{root}.layers.{layer}.input_layernorm.weight"
        return torch.cat([adjacent_pair_columns(self.folded(f"{attn}.q_proj", norm), DECODER_HEADS),
                          adjacent_pair_columns(self.folded(f"{attn}.k_proj", norm), 1),
                          self.folded(f"{attn}.v_proj", norm)], dim=1)


def _bf16(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 2 and not t.is_contiguous() and t.T.is_contiguous():
        return t.T.to(torch.bfloat16).T.contiguous()      # round in the stored layout, transpose the 2-byte values
    return t.to(torch.bfloat16).contiguous()


def _per_layer(count: int, make: Callable[[int], torch.Tensor]) -> torch.Tensor:
    """The layers' tensors stacked as bf16. Each layer is rounded (and, for a transposed view, transposed) straight into
    its slot of the result, so no per-layer bf16 copies are made: a Pi0 checkpoint moves 5.4 GB through here."""
    out = None
    for i in range(count):
        value = make(i)
        if out is None:
            out = torch.empty((count,) + tuple(value.shape), dtype=torch.bfloat16, device=value.device)
        out[i].copy_(value)
    return out


def _vision_recipes(src: _Source) -> dict[str, Callable[[], torch.Tensor]]:
    emb = f"{VISION_ROOT}.embeddings"

    def layer(i: int) -> str:
        return f"{VISION_ROOT}.encoder.layers.{i}"

    def each(make):
        return lambda: _per_layer(VISION_LAYERS, make)

    recipes = {
        # conv weight (out, c, ky, kx) -> (ky, kx, c, out): patch features ordered row, column, channel
        "vision_patch_embedding_w": lambda: _bf16(src.tensor(f"{emb}.patch_embedding.weight").permute(2, 3, 1, 0)),
        "vision_patch_embedding_b": lambda: _bf16(src.tensor(f"{emb}.patch_embedding.bias")),
        "vision_position_embedding": lambda: _bf16(src.tensor(f"{emb}.position_embedding.weight")),
        "vision_attn_qkv_w": each(lambda i: torch.cat(
            [src.linear(f"{layer(i)}.self_attn.{p}_proj") for p in "qkv"], dim=1)),
        "vision_attn_qkv_b": each(lambda i: torch.cat(
            [src.tensor(f"{layer(i)}.self_attn.{p}_proj.bias") for p in "qkv"])),
        "vision_final_norm_w": lambda: _bf16(src.tensor(f"{VISION_ROOT}.post_layernorm.weight")),
        "vision_final_norm_b": lambda: _bf16(src.tensor(f"{VISION_ROOT}.post_layernorm.bias")),
    }
    for target, module in (("attn_o", "self_attn.out_proj"), ("ffn_up", "mlp.fc1"), ("ffn_down", "mlp.fc2")):
        recipes[f"vision_{target}_w"] = each(lambda i, m=module: src.linear(f"{layer(i)}.{m}"))
        recipes[f"vision_{target}_b"] = each(lambda i, m=module: src.tensor(f"{layer(i)}.{m}.bias"))
    for target, module in (("pre_attn_norm", "layer_norm1"), ("pre_ffn_norm", "layer_norm2")):
        recipes[f"vision_{target}_w"] = each(lambda i, m=module: src.tensor(f"{layer(i)}.{m}.weight"))
        recipes[f"vision_{target}_b"] = each(lambda i, m=module: src.tensor(f"{layer(i)}.{m}.bias"))
    return recipes


def _gemma_recipes(src: _Source, prefix: str, root: str) -> dict[str, Callable[[], torch.Tensor]]:
    def each(make):
        return lambda: _per_layer(ENCODER_LAYERS, make)

    def post_norm(i: int) -> str:
        return f"{root}.layers.{i}.post_attention_layernorm.weight"

    return {
        f"{prefix}_attn_qkv_w": each(lambda i: src.packed_qkv(root, i)),
        f"{prefix}_attn_o_w": each(lambda i: src.linear(f"{root}.layers.{i}.self_attn.o_proj")),
        f"{prefix}_ffn_gate_w": each(lambda i: src.folded(f"{root}.layers.{i}.mlp.gate_proj", post_norm(i))),
        f"{prefix}_ffn_up_w": each(lambda i: src.folded(f"{root}.layers.{i}.mlp.up_proj", post_norm(i))),
        f"{prefix}_ffn_down_w": each(lambda i: src.linear(f"{root}.layers.{i}.mlp.down_proj")),
    }


def _action_recipes(src: _Source, time_embedding) -> dict[str, Callable[[], torch.Tensor]]:
    def mix():
        w = src.tensor("action_time_mlp_in.weight")          # (1024, 2048): [action half | time half]
        return w[:, :DECODER_DIM].T, w[:, DECODER_DIM:].T

    def time_biases():
        action_mix, time_mix = mix()
        dt = torch.tensor(EULER_DT, dtype=torch.float32)
        t = torch.tensor(1.0, dtype=torch.float32)
        times = []
        for _ in range(DIFFUSION_STEPS):                      # running fp32 sum, as the sampler steps it
            times.append(t.clone())
            t = t + dt
        emb = time_embedding(torch.stack(times), DECODER_DIM, 4e-3, 4.0).float()
        return _bf16(src.tensor("action_in_proj.bias") @ action_mix + emb @ time_mix
                     + src.tensor("action_time_mlp_in.bias"))

    def out_w():
        scale = 1.0 + src.tensor(f"{DECODER_ROOT}.norm.weight")
        return _bf16(torch.tensor(EULER_DT) * scale[:, None] * src.linear("action_out_proj"))

    return {
        "decoder_state_in_proj_w": lambda: _bf16(src.linear("state_proj")),
        "decoder_state_in_proj_b": lambda: _bf16(src.tensor("state_proj.bias")),
        "decoder_action_fused_in_proj_w": lambda: _bf16(src.linear("action_in_proj") @ mix()[0]),
        "decoder_action_fused_time_biases": time_biases,
        "decoder_action_mlp_w": lambda: _bf16(src.linear("action_time_mlp_out")),
        "decoder_action_mlp_b": lambda: _bf16(src.tensor("action_time_mlp_out.bias")),
        "decoder_action_fused_out_proj_w": out_w,
        "decoder_action_fused_out_proj_b": lambda: _bf16(torch.tensor(EULER_DT) * src.tensor("action_out_proj.bias")),
    }


@torch.inference_mode()
def target_checkpoint(model_or_state, time_embedding=sinusoidal_time_embedding) -> dict[str, torch.Tensor]:
    """Convert an OpenPI PyTorch Pi0 model (or its `state_dict`) into this target's checkpoint
    (`weight_shapes(prompt_len=0)`: 38 bf16 tensors, empty `language_embeds`). Raises `KeyError` for a
    missing source tensor and `ValueError` when a result has the wrong shape, like the reference
    (`eval/baselines/openpi.py:75-79`, `:304-311`). `time_embedding(times, dim, min_period, max_period)`
    may be OpenPI's own function."""
    state = model_or_state.state_dict() if hasattr(model_or_state, "state_dict") else model_or_state
    for name in openpi_state_shapes():                        # fail before converting gigabytes, with the reference's message
        if name not in state:
            raise KeyError(f"OpenPI checkpoint is missing {name!r}")
    src = _Source(state)
    recipes: dict[str, Callable[[], torch.Tensor]] = {}
    recipes.update(_vision_recipes(src))
    recipes["encoder_multi_modal_projector_w"] = lambda: _bf16(src.linear(PROJECTOR_ROOT))
    recipes["encoder_multi_modal_projector_b"] = lambda: _bf16(src.tensor(f"{PROJECTOR_ROOT}.bias"))
    recipes.update(_gemma_recipes(src, "encoder", ENCODER_ROOT))
    recipes.update(_gemma_recipes(src, "decoder", DECODER_ROOT))
    recipes.update(_action_recipes(src, time_embedding))
    device = src.tensor("action_in_proj.weight").device
    recipes["language_embeds"] = lambda: torch.empty((0, ENCODER_DIM), dtype=torch.bfloat16, device=device)

    expected = weight_shapes(prompt_len=0)
    if set(recipes) != set(expected):
        raise ValueError(f"converter recipes do not cover the schema: missing={sorted(set(expected) - set(recipes))}, "
                         f"extra={sorted(set(recipes) - set(expected))}")
    out = {}
    for name, shape in expected.items():                      # schema order
        value = recipes[name]()
        if tuple(value.shape) != tuple(shape):
            raise ValueError(f"{name} has shape {tuple(value.shape)}, expected {shape}")
        out[name] = value
    return out


def openpi_state_shapes() -> dict[str, tuple[int, ...]]:
    """Name -> shape of every OpenPI tensor the conversion reads (Pi0 base: SigLIP-So400m/14, Gemma-2B,
    Gemma-300M expert). Used to build synthetic state dicts for tests."""
    from .spec import (ACTION_DIM, DECODER_FFN, ENCODER_FFN, HEAD_DIM, PATCH, VISION_DIM, VISION_FFN, VISION_TOKENS)
    s: dict[str, tuple[int, ...]] = {}
    emb = f"{VISION_ROOT}.embeddings"
    s[f"{emb}.patch_embedding.weight"] = (VISION_DIM, 3, PATCH, PATCH)
    s[f"{emb}.patch_embedding.bias"] = (VISION_DIM,)
    s[f"{emb}.position_embedding.weight"] = (VISION_TOKENS, VISION_DIM)
    for i in range(VISION_LAYERS):
        layer = f"{VISION_ROOT}.encoder.layers.{i}"
        for p in ("q_proj", "k_proj", "v_proj", "out_proj"):
            s[f"{layer}.self_attn.{p}.weight"] = (VISION_DIM, VISION_DIM)
            s[f"{layer}.self_attn.{p}.bias"] = (VISION_DIM,)
        s[f"{layer}.mlp.fc1.weight"], s[f"{layer}.mlp.fc1.bias"] = (VISION_FFN, VISION_DIM), (VISION_FFN,)
        s[f"{layer}.mlp.fc2.weight"], s[f"{layer}.mlp.fc2.bias"] = (VISION_DIM, VISION_FFN), (VISION_DIM,)
        for n in ("layer_norm1", "layer_norm2"):
            s[f"{layer}.{n}.weight"] = s[f"{layer}.{n}.bias"] = (VISION_DIM,)
    s[f"{VISION_ROOT}.post_layernorm.weight"] = s[f"{VISION_ROOT}.post_layernorm.bias"] = (VISION_DIM,)
    s[f"{PROJECTOR_ROOT}.weight"], s[f"{PROJECTOR_ROOT}.bias"] = (ENCODER_DIM, VISION_DIM), (ENCODER_DIM,)
    for root, width, ffn in ((ENCODER_ROOT, ENCODER_DIM, ENCODER_FFN), (DECODER_ROOT, DECODER_DIM, DECODER_FFN)):
        for i in range(ENCODER_LAYERS):
            layer = f"{root}.layers.{i}"
            s[f"{layer}.self_attn.q_proj.weight"] = (DECODER_HEADS * HEAD_DIM, width)
            s[f"{layer}.self_attn.k_proj.weight"] = s[f"{layer}.self_attn.v_proj.weight"] = (HEAD_DIM, width)
            s[f"{layer}.self_attn.o_proj.weight"] = (width, DECODER_HEADS * HEAD_DIM)
            s[f"{layer}.mlp.gate_proj.weight"] = s[f"{layer}.mlp.up_proj.weight"] = (ffn, width)
            s[f"{layer}.mlp.down_proj.weight"] = (width, ffn)
            s[f"{layer}.input_layernorm.weight"] = s[f"{layer}.post_attention_layernorm.weight"] = (width,)
    s[f"{DECODER_ROOT}.norm.weight"] = (DECODER_DIM,)
    s["state_proj.weight"], s["state_proj.bias"] = (DECODER_DIM, ACTION_DIM), (DECODER_DIM,)
    s["action_in_proj.weight"], s["action_in_proj.bias"] = (DECODER_DIM, ACTION_DIM), (DECODER_DIM,)
    s["action_time_mlp_in.weight"], s["action_time_mlp_in.bias"] = (DECODER_DIM, 2 * DECODER_DIM), (DECODER_DIM,)
    s["action_time_mlp_out.weight"], s["action_time_mlp_out.bias"] = (DECODER_DIM, DECODER_DIM), (DECODER_DIM,)
    s["action_out_proj.weight"], s["action_out_proj.bias"] = (ACTION_DIM, DECODER_DIM), (ACTION_DIM,)
    return s


def synthetic_openpi_state(seed: int = 0, scale: float = 0.02) -> dict[str, torch.Tensor]:
    """A full-shape OpenPI-style state dict drawn from N(0, scale^2) in bf16 (norm scales and biases
    included), one CPU generator, `openpi_state_shapes()` order. 5.4 GB. Stands in for a real checkpoint,
    which cannot be downloaded where this is built."""
    g = torch.Generator().manual_seed(seed)
    return {name: (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)
            for name, shape in openpi_state_shapes().items()}


def error_metrics(reference: torch.Tensor, output: torch.Tensor) -> dict[str, float]:
    """The five figures the reference's parity script reports (`eval/correctness/pi0/openpi_parity.py:14-28`):
    max / mean / RMS / 99th-percentile absolute error and cosine similarity."""
    if reference.shape != output.shape:
        raise ValueError(f"shape mismatch: reference={tuple(reference.shape)}, output={tuple(output.shape)}")
    a, o = reference.float().flatten(), output.float().flatten()
    err = (o - a).abs()
    return {"max_abs": err.max().item(), "mean_abs": err.mean().item(),
            "rms_error": (o - a).pow(2).mean().sqrt().item(), "p99_abs": torch.quantile(err, 0.99).item(),
            "cosine_similarity": torch.nn.functional.cosine_similarity(a, o, dim=0).item()}
