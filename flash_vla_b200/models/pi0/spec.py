"""Pi0 checkpoint schema: model constants and the tensors a checkpoint must hold.

Mirrors the contract of the reference's `src/flash_vla/models/pi0/spec.py:3-47`
(38 tensors, 2.709 G parameters, linear weights stored (in, out) with the
output axis contiguous). The insertion order of the returned dict is part of
the contract: `random_checkpoint` draws tensors in this order from a single
generator, so a different order would give different synthetic weights.
"""
from __future__ import annotations

VISION_LAYERS = 27
ENCODER_LAYERS = 18
HEAD_DIM = 256
DECODER_HEADS = 8
ROPE_THETA = 10000

VISION_DIM = 1152
VISION_FFN = 4304
VISION_HEADS = 16
VISION_HEAD_DIM = 72
VISION_TOKENS = 256          # 16 x 16 patches of 14 x 14 pixels per 224 x 224 view
PATCH = 14
PATCH_FEATURES = PATCH * PATCH * 3
ENCODER_DIM = 2048
ENCODER_FFN = 16384
DECODER_DIM = 1024
DECODER_FFN = 4096
QKV_DIM = (DECODER_HEADS + 2) * HEAD_DIM   # 8 query heads + one K head + one V head
ACTION_DIM = 32
DIFFUSION_STEPS = 10


def _vision(L=VISION_LAYERS, D=VISION_DIM, F=VISION_FFN):
    yield "vision_patch_embedding_w", (PATCH, PATCH, 3, D)
    yield "vision_patch_embedding_b", (D,)
    yield "vision_position_embedding", (VISION_TOKENS, D)
    for stem, k, n in (("attn_qkv", D, 3 * D), ("attn_o", D, D),
                       ("ffn_up", D, F), ("ffn_down", F, D)):
        yield f"vision_{stem}_w", (L, k, n)
        yield f"vision_{stem}_b", (L, n)
    for stem in ("pre_attn_norm", "pre_ffn_norm"):
        yield f"vision_{stem}_w", (L, D)
        yield f"vision_{stem}_b", (L, D)
    yield "vision_final_norm_w", (D,)
    yield "vision_final_norm_b", (D,)


def _stack(prefix: str, width: int, ffn: int, L=ENCODER_LAYERS):
    yield f"{prefix}_attn_qkv_w", (L, width, QKV_DIM)
    yield f"{prefix}_attn_o_w", (L, DECODER_HEADS * HEAD_DIM, width)
    yield f"{prefix}_ffn_gate_w", (L, width, ffn)
    yield f"{prefix}_ffn_up_w", (L, width, ffn)
    yield f"{prefix}_ffn_down_w", (L, ffn, width)


def _decoder_io(D=DECODER_DIM, A=ACTION_DIM):
    yield "decoder_state_in_proj_w", (A, D)
    yield "decoder_state_in_proj_b", (D,)
    yield "decoder_action_fused_in_proj_w", (A, D)
    yield "decoder_action_fused_time_biases", (DIFFUSION_STEPS, D)
    yield "decoder_action_mlp_w", (D, D)
    yield "decoder_action_mlp_b", (D,)


def weight_shapes(prompt_len: int) -> dict[str, tuple[int, ...]]:
    """Name -> shape of every checkpoint tensor for a prompt of `prompt_len` tokens."""
    shapes: dict[str, tuple[int, ...]] = {}
    shapes.update(_vision())
    shapes["encoder_multi_modal_projector_w"] = (VISION_DIM, ENCODER_DIM)
    shapes["encoder_multi_modal_projector_b"] = (ENCODER_DIM,)
    shapes.update(_stack("encoder", ENCODER_DIM, ENCODER_FFN))
    shapes.update(_decoder_io())
    shapes.update(_stack("decoder", DECODER_DIM, DECODER_FFN))
    shapes["decoder_action_fused_out_proj_w"] = (DECODER_DIM, ACTION_DIM)
    shapes["decoder_action_fused_out_proj_b"] = (ACTION_DIM,)
    shapes["language_embeds"] = (prompt_len, ENCODER_DIM)
    return shapes
