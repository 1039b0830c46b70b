"""The Pi0 forward pass of the B200 target as calls into an operation table.

Three stages, each a pure sequence of `ops.<name>(...)` calls on static buffers, following
the reference's orchestration (`.../h100/pi0/pipeline.py:21-135`) call for call. Differences,
all on the B200 side of the drop-in boundary:

  * SigLIP and prefix attention go through the table (`ops.vision_attention`,
    `ops.encoder_attention`) into preallocated buffers instead of being torch calls.
  * When the buffer plan holds `diffusion_noise_f32`, the Euler updates accumulate in it and
    the bf16 `diffusion_noise` is refreshed once at the end of the decoder.
"""
from __future__ import annotations

from flash_vla_b200.models.pi0.spec import (DECODER_HEADS, DIFFUSION_STEPS, ENCODER_LAYERS, HEAD_DIM,
                                           VISION_LAYERS, VISION_TOKENS)


def vision_encoder(ops, weights, buffers, num_views):
    """Patch-embed the views and run the 27 SigLIP layers in place on `vision_x`. The buffers may hold the
    views of several episodes back to back (`num_views` is the count per episode): every op of the tower
    works per view or per token, so a batch is simply more rows."""
    if num_views == 2:
        raise NotImplementedError("num_views == 2 is not supported (as in the reference, pipeline.py:23)")
    w, b = weights, buffers
    x, xn = b["vision_x"], b["vision_x_norm"]
    ops.vision_patch_embed(b["observation_images_normalized"], w["vision_patch_embedding_w"],
                           w["vision_patch_embedding_b"], w["vision_position_embedding"], x)
    for layer in range(VISION_LAYERS):
        ops.vision_norm_qkv(x, w["vision_pre_attn_norm_w"][layer], w["vision_pre_attn_norm_b"][layer],
                            w["vision_attn_qkv_w"][layer], w["vision_attn_qkv_b"][layer],
                            b["vision_QKV"], xn)
        ops.vision_attention(b["vision_QKV"], b["vision_attn"])
        ops.vision_out_proj_residual(b["vision_attn"], w["vision_attn_o_w"][layer],
                                     w["vision_attn_o_b"][layer], x, x)
        ops.vision_norm_ffn_up(x, w["vision_pre_ffn_norm_w"][layer], w["vision_pre_ffn_norm_b"][layer],
                               w["vision_ffn_up_w"][layer], w["vision_ffn_up_b"][layer],
                               b["vision_hidden"], xn)
        ops.vision_ffn_down_residual(b["vision_hidden"], w["vision_ffn_down_w"][layer],
                                     w["vision_ffn_down_b"][layer], x, x)


def transformer_encoder(ops, weights, buffers, encoder_seq_len, after_qkv=None):
    """Project vision tokens to encoder width and fill the prefix KV cache of all 18 layers.

    The last layer only needs its K and V, so it stops after the QKV projection. `after_qkv(layer)`,
    if given, is called once layer `layer`'s prefix K/V have been enqueued: from then on a decoder
    layer of the same index has everything it needs from the encoder.
    """
    w, b, S = weights, buffers, encoder_seq_len
    x = b["encoder_x"]
    ops.encoder_projector(b["vision_x"], w["vision_final_norm_w"], w["vision_final_norm_b"],
                          w["encoder_multi_modal_projector_w"], w["encoder_multi_modal_projector_b"],
                          x, b["vision_x_norm"])
    for layer in range(ENCODER_LAYERS):
        k_prefix, v_prefix = b["encoder_K"][layer, :S], b["encoder_V"][layer, :S]
        ops.encoder_norm_qkv_rope(x, w["encoder_attn_qkv_w"][layer], b["encoder_rope_weights"],
                                  b["encoder_Q"], k_prefix, v_prefix, b["encoder_x_norm"])
        if after_qkv is not None:
            after_qkv(layer)
        if layer == ENCODER_LAYERS - 1:
            return
        ops.encoder_attention(b["encoder_Q"], k_prefix, v_prefix, HEAD_DIM ** -0.5, b["encoder_attn"])
        ops.encoder_out_proj_residual(b["encoder_attn"], w["encoder_attn_o_w"][layer], x)
        ops.encoder_norm_gated_ffn(x, w["encoder_ffn_gate_w"][layer], w["encoder_ffn_up_w"][layer],
                                   b["encoder_hidden"], b["encoder_x_norm"])
        ops.encoder_ffn_down_residual(b["encoder_hidden"], w["encoder_ffn_down_w"][layer], x)


def transformer_encoder_batched(ops, weights, buffers, encoder_seq_len, num_views, episodes, after_qkv=None,
                                per_episode=None):
    """The prefix encoder over `episodes` sequences of `encoder_seq_len` tokens laid end to end in the batched
    buffers (`allocate_batched_buffers`): every projection runs once over all rows, so its weights are
    streamed once for the whole batch; attention, which mixes tokens, runs per episode. K / V of layer L go
    straight into rows [0, S) of every episode's cache. Same ops and call order per layer as
    `transformer_encoder`. `per_episode(e)`, if given, returns a context manager under which episode e's
    attention is enqueued (the engine uses it to put the episodes' attention launches, 48 CTAs each, side by
    side on streams of their own) and `per_episode(None)` is called once after the last episode to join."""
    import contextlib
    w, b, S, E = weights, buffers, encoder_seq_len, episodes
    x = b["encoder_x"]
    for e in range(E):
        views = slice(e * num_views, (e + 1) * num_views)
        ops.encoder_projector(b["vision_x"][views], w["vision_final_norm_w"], w["vision_final_norm_b"],
                              w["encoder_multi_modal_projector_w"], w["encoder_multi_modal_projector_b"],
                              x[e * S:(e + 1) * S], b["vision_x_norm"][views])
    for layer in range(ENCODER_LAYERS):
        k_prefix, v_prefix = b["encoder_K"][:, layer, :S], b["encoder_V"][:, layer, :S]      # (E, S, 256) views
        ops.encoder_norm_qkv_rope(x, w["encoder_attn_qkv_w"][layer], b["encoder_rope_weights"],
                                  b["encoder_Q"], k_prefix, v_prefix, b["encoder_x_norm"])
        if after_qkv is not None:
            after_qkv(layer)
        if layer == ENCODER_LAYERS - 1:
            return
        for e in range(E):
            rows = slice(e * S, (e + 1) * S)
            with (per_episode(e) if per_episode is not None else contextlib.nullcontext()):
                ops.encoder_attention(b["encoder_Q"][e * S * DECODER_HEADS:(e + 1) * S * DECODER_HEADS], k_prefix[e], v_prefix[e],
                                      HEAD_DIM ** -0.5, b["encoder_attn"][rows])
        if per_episode is not None:
            per_episode(None)
        ops.encoder_out_proj_residual(b["encoder_attn"], w["encoder_attn_o_w"][layer], x)
        ops.encoder_norm_gated_ffn(x, w["encoder_ffn_gate_w"][layer], w["encoder_ffn_up_w"][layer],
                                   b["encoder_hidden"], b["encoder_x_norm"])
        ops.encoder_ffn_down_residual(b["encoder_hidden"], w["encoder_ffn_down_w"][layer], x)


def _copy(ops, dst, src):
    """dst <- src through the table's own copy kernel when it has one (it also refreshes a bf16 shadow of
    `dst`), else a framework copy followed by the shadow refresh."""
    if ops is not None and hasattr(ops, "copy_rows"):
        ops.copy_rows(dst, src)
        return
    dst.copy_(src)
    if ops is not None and hasattr(ops, "sync_shadow"):
        ops.sync_shadow(dst)


def decoder_step(ops, weights, buffers, encoder_seq_len, step, layers=ENCODER_LAYERS, noise=None,
                 before_layer=None):
    """One flow-matching Euler step over `noise` (default: the plan's master copy). `before_layer(layer)`,
    if given, is called before layer `layer` is enqueued (the place to wait for that layer's prefix K/V)."""
    w, b, S = weights, buffers, encoder_seq_len
    if noise is None:
        noise = b["diffusion_noise_f32"] if "diffusion_noise_f32" in b else b["diffusion_noise"]
    x, nf = b["decoder_x"], b["decoder_norm_factor_buf"]
    _copy(ops, x[:1], b["decoder_state_buf"])
    ops.decoder_action_in_proj(noise, w["decoder_action_fused_in_proj_w"],
                               w["decoder_action_fused_time_biases"][step % DIFFUSION_STEPS],
                               b["decoder_x_buf"])
    ops.decoder_action_mlp(b["decoder_x_buf"], w["decoder_action_mlp_w"], w["decoder_action_mlp_b"], x[1:])
    q = b["decoder_q_buf"]
    for layer in range(layers):
        k_cache, v_cache = b["encoder_K"][layer], b["encoder_V"][layer]
        if before_layer is not None:
            before_layer(layer)
        ops.decoder_norm_qkv_rope(x, w["decoder_attn_qkv_w"][layer], b["decoder_rope_weights"], q,
                                  k_cache[S:], v_cache[S:], nf)
        ops.decoder_attention(q, k_cache, v_cache, b["decoder_attn_buf"], q, S)
        ops.decoder_out_proj_residual(q.view(-1, DECODER_HEADS * HEAD_DIM), w["decoder_attn_o_w"][layer], x)
        ops.decoder_norm_gated_ffn(x, w["decoder_ffn_gate_w"][layer], w["decoder_ffn_up_w"][layer],
                                   b["decoder_hidden"], nf)
        ops.decoder_ffn_down_residual(b["decoder_hidden"], w["decoder_ffn_down_w"][layer], x)
    ops.decoder_action_out_proj(x[1:], w["decoder_action_fused_out_proj_w"],
                                w["decoder_action_fused_out_proj_b"], noise, nf)


def decoder_prologue_batched(ops, weights, dec):
    """`decoder_prologue` for the batched decoder buffers: all episodes' state tokens in one projection."""
    ops.decoder_state_proj(dec["observation_state_normalized"], weights["decoder_state_in_proj_w"],
                           weights["decoder_state_in_proj_b"], dec["decoder_state_buf"])
    dec["diffusion_noise_f32"].copy_(dec["diffusion_noise"].view(-1, dec["diffusion_noise"].shape[-1]))


def decoder_step_batched(ops, weights, prefix, dec, encoder_seq_len, step, episodes, layers=ENCODER_LAYERS,
                         before_layer=None):
    """One Euler step of ALL episodes at once: every projection of the action expert runs over the
    episodes' rows laid end to end (M = episodes x (chunk + 1)), so the decoder's weights are streamed once
    per layer-step for the whole batch; attention runs per episode inside one launch, each episode against
    its own KV cache. Same ops and order per layer as `decoder_step`."""
    w, S, E = weights, encoder_seq_len, episodes
    x, nf, q = dec["decoder_x"], dec["decoder_norm_factor_buf"], dec["decoder_q_buf"]
    D = x.shape[0] // E
    x3 = x.view(E, D, x.shape[1])
    x3[:, 0].copy_(dec["decoder_state_buf"])
    ops.decoder_action_in_proj(dec["diffusion_noise_f32"], w["decoder_action_fused_in_proj_w"],
                               w["decoder_action_fused_time_biases"][step % DIFFUSION_STEPS], dec["decoder_x_buf"])
    ops.decoder_action_mlp(dec["decoder_x_buf"], w["decoder_action_mlp_w"], w["decoder_action_mlp_b"], dec["decoder_mlp_out"])
    x3[:, 1:].copy_(dec["decoder_mlp_out"].view(E, D - 1, x.shape[1]))
    for layer in range(layers):
        k_all, v_all = prefix["encoder_K"][:, layer], prefix["encoder_V"][:, layer]      # (E, S + D, 256) views
        if before_layer is not None:
            before_layer(layer)
        ops.decoder_norm_qkv_rope(x, w["decoder_attn_qkv_w"][layer], dec["decoder_rope_weights"], q,
                                  k_all[:, S:], v_all[:, S:], nf)
        ops.decoder_attention(q, k_all, v_all, None, q, S)
        # the two residual projections see the rows as E groups of D (3-D operands): with D <= 64 the backend
        # runs its weight-streaming decoder kernel once per episode inside one launch
        ops.decoder_out_proj_residual(q.view(E, D, DECODER_HEADS * HEAD_DIM), w["decoder_attn_o_w"][layer], x3)
        ops.decoder_norm_gated_ffn(x, w["decoder_ffn_gate_w"][layer], w["decoder_ffn_up_w"][layer], dec["decoder_hidden"], nf)
        ops.decoder_ffn_down_residual(dec["decoder_hidden"].view(E, D, -1), w["decoder_ffn_down_w"][layer], x3)
    dec["decoder_x_rows"].view(E, D - 1, x.shape[1]).copy_(x3[:, 1:])
    ops.decoder_action_out_proj(dec["decoder_x_rows"], w["decoder_action_fused_out_proj_w"],
                                w["decoder_action_fused_out_proj_b"], dec["diffusion_noise_f32"], nf)


def decoder_epilogue_batched(dec):
    dec["diffusion_noise"].view(-1, dec["diffusion_noise"].shape[-1]).copy_(dec["diffusion_noise_f32"])


def decoder_prologue(ops, weights, buffers):
    """What the decoder needs before its first step and that does not depend on the encoder: the state
    token's projection and the fp32 master copy of the noise."""
    b = buffers
    ops.decoder_state_proj(b["observation_state_normalized"], weights["decoder_state_in_proj_w"],
                           weights["decoder_state_in_proj_b"], b["decoder_state_buf"])
    master = b.get("diffusion_noise_f32")
    if master is not None:
        _copy(ops, master, b["diffusion_noise"])


def decoder_epilogue(buffers, ops=None):
    """Refresh the bf16 action chunk from its fp32 master."""
    master = buffers.get("diffusion_noise_f32")
    if master is not None:
        _copy(ops, buffers["diffusion_noise"], master)


def transformer_decoder(ops, weights, buffers, encoder_seq_len, steps=DIFFUSION_STEPS,
                        layers=ENCODER_LAYERS, first_step=0):
    """Denoise the action chunk in `diffusion_noise` over `steps` Euler steps. `first_step > 0` resumes
    after steps that were run separately (prologue included), see `Pi0Inference`."""
    b = buffers
    master = b.get("diffusion_noise_f32")
    if first_step == 0:
        decoder_prologue(ops, weights, b)
    for step in range(first_step, steps):
        decoder_step(ops, weights, b, encoder_seq_len, step, layers, noise=master)
    decoder_epilogue(b, ops)
