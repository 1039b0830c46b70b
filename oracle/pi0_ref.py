"""CPU restatement of the Pi0 forward pass of revollllt/flash-vla. TEST INFRASTRUCTURE ONLY.

This file is the parity oracle and the timed CPU baseline. It is never on the
product path: only `tests/`, `__graft_entry__.smoke()` and the `cpu_baseline` /
`--impl reference` legs of `bench.py` import it.

PARITY PINNED BY THE REFERENCE'S OWN GPU CODE: the reference ships no golden vectors, no
known-answer tests and no CPU or PyTorch implementation of its pipeline, so the oracle is a
line-by-line restatement of the reference's kernel sources (citations below are paths inside that
project). What pins it is a fixture made by running the reference itself (its TileLang kernels, op
table, pipeline and engine, from an installed copy, on a B200):
`tests/golden/reference_gpu.pt`, produced by `tests/golden/make_reference_gpu_golden.py`.
`tests/test_reference_gpu_parity.py` holds every op of this oracle's table, its whole forward and
its one-decoder-step configuration to those outputs (every op inside the default elementwise bound).
Only the reference's fused op table (its engine's default) was run: the three unfused decoder
forms it replaces (three-kernel attention, separate norm-factor forms of the gated FFN and the
action projection) are pinned through the fused forms only. Beside that, `tests/test_oracle.py`
checks the ops against independent one-line torch expressions and, where the reference has
CPU-runnable pieces (`rope_table`, `random_checkpoint`, its torch attention functions, its
`pipeline.py` orchestration), against those pieces themselves via committed fixtures
(`tests/golden/make_golden.py`).

Every op has the positional signature of the reference's call-site wrapper of
the same name (`.../h100/pi0/backends/tilelang/wrappers.py`,
`fused_wrappers.py`) and writes its destination in place, so the same
orchestration can drive either this oracle or the CUDA backend.

Three precision levels:
  * fp32 buffers + `faithful=False`: bf16-valued inputs upcast, every
    intermediate kept in fp32. This is the parity target.
  * bf16 buffers + `faithful=False`: each op output is rounded to bf16 when it
    is stored, as any bf16-storage implementation must.
  * `faithful=True`: additionally rounds at the reference kernels' internal
    rounding points (listed per op), to attribute differences.

A fourth switch, `operands_bf16=True` (decoder ops only), answers a different question: how far
from the fp32 result must ANY bf16 tensor-core implementation land? It rounds to bf16 exactly
the activation operands a tensor-core GEMM has to take in bf16 (the rows fed to the QKV, gate/up,
out, down and action-MLP projections; Q, K, V and the probabilities in attention) and keeps the
residual stream, every accumulator, the norm factors, RoPE and the Euler update in fp32. The
distance of that run from the plain fp32 run is the floor below which the step tolerance of a
config cannot be pushed by better kernels.
"""
from __future__ import annotations

import math
from types import SimpleNamespace

import torch
import torch.nn.functional as F

VISION_LAYERS = 27
ENCODER_LAYERS = 18
HEAD_DIM = 256
HEADS = 8
VISION_TOKENS = 256
VISION_DIM = 1152
VISION_HEADS = 16
VISION_HEAD_DIM = 72
PATCH_FEATURES = 588
ROPE_THETA = 10000
GELU_C0 = 1.5957691216057308     # kernels/base.py:69
GELU_C1 = 0.044715               # kernels/base.py:70

bf16 = torch.bfloat16


def _f(x: torch.Tensor) -> torch.Tensor:
    return x if x.dtype == torch.float32 else x.float()


def _r(x: torch.Tensor, on: bool) -> torch.Tensor:
    """Round through bf16 when `on` (a reference rounding point), else identity."""
    return x.to(bf16).float() if on else x


def gelu(v: torch.Tensor) -> torch.Tensor:
    """v * sigmoid(C0 * v * (1 + C1 v^2)) == tanh-GELU (kernels/base.py:77-78)."""
    return v * torch.sigmoid(GELU_C0 * v * (1.0 + GELU_C1 * v * v))


def silu(v: torch.Tensor) -> torch.Tensor:
    """kernels/base.py:73-74."""
    return v * torch.sigmoid(v)


def rms_factor(x: torch.Tensor) -> torch.Tensor:
    """rsqrt(mean(x^2) + 1e-6) per row (kernels/base.py:344-370); no learned weight."""
    x = _f(x)
    return torch.rsqrt((x * x).mean(dim=-1) + 1e-6)


def layer_norm(x, w, b, eps=1e-5):
    """(x - mean) * rsqrt(E[x^2] - mean^2 + eps) * w + b (kernels/base.py:406-447)."""
    x = _f(x)
    mean = x.mean(dim=-1, keepdim=True)
    var = (x * x).mean(dim=-1, keepdim=True) - mean * mean
    return (x - mean) * torch.rsqrt(var + eps) * _f(w) + _f(b)


def rope_table(seq_len: int, offset: int, head_dim: int = HEAD_DIM) -> torch.Tensor:
    """Row r = [cos t0, sin t0, cos t1, sin t1, ...], t_p = (offset + r) * theta^(-2p/head_dim),
    cos/sin rounded to bf16 (hardware/nvidia/h100/pi0/buffers.py:15-23)."""
    pos = torch.arange(seq_len) + offset
    inv = 1.0 / (ROPE_THETA ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    phase = inv[None, :] * pos[:, None]
    return torch.stack([torch.cos(phase).to(bf16), torch.sin(phase).to(bf16)], dim=2).reshape(
        seq_len, head_dim)


def _rotate_scatter(proj, rope, Q, K, V):
    """Rotate adjacent column pairs of the Q and K parts, scatter into Q / K / V.

    proj (M, (heads + 2) * hd) fp32. Pair (2p, 2p+1) of every Q head and of K is
    rotated by (cos, sin) = rope[row, 2p], rope[row, 2p+1]; V is copied
    (kernels/base.py:651-669, :696-726).
    """
    M = proj.shape[0]
    hd = V.shape[1]
    heads = Q.shape[0] // M
    rope = _f(rope)[:M]
    cos, sin = rope[:, 0::2], rope[:, 1::2]                     # (M, hd/2)
    qk = proj[:, :(heads + 1) * hd].reshape(M, heads + 1, hd // 2, 2)
    x0, x1 = qk[..., 0], qk[..., 1]
    rot = torch.stack([x0 * cos[:, None] - x1 * sin[:, None],
                       x1 * cos[:, None] + x0 * sin[:, None]], dim=-1).reshape(M, heads + 1, hd)
    Q.view(M, heads * hd).copy_(rot[:, :heads].reshape(M, heads * hd))
    K.copy_(rot[:, heads])
    V.copy_(proj[:, (heads + 1) * hd:])


def _make_ops(fused: bool, faithful: bool, operands_bf16: bool = False) -> dict:
    R = faithful
    A = operands_bf16

    def _a(x):
        """A tensor-core activation operand: bf16 when `operands_bf16`, else as stored."""
        return _r(_f(x), A)

    # ------------------------------------------------------------------ vision
    def vision_patch_embed(images, patch_w, patch_b, pos_emb, out):
        """wrappers.py:252-265 + kernels/base.py:232-269."""
        views = images.shape[0]
        M = views * VISION_TOKENS
        patches = (_f(images).view(views, 16, 14, 16, 14, 3).permute(0, 1, 3, 2, 4, 5)
                   .reshape(M, PATCH_FEATURES))
        y = patches @ _f(patch_w).reshape(PATCH_FEATURES, VISION_DIM) + _f(patch_b)
        y = y + _f(pos_emb)[torch.arange(M) % VISION_TOKENS]
        out.view(M, VISION_DIM).copy_(y)
        return out

    def vision_norm_qkv(x, norm_w, norm_b, qkv_w, qkv_b, out, x_norm):
        """wrappers.py:268-276: LayerNorm (stored bf16 in x_norm) then x_norm @ W + b."""
        M = x.shape[0] * VISION_TOKENS
        xn = layer_norm(x.view(M, VISION_DIM), norm_w, norm_b)
        x_norm.view(M, VISION_DIM).copy_(xn)
        xn = _r(xn, R)
        out.view(M, -1).copy_(xn @ _f(qkv_w) + _f(qkv_b))
        return out

    def vision_attention(QKV, out=None):
        """kernels/attention.py:20-26: per view, 16 heads x 72, softmax(QK^T / sqrt(72)) V."""
        views = QKV.shape[0]
        q, k, v = _f(QKV).view(views, VISION_TOKENS, 3, VISION_HEADS, VISION_HEAD_DIM).permute(
            2, 0, 3, 1, 4)
        s = (q @ k.transpose(-1, -2)) * (VISION_HEAD_DIM ** -0.5)
        p = _r(torch.softmax(s, dim=-1), R)
        o = (p @ v).transpose(1, 2).reshape(views, VISION_TOKENS, VISION_DIM)
        if out is None:
            return o.to(QKV.dtype)
        out.view(views, VISION_TOKENS, VISION_DIM).copy_(o)
        return out

    def vision_out_proj_residual(x, weight, bias, res, out):
        """wrappers.py:279-288: out = x @ W + b + res (res aliases out)."""
        M = x.shape[0] * VISION_TOKENS if x.dim() == 3 else x.shape[0]
        y = _f(x).reshape(M, -1) @ _f(weight) + _f(bias) + _f(res).reshape(M, -1)
        out.view(M, -1).copy_(y)
        return out

    def vision_norm_ffn_up(x, norm_w, norm_b, weight, bias, out, x_norm):
        """wrappers.py:291-298: LayerNorm then gelu(x_norm @ W + b)."""
        M = x.shape[0] * VISION_TOKENS
        xn = layer_norm(x.view(M, VISION_DIM), norm_w, norm_b)
        x_norm.view(M, VISION_DIM).copy_(xn)
        xn = _r(xn, R)
        out.view(M, -1).copy_(gelu(xn @ _f(weight) + _f(bias)))
        return out

    vision_ffn_down_residual = vision_out_proj_residual       # wrappers.py:301-306

    # ----------------------------------------------------------------- encoder
    def encoder_projector(x, norm_w, norm_b, proj_w, proj_b, out, x_norm):
        """wrappers.py:336-344: final vision LayerNorm, then project to encoder width."""
        M = x.shape[0] * VISION_TOKENS
        xn = layer_norm(x.view(M, VISION_DIM), norm_w, norm_b)
        x_norm.view(M, VISION_DIM).copy_(xn)
        xn = _r(xn, R)
        out[:M].copy_(xn @ _f(proj_w) + _f(proj_b))
        return out

    def encoder_norm_qkv_rope(x, weight_qkv, rope, Q, K, V, x_norm):
        """wrappers.py:347-363: x_norm = bf16(x * rstd); proj = bf16(x_norm @ W);
        rotate in fp32 on the rounded projection (kernels/base.py:672-726)."""
        M = x.shape[0]
        xn = _f(x) * rms_factor(x)[:, None]
        x_norm[:M].copy_(xn)
        proj = _r(_r(xn, R) @ _f(weight_qkv), R)
        _rotate_scatter(proj, rope, Q, K, V)

    def encoder_attention(Q, K, V, scale, out=None):
        """kernels/attention.py:29-34: multi-query, unmasked; flat row = token * 8 + head."""
        s = _r(_r(_f(Q) @ _f(K).T, R) * scale, R)
        p = _r(torch.softmax(s, dim=-1), R)
        o = (p @ _f(V)).view(-1, HEADS * HEAD_DIM)
        if out is None:
            return o.to(Q.dtype)
        out.view(-1, HEADS * HEAD_DIM).copy_(o)
        return out

    def encoder_out_proj_residual(x, weight, out):
        """wrappers.py:366-371: out += x @ W."""
        out.copy_(_f(out) + _f(x) @ _f(weight))
        return out

    def encoder_norm_gated_ffn(x, gate_w, up_w, out, x_norm):
        """wrappers.py:374-380: bf16 RMS norm, then gelu(xn @ Wg) * (xn @ Wu)."""
        M = x.shape[0]
        xn = _f(x) * rms_factor(x)[:, None]
        x_norm[:M].copy_(xn)
        xn = _r(xn, R)
        out[:M].copy_(gelu(xn @ _f(gate_w)) * (xn @ _f(up_w)))
        return out

    encoder_ffn_down_residual = encoder_out_proj_residual      # wrappers.py:383-392

    # ----------------------------------------------------------------- decoder
    def decoder_state_proj(x, weight, bias, out):
        """wrappers.py:108-112."""
        out.copy_(_f(x).view(1, -1) @ _f(weight) + _f(bias))
        return out

    def decoder_action_in_proj(x, weight, bias, out):
        """wrappers.py:115-120: silu(x @ W + time_bias)."""
        out.copy_(silu(_f(x) @ _f(weight) + _f(bias)))
        return out

    def decoder_action_mlp(x, weight, bias, out):
        """wrappers.py:123-128."""
        out.copy_(_a(x) @ _f(weight) + _f(bias))
        return out

    def decoder_norm_qkv_rope(x, weight_qkv, rope, Q, K, V, norm_factor):
        """wrappers.py:131-144: factor (stored bf16) scales the fp32 accumulator, RoPE in
        fp32, one rounding at the store (kernels/base.py:647-669)."""
        M = x.shape[0]
        f = rms_factor(x)
        norm_factor[:M].copy_(f)
        proj = (_a(x) @ _f(weight_qkv)) * _r(f, R)[:, None]
        _rotate_scatter(proj, rope, Q, K, V)

    def _attn_mask(queries, keys, encoder_seq_len):
        gi = torch.arange(queries)[:, None]
        j = torch.arange(keys)[None, :]
        return (gi >= HEADS) | (j <= encoder_seq_len)          # kernels/base.py:790, :858-862

    def decoder_attention(Q, K, V, scores, out, encoder_seq_len):
        """Unfused: wrappers.py:147-173 (bf16 scores, bf16 probabilities written to
        `scores`). Fused: fused_wrappers.py:88-115 (flash-decoding; `scores` untouched).
        The state token (flat rows 0..7) sees the prefix and itself; action tokens see all."""
        queries, hd = Q.shape
        keys = K.shape[0]
        s = (_a(Q) @ _a(K).T) * (hd ** -0.5)
        if not fused:
            s = _r(s, R)
        s = s.masked_fill(~_attn_mask(queries, keys, encoder_seq_len), float("-inf"))
        p = torch.softmax(s, dim=-1)
        if not fused:
            scores[:, :keys].copy_(p)
        o = _r(p, R or A) @ _a(V)
        out.copy_(o)
        return out

    def decoder_out_proj_residual(x, weight, out):
        """wrappers.py:176-181."""
        out.copy_(_f(out) + _a(x) @ _f(weight))
        return out

    decoder_ffn_down_residual = decoder_out_proj_residual       # wrappers.py:184-189

    def decoder_norm_gated_ffn(x, gate_w, up_w, out, norm_factor):
        """Unfused (wrappers.py:192-198, kernels/base.py:453-505): x * F rounded to bf16 per
        element before the GEMM. Fused (kernels/fused_norm.py:26-78): fp32 accumulators
        scaled by the bf16-rounded factor; `norm_factor` untouched."""
        M = x.shape[0]
        f = rms_factor(x)
        if fused:
            g = (_a(x) @ _f(gate_w)) * _r(f, R)[:, None]
            u = (_a(x) @ _f(up_w)) * _r(f, R)[:, None]
        else:
            norm_factor[:M].copy_(f)
            xs = _r(_f(x) * _r(f, R)[:, None], R)
            g, u = xs @ _f(gate_w), xs @ _f(up_w)
        out.copy_(gelu(g) * u)
        return out

    def decoder_action_out_proj(x, weight, bias, out, norm_factor):
        """out += b + rms(x) @ W, the Euler update (wrappers.py:201-208 /
        kernels/fused_norm.py:81-125)."""
        M = x.shape[0]
        f = rms_factor(x)
        if fused:
            y = (_f(x) @ _f(weight)) * _r(f, R)[:, None]
        else:
            norm_factor[:M].copy_(f)
            y = _r(_f(x) * _r(f, R)[:, None], R) @ _f(weight)
        out.copy_(_f(out) + _f(bias) + y)
        return out

    return {k: v for k, v in locals().items() if callable(v) and not k.startswith("_")}



def op_table(fused: bool = True, faithful: bool = False, operands_bf16: bool = False) -> SimpleNamespace:
    """Oracle op table: the 19 reference op names plus `vision_attention` and
    `encoder_attention` (which the reference pipeline imports directly)."""
    return SimpleNamespace(**_make_ops(fused, faithful, operands_bf16))


# ---------------------------------------------------------------------------
# Buffers and orchestration (hardware/nvidia/h100/pi0/buffers.py:26-64,
# pipeline.py:21-135, engine.py:58-65), restated independently of the package.
# ---------------------------------------------------------------------------
def allocate_buffers(num_views: int, chunk_size: int, prompt_len: int, dtype=torch.float32):
    S = num_views * VISION_TOKENS + prompt_len
    D = chunk_size + 1
    cache = S + D

    def buf(*shape):
        return torch.zeros(shape, dtype=dtype)

    b = {
        "observation_images_normalized": buf(num_views, 224, 224, 3),
        "observation_state_normalized": buf(32),
        "diffusion_noise": buf(chunk_size, 32),
        "vision_x": buf(num_views, VISION_TOKENS, VISION_DIM),
        "vision_x_norm": buf(num_views, VISION_TOKENS, VISION_DIM),
        "vision_QKV": buf(num_views, VISION_TOKENS, 3 * VISION_DIM),
        "vision_attn": buf(num_views, VISION_TOKENS, VISION_DIM),
        "vision_hidden": buf(num_views, VISION_TOKENS, 4304),
        "encoder_rope_weights": rope_table(S, 0).to(dtype),
        "encoder_x": buf(S, 2048),
        "encoder_x_norm": buf(S, 2048),
        "encoder_K": buf(ENCODER_LAYERS, cache, HEAD_DIM),
        "encoder_V": buf(ENCODER_LAYERS, cache, HEAD_DIM),
        "encoder_Q": buf(S * HEADS, HEAD_DIM),
        "encoder_attn": buf(S, HEADS * HEAD_DIM),
        "encoder_hidden": buf(S, 16384),
        "decoder_rope_weights": rope_table(D, S).to(dtype),
        "decoder_x": buf(D, 1024),
        "decoder_x_buf": buf(chunk_size, 1024),
        "decoder_state_buf": buf(1, 1024),
        "decoder_norm_factor_buf": buf(D),
        "decoder_q_buf": buf(D * HEADS, HEAD_DIM),
        "decoder_attn_buf": buf(D * HEADS, cache),
        "decoder_hidden": buf(D, 4096),
    }
    return b, S


def vision_encoder(ops, w, b, num_views, layers=None):
    """`layers` < 27 runs a prefix of the tower (used only for bounded timing samples)."""
    ops.vision_patch_embed(b["observation_images_normalized"], w["vision_patch_embedding_w"],
                           w["vision_patch_embedding_b"], w["vision_position_embedding"],
                           b["vision_x"])
    for i in range(VISION_LAYERS if layers is None else layers):
        ops.vision_norm_qkv(b["vision_x"], w["vision_pre_attn_norm_w"][i],
                            w["vision_pre_attn_norm_b"][i], w["vision_attn_qkv_w"][i],
                            w["vision_attn_qkv_b"][i], b["vision_QKV"], b["vision_x_norm"])
        ops.vision_attention(b["vision_QKV"], b["vision_attn"])
        ops.vision_out_proj_residual(b["vision_attn"], w["vision_attn_o_w"][i],
                                     w["vision_attn_o_b"][i], b["vision_x"], b["vision_x"])
        ops.vision_norm_ffn_up(b["vision_x"], w["vision_pre_ffn_norm_w"][i],
                               w["vision_pre_ffn_norm_b"][i], w["vision_ffn_up_w"][i],
                               w["vision_ffn_up_b"][i], b["vision_hidden"], b["vision_x_norm"])
        ops.vision_ffn_down_residual(b["vision_hidden"], w["vision_ffn_down_w"][i],
                                     w["vision_ffn_down_b"][i], b["vision_x"], b["vision_x"])


def transformer_encoder(ops, w, b, S, layers=None):
    """`layers` < 18 runs that many full layers (used only for bounded timing samples)."""
    ops.encoder_projector(b["vision_x"], w["vision_final_norm_w"], w["vision_final_norm_b"],
                          w["encoder_multi_modal_projector_w"],
                          w["encoder_multi_modal_projector_b"], b["encoder_x"], b["vision_x_norm"])
    for i in range(ENCODER_LAYERS if layers is None else layers):
        ops.encoder_norm_qkv_rope(b["encoder_x"], w["encoder_attn_qkv_w"][i],
                                  b["encoder_rope_weights"], b["encoder_Q"],
                                  b["encoder_K"][i, :S], b["encoder_V"][i, :S], b["encoder_x_norm"])
        if layers is None and i == ENCODER_LAYERS - 1:
            break
        ops.encoder_attention(b["encoder_Q"], b["encoder_K"][i, :S], b["encoder_V"][i, :S],
                              HEAD_DIM ** -0.5, b["encoder_attn"])
        ops.encoder_out_proj_residual(b["encoder_attn"], w["encoder_attn_o_w"][i], b["encoder_x"])
        ops.encoder_norm_gated_ffn(b["encoder_x"], w["encoder_ffn_gate_w"][i],
                                   w["encoder_ffn_up_w"][i], b["encoder_hidden"],
                                   b["encoder_x_norm"])
        ops.encoder_ffn_down_residual(b["encoder_hidden"], w["encoder_ffn_down_w"][i],
                                      b["encoder_x"])


def decoder_step(ops, w, b, S, step, layers=18):
    """One flow-matching Euler step (pipeline.py:103-135); `step % 10` selects the time bias."""
    b["decoder_x"][:1].copy_(b["decoder_state_buf"])
    ops.decoder_action_in_proj(b["diffusion_noise"], w["decoder_action_fused_in_proj_w"],
                               w["decoder_action_fused_time_biases"][step % 10], b["decoder_x_buf"])
    ops.decoder_action_mlp(b["decoder_x_buf"], w["decoder_action_mlp_w"],
                           w["decoder_action_mlp_b"], b["decoder_x"][1:])
    for i in range(layers):
        ops.decoder_norm_qkv_rope(b["decoder_x"], w["decoder_attn_qkv_w"][i],
                                  b["decoder_rope_weights"], b["decoder_q_buf"],
                                  b["encoder_K"][i][S:], b["encoder_V"][i][S:],
                                  b["decoder_norm_factor_buf"])
        ops.decoder_attention(b["decoder_q_buf"], b["encoder_K"][i], b["encoder_V"][i],
                              b["decoder_attn_buf"], b["decoder_q_buf"], S)
        ops.decoder_out_proj_residual(b["decoder_q_buf"].view(-1, 2048), w["decoder_attn_o_w"][i],
                                      b["decoder_x"])
        ops.decoder_norm_gated_ffn(b["decoder_x"], w["decoder_ffn_gate_w"][i],
                                   w["decoder_ffn_up_w"][i], b["decoder_hidden"],
                                   b["decoder_norm_factor_buf"])
        ops.decoder_ffn_down_residual(b["decoder_hidden"], w["decoder_ffn_down_w"][i],
                                      b["decoder_x"])
    ops.decoder_action_out_proj(b["decoder_x"][1:], w["decoder_action_fused_out_proj_w"],
                                w["decoder_action_fused_out_proj_b"], b["diffusion_noise"],
                                b["decoder_norm_factor_buf"])


def transformer_decoder(ops, w, b, S, steps=10, layers=18, trace=None):
    ops.decoder_state_proj(b["observation_state_normalized"], w["decoder_state_in_proj_w"],
                           w["decoder_state_in_proj_b"], b["decoder_state_buf"])
    for step in range(steps):
        decoder_step(ops, w, b, S, step, layers)
        if trace is not None:
            trace.append(b["diffusion_noise"].float().clone())


def forward(w, images, state, noise, num_views=3, chunk_size=50, steps=10, layers=18,
            fused=True, faithful=False, dtype=torch.float32, trace=None, buffers=None):
    """Whole Pi0 forward on the CPU; returns (actions, buffers). `w` maps checkpoint names
    to tensors (bf16 or pre-upcast fp32)."""
    prompt_len = w["language_embeds"].shape[0]
    if buffers is None:
        b, S = allocate_buffers(num_views, chunk_size, prompt_len, dtype)
    else:
        b, S = buffers, num_views * VISION_TOKENS + prompt_len
    ops = op_table(fused, faithful)
    b["observation_images_normalized"].copy_(images)
    b["observation_state_normalized"].copy_(state)
    b["diffusion_noise"].copy_(noise)
    b["encoder_x"][num_views * VISION_TOKENS:].copy_(w["language_embeds"])     # engine.py:60
    vision_encoder(ops, w, b, num_views)
    transformer_encoder(ops, w, b, S)
    transformer_decoder(ops, w, b, S, steps, layers, trace)
    return b["diffusion_noise"], b


def embed_prompt(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """language_embeds = table[ids]: a plain row gather, no scaling. An extension beyond the
    reference (which only accepts precomputed `language_embeds`, engine.py:43, :60)."""
    return table[ids]


def error_metrics(reference: torch.Tensor, output: torch.Tensor) -> dict:
    """max/mean/RMS/P99 absolute error and cosine (eval/correctness/pi0/openpi_parity.py:14-28)."""
    a, o = reference.float().flatten(), output.float().flatten()
    err = (o - a).abs()
    return {"max_abs": err.max().item(), "mean_abs": err.mean().item(),
            "rms_error": math.sqrt(((o - a) ** 2).mean().item()),
            "p99_abs": torch.quantile(err, 0.99).item(),
            "cosine_similarity": F.cosine_similarity(a, o, dim=0).item()}
