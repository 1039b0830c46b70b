"""Call-site wrappers of the CUDA backend: one function per Pi0 operation.

Names and positional signatures are those of the reference's TileLang wrappers
(`.../h100/pi0/backends/tilelang/wrappers.py:108-208`, `:252-306`, `:336-392`): torch
tensors in, destination passed in and written in place. Each wrapper checks its tensors on
the host, takes any scratch it needs from the active `ScratchPool`, and makes one call into
libfvla_b200 on torch's current stream. Two names are added to the reference's nineteen,
`vision_attention` and `encoder_attention`, which the reference pipeline calls as torch
functions outside its table (`pipeline.py:16`).
"""
from __future__ import annotations

import contextlib

import torch

from flash_vla_b200.runtime.cuda import ScratchPool

from . import _lib

_POOL = ScratchPool()

DECODER_HEADS = 8
VISION_TOKENS = 256
VISION_DIM = 1152
VISION_HEADS = 16
VISION_HEAD_DIM = 72


def set_pool(pool: ScratchPool) -> None:
    """Install the scratch pool used by every wrapper."""
    global _POOL
    _POOL = pool


@contextlib.contextmanager
def use_pool(pool: ScratchPool):
    """Route scratch requests through `pool` for the duration of the block."""
    global _POOL
    previous, _POOL = _POOL, pool
    try:
        yield
    finally:
        _POOL = previous


# A bf16 shadow is a bf16 copy of an fp32 tensor that every op of this backend refreshes when it writes
# the fp32 tensor, so that the GEMMs reading the tensor can fetch ready-made bf16 rows by TMA instead of
# converting fp32 in the kernel. The pairing lives ON the fp32 tensor object (an attribute), not in a
# table keyed by address: it is found again through `view._base`, it cannot outlive the tensor, and a
# later allocation that happens to reuse the address is never mistaken for it. Code that writes a
# registered tensor by other means must call `sync_shadow` afterwards.
_SHADOW_ATTR = "_fvla_bf16_shadow"


def register_bf16_shadow(master: torch.Tensor, shadow: torch.Tensor) -> None:
    """Declare `shadow` (bf16, same shape, contiguous) as the maintained copy of fp32 `master`."""
    if master.dtype != torch.float32 or shadow.dtype != torch.bfloat16 or master.shape != shadow.shape:
        raise ValueError("register_bf16_shadow: need an fp32 master and a bf16 shadow of equal shape")
    if not (master.is_contiguous() and shadow.is_contiguous()):
        raise ValueError("register_bf16_shadow: tensors must be contiguous")
    if master._base is not None:
        raise ValueError("register_bf16_shadow: register the owning tensor, not a view of it")
    setattr(master, _SHADOW_ATTR, shadow)
    shadow.copy_(master)


def unregister_bf16_shadow(master: torch.Tensor) -> None:
    if hasattr(master, _SHADOW_ATTR):
        delattr(master, _SHADOW_ATTR)


def _shadow_and_offset(t: torch.Tensor):
    """(shadow tensor, element offset of `t` inside its owner) when `t` is a registered fp32 tensor or a
    contiguous view of one, else (None, 0)."""
    if not isinstance(t, torch.Tensor) or t.dtype != torch.float32:
        return None, 0
    owner = t if t._base is None else t._base
    shadow = getattr(owner, _SHADOW_ATTR, None)
    if shadow is None:
        return None, 0
    return shadow, (t.data_ptr() - owner.data_ptr()) // 4


def _shadow_of(t: torch.Tensor):
    """Device address inside the registered shadow that mirrors the first element of `t` (which may be
    a row-offset view of the master), or None."""
    shadow, first = _shadow_and_offset(t)
    return None if shadow is None else shadow.data_ptr() + 2 * first


def sync_shadow(t: torch.Tensor) -> None:
    """Refresh the shadow rows mirroring `t` after `t` was written outside this backend."""
    shadow, first = _shadow_and_offset(t)
    if shadow is not None:
        shadow.view(-1)[first:first + t.numel()].copy_(t.reshape(-1))


def copy_rows(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """dst.copy_(src) for contiguous bf16 / fp32 CUDA tensors of equal size, as one kernel of this library
    (it also refreshes the bf16 shadow of a registered fp32 `dst`). The pipeline's small copies (state token
    into the residual stream, action chunk to and from its fp32 master) use it so that no framework kernel
    interrupts the chain of dependent launches. Not in the reference table, where these are torch copies."""
    if dst.numel() != src.numel():
        raise ValueError(f"copy_rows: {src.numel()} elements into {dst.numel()}")
    _lib.call("fvla_convert_copy", _chk("src", src, dtype=None), _is_f32("src", src), _chk("dst", dst, dtype=None),
              _is_f32("dst", dst), _shadow_of(dst), dst.numel(), _stream())
    return dst


def embed_prompt(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = table[ids[r]]: the prompt embedding lookup (a plain row gather, no scaling). Not in the
    reference table, which only accepts precomputed `language_embeds` (engine.py:43, :60)."""
    vocab, dim = table.shape
    rows = ids.numel()
    if ids.dtype != torch.int64 or not ids.is_cuda or not ids.is_contiguous():
        raise ValueError("embed_prompt: ids must be a contiguous int64 CUDA tensor")
    if tuple(out.shape) != (rows, dim):
        raise ValueError(f"embed_prompt: out has shape {tuple(out.shape)}, expected {(rows, dim)}")
    if rows:
        _lib.call("fvla_embed_rows", _chk("table", table), ids.data_ptr(), _chk("out", out), rows, dim, vocab, _stream())
    return out


def scratch(role: str, shape, dtype, device) -> torch.Tensor:
    """Graph-safe temporary from the pool that is active at call time."""
    return _POOL.get(role, shape, dtype, device)


def _ws(role: str, nbytes: int, device):
    """(pointer, size) of a zero-initialised byte scratch, or (None, 0)."""
    if nbytes == 0:
        return None, 0
    buf = scratch(role, (nbytes,), torch.uint8, device)
    return buf.data_ptr(), nbytes


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _is_f32(name: str, t: torch.Tensor) -> int:
    """1 for an fp32 tensor, 0 for bf16; anything else is rejected."""
    if t.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"{name}: expected bf16 or fp32, got {t.dtype}")
    return int(t.dtype == torch.float32)


def _chk(name: str, t: torch.Tensor, shape=None, dtype=torch.bfloat16) -> int:
    """Validate one operand on the host and return its device address."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name}: expected a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name}: expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous tensor, got strides {t.stride()}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    return t.data_ptr()


# --------------------------------------------------------------------------- vision
def vision_patch_embed(images, patch_w, patch_b, pos_emb, out):
    """out = patches(images) @ patch_w + patch_b + pos_emb[row % 256] (wrappers.py:252-265)."""
    views = images.shape[0]
    lib = _lib.load()
    ws, nb = _ws("patches", lib.fvla_patch_embed_workspace_bytes(views), images.device)
    _lib.call("fvla_vision_patch_embed", _chk("images", images, (views, 224, 224, 3)),
              _chk("patch_w", patch_w, (14, 14, 3, VISION_DIM)), _chk("patch_b", patch_b, (VISION_DIM,)),
              _chk("pos_emb", pos_emb, (VISION_TOKENS, VISION_DIM)),
              _chk("out", out, (views, VISION_TOKENS, VISION_DIM)), views, ws, nb, _stream())
    return out


def _norm_linear(entry, x, norm_w, norm_b, weight, bias, out, x_norm):
    M = x.shape[0] * VISION_TOKENS
    K, N = weight.shape
    _lib.call(entry, _chk("x", x, (x.shape[0], VISION_TOKENS, K)), _chk("norm_w", norm_w, (K,)),
              _chk("norm_b", norm_b, (K,)), _chk("weight", weight), _chk("bias", bias, (N,)),
              _chk("out", out), _chk("x_norm", x_norm, x.shape), M, N, K, _stream())
    return out


def vision_norm_qkv(x, norm_w, norm_b, qkv_w, qkv_b, out, x_norm):
    """x_norm = LayerNorm(x); out = x_norm @ qkv_w + qkv_b (wrappers.py:268-276)."""
    if out.numel() != x.shape[0] * VISION_TOKENS * qkv_w.shape[1]:
        raise ValueError("vision_norm_qkv: out has the wrong size")
    return _norm_linear("fvla_vision_norm_qkv", x, norm_w, norm_b, qkv_w, qkv_b, out, x_norm)


_FOLDED_ATTR = "_fvla_folded_layernorm"


def _folded_layernorm(weight, norm_w, norm_b, bias):
    """(weight_folded, colsum, bias_folded) of `fvla_fold_layernorm` for this LayerNorm + linear pair, made on first
    use and kept ON the tensor that owns `weight`'s storage (found again through `view._base`, gone with it).
    The entry also remembers the versions of the four tensors: an in-place update of any of them refolds.
    None while a CUDA graph is being captured and nothing has been folded yet (folding allocates)."""
    owner = weight if weight._base is None else weight._base
    table = getattr(owner, _FOLDED_ATTR, None)
    if table is None:
        table = {}
        setattr(owner, _FOLDED_ATTR, table)
    key = (weight.data_ptr(), norm_w.data_ptr(), norm_b.data_ptr(), bias.data_ptr())
    versions = (weight._version, norm_w._version, norm_b._version, bias._version)
    entry = table.get(key)
    if entry is not None and entry[0] == versions:
        return entry[1]
    if torch.cuda.is_current_stream_capturing():
        return None
    K, N = weight.shape
    folded = (torch.empty_like(weight, memory_format=torch.contiguous_format),
              torch.empty(N, dtype=torch.float32, device=weight.device),
              torch.empty(N, dtype=torch.float32, device=weight.device))
    _lib.call("fvla_fold_layernorm", _chk("norm_w", norm_w, (K,)), _chk("norm_b", norm_b, (K,)), _chk("weight", weight),
              _chk("bias", bias, (N,)), folded[0].data_ptr(), folded[1].data_ptr(), folded[2].data_ptr(), N, K, _stream())
    table[key] = (versions, folded)
    return folded


def _folded_norm_linear(entry, act, x, norm_w, norm_b, weight, bias, out, x_norm):
    """The fused table's LayerNorm + linear: the norm happens inside the GEMM and `x_norm` stays untouched. Shapes
    outside the fused form (a CTA would own several tiles) and calls that would have to fold weights during
    graph capture take the two-kernel form of the unfused table."""
    M = x.shape[0] * VISION_TOKENS
    K, N = weight.shape
    folded = _folded_layernorm(weight, norm_w, norm_b, bias) if _lib.load().fvla_fused_norm_supported(M, N, K, 0) else None
    if folded is None:
        return _norm_linear(entry, x, norm_w, norm_b, weight, bias, out, x_norm)
    _lib.call("fvla_vision_folded_norm_linear", _chk("x", x, (x.shape[0], VISION_TOKENS, K)), folded[0].data_ptr(),
              folded[1].data_ptr(), folded[2].data_ptr(), _chk("out", out), M, N, K, act, _stream())
    return out


def vision_norm_qkv_fused(x, norm_w, norm_b, qkv_w, qkv_b, out, x_norm):
    """out = LayerNorm(x) @ qkv_w + qkv_b with the norm folded into the GEMM; `x_norm` is not written."""
    if out.numel() != x.shape[0] * VISION_TOKENS * qkv_w.shape[1]:
        raise ValueError("vision_norm_qkv: out has the wrong size")
    return _folded_norm_linear("fvla_vision_norm_qkv", 0, x, norm_w, norm_b, qkv_w, qkv_b, out, x_norm)


def vision_norm_ffn_up_fused(x, norm_w, norm_b, weight, bias, out, x_norm):
    """out = gelu(LayerNorm(x) @ weight + bias) with the norm folded into the GEMM; `x_norm` is not written."""
    if out.numel() != x.shape[0] * VISION_TOKENS * weight.shape[1]:
        raise ValueError("vision_norm_ffn_up: out has the wrong size")
    return _folded_norm_linear("fvla_vision_norm_ffn_up", 1, x, norm_w, norm_b, weight, bias, out, x_norm)


def vision_attention(QKV, out):
    """Per-view 16-head attention over the packed QKV buffer (kernels/attention.py:20-26)."""
    views = QKV.shape[0]
    _lib.call("fvla_vision_attention", _chk("QKV", QKV, (views, VISION_TOKENS, 3 * VISION_DIM)),
              _chk("out", out, (views, VISION_TOKENS, VISION_DIM)), views, VISION_TOKENS,
              VISION_HEADS, VISION_HEAD_DIM, _stream())
    return out


def _linear_bias_residual(role, x, weight, bias, res, out):
    K, N = weight.shape
    M = x.numel() // K
    if res.numel() != M * N or out.numel() != M * N:
        raise ValueError("linear_bias_residual: res/out have the wrong size")
    ws, nb = _ws(role, _lib.load().fvla_gemm_workspace_bytes(M, N, K, 0), x.device)
    _lib.call("fvla_vision_linear_bias_residual", _chk("x", x), _chk("weight", weight),
              _chk("bias", bias, (N,)), _chk("res", res), _chk("out", out), M, N, K, ws, nb, _stream())
    return out


def vision_out_proj_residual(x, weight, bias, res, out):
    """out = x @ weight + bias + res; res and out may be one buffer (wrappers.py:279-288)."""
    return _linear_bias_residual("vis_o_ws", x, weight, bias, res, out)


def vision_norm_ffn_up(x, norm_w, norm_b, weight, bias, out, x_norm):
    """x_norm = LayerNorm(x); out = gelu(x_norm @ weight + bias) (wrappers.py:291-298)."""
    if out.numel() != x.shape[0] * VISION_TOKENS * weight.shape[1]:
        raise ValueError("vision_norm_ffn_up: out has the wrong size")
    return _norm_linear("fvla_vision_norm_ffn_up", x, norm_w, norm_b, weight, bias, out, x_norm)


def vision_ffn_down_residual(x, weight, bias, res, out):
    """out = hidden @ weight + bias + res (wrappers.py:301-306)."""
    return _linear_bias_residual("vis_down_ws", x, weight, bias, res, out)


# -------------------------------------------------------------------------- encoder
def encoder_projector(x, norm_w, norm_b, proj_w, proj_b, out, x_norm):
    """Final vision LayerNorm, then projection into encoder width (wrappers.py:336-344)."""
    M = x.shape[0] * VISION_TOKENS
    if out.shape[0] < M or out.shape[1] != proj_w.shape[1]:
        raise ValueError("encoder_projector: out is too small")
    return _norm_linear("fvla_encoder_projector", x, norm_w, norm_b, proj_w, proj_b, out, x_norm)


def _kv_destination(name: str, t: torch.Tensor, M: int, hd: int):
    """K / V destination of the prefix QKV projection as (address, sequence rows, pitch in rows).
    2-D (M, hd) contiguous: one sequence. 3-D (sequences, rows, hd) whose (rows, hd) blocks are contiguous
    and evenly spaced: a batch of episodes, each block being the prefix rows of that episode's cache."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.bfloat16:
        raise ValueError(f"{name}: expected a bf16 CUDA tensor")
    if t.ndim == 2:
        return _chk(name, t, (M, hd)), 0, 0
    if t.ndim != 3 or t.shape[2] != hd or t.shape[0] * t.shape[1] != M or t.stride(2) != 1 or t.stride(1) != hd \
            or t.stride(0) % hd or t.stride(0) < t.shape[1] * hd:
        raise ValueError(f"{name}: expected (M, hd) or evenly spaced (sequences, rows, hd) blocks, got shape "
                         f"{tuple(t.shape)} strides {t.stride()}")
    return t.data_ptr(), t.shape[1], t.stride(0) // hd


def encoder_norm_qkv_rope(x, weight_qkv, rope, Q, K, V, x_norm, _entry="fvla_encoder_norm_qkv_rope"):
    """RMS norm, QKV projection rounded to bf16, RoPE, scatter to Q/K/V (wrappers.py:347-363).

    Extension for batches of episodes: when K and V are 3-D views (episodes, S, hd) of the episodes' caches,
    x holds the episodes' S-row sequences end to end, `rope` is the table of ONE sequence, and each episode's
    K / V rows land in its own cache."""
    M, Kdim = x.shape
    hd = V.shape[-1]
    heads = Q.shape[0] // M
    k_ptr, group, pitch = _kv_destination("K", K, M, hd)
    v_ptr, group_v, pitch_v = _kv_destination("V", V, M, hd)
    if (group, pitch) != (group_v, pitch_v):
        raise ValueError("encoder_norm_qkv_rope: K and V must have the same layout")
    rope_rows = group or M
    _lib.call(_entry, _chk("x", x), _chk("weight_qkv", weight_qkv, (Kdim, (heads + 2) * hd)),
              _chk("rope", rope[:rope_rows], (rope_rows, hd)), _chk("Q", Q, (M * heads, hd)), k_ptr, v_ptr,
              _chk("x_norm", x_norm[:M], (M, Kdim)), M, Kdim, heads, hd, group, pitch, _stream())


def encoder_norm_qkv_rope_fused(x, weight_qkv, rope, Q, K, V, x_norm):
    """The same op with the RMS norm applied to the GEMM's accumulators; `x_norm` is not written (unless the
    shape gives a CTA several tiles, where the library falls back to the two-kernel form)."""
    return encoder_norm_qkv_rope(x, weight_qkv, rope, Q, K, V, x_norm, _entry="fvla_encoder_qkv_rope_fused_norm")


def encoder_attention(Q, K, V, scale, out):
    """Unmasked multi-query attention, Q flat (tokens * heads, hd) (kernels/attention.py:29-34)."""
    queries, hd = Q.shape
    keys = K.shape[0]
    if out.numel() != queries * hd:
        raise ValueError("encoder_attention: out has the wrong size")
    ws, nb = _ws("enc_attn_ws", _lib.load().fvla_encoder_attention_workspace_bytes(queries, keys), Q.device)
    _lib.call("fvla_encoder_attention", _chk("Q", Q), _chk("K", K, (keys, hd)), _chk("V", V, (keys, hd)),
              _chk("out", out), queries, keys, hd, float(scale), ws, nb, _stream())
    return out


def _linear_residual(role, x, weight, out):
    """out += x @ weight. Extension for batches of episodes: 3-D `x` (episodes, rows, K) and `out` (episodes,
    rows, N), contiguous, mean that many independent row groups; with at most 64 rows per group the
    decoder's weight-streaming kernel serves every group inside one launch."""
    group_rows = 0
    if x.ndim == 3:
        if out.ndim != 3 or out.shape[:2] != x.shape[:2]:
            raise ValueError("linear_residual: batched x and out must agree in their leading dimensions")
        group_rows = x.shape[1]
        x, out = x.reshape(-1, x.shape[2]), out.reshape(-1, out.shape[2])
    M, K = x.shape
    N = weight.shape[1]
    lib = _lib.load()
    ws, nb = _ws(role, lib.fvla_gemm_workspace_bytes(M, N, K, 0), x.device)
    _lib.call("fvla_linear_residual", _chk("x", x), _chk("weight", weight, (K, N)),
              _chk("out", out, (M, N), dtype=None), _is_f32("out", out), _shadow_of(out), M, N, K, group_rows, ws, nb,
              _stream())
    return out


def encoder_out_proj_residual(x, weight, out):
    """out += x @ weight (wrappers.py:366-371)."""
    return _linear_residual("enc_o_ws", x, weight, out)


def encoder_norm_gated_ffn(x, gate_w, up_w, out, x_norm):
    """x_norm = rms(x); out = gelu(x_norm @ gate_w) * (x_norm @ up_w) (wrappers.py:374-380)."""
    M, K = x.shape
    N = gate_w.shape[1]
    _lib.call("fvla_encoder_norm_gated_ffn", _chk("x", x), _chk("gate_w", gate_w, (K, N)),
              _chk("up_w", up_w, (K, N)), _chk("out", out[:M], (M, N)), _chk("x_norm", x_norm[:M], (M, K)),
              M, N, K, _stream())
    return out


def encoder_ffn_down_residual(x, weight, out):
    """out += hidden @ weight (wrappers.py:383-392)."""
    return _linear_residual("enc_down_ws", x, weight, out)


# -------------------------------------------------------------------------- decoder
def _small_proj(role, x, weight, bias, out, act):
    K, N = weight.shape
    M = x.numel() // K
    lib = _lib.load()
    ws, nb = _ws(role, lib.fvla_gemm_workspace_bytes(M, N, K, 0) if K > 64 else 0, x.device)
    if out.numel() != M * N:
        raise ValueError(f"{role}: out has the wrong size")
    _lib.call("fvla_decoder_small_proj", _chk("x", x, dtype=None), _is_f32("x", x),
              _chk("weight", weight), _chk("bias", bias, (N,)), _chk("out", out, dtype=None),
              _is_f32("out", out), _shadow_of(out) if K > 64 else None, M, N, K, act, ws, nb, _stream())
    return out


def decoder_state_proj(x, weight, bias, out):
    """out = x @ weight + bias for the single state token (wrappers.py:108-112)."""
    return _small_proj("dec_state_ws", x, weight, bias, out, 0)


def decoder_action_in_proj(x, weight, bias, out):
    """out = silu(x @ weight + bias); x may be the fp32 master copy of the noise (wrappers.py:115-120)."""
    return _small_proj("dec_in_ws", x, weight, bias, out, 2)


def decoder_action_mlp(x, weight, bias, out):
    """out = x @ weight + bias (wrappers.py:123-128)."""
    return _small_proj("dec_mlp_ws", x, weight, bias, out, 0)


def decoder_norm_qkv_rope(x, weight_qkv, rope, Q, K, V, norm_factor):
    """RMS factor, QKV projection, RoPE in fp32, scatter into Q and the KV-cache tail
    (wrappers.py:131-144). `norm_factor[:M]` receives the bf16 factor.

    Extension for batches of episodes: with K and V 3-D views (episodes, D, hd) of the tails of the
    episodes' caches, x holds the episodes' D rows end to end and `rope` is the table of one episode."""
    M, Kdim = x.shape
    hd = V.shape[-1]
    heads = Q.shape[0] // M
    N = (heads + 2) * hd
    lib = _lib.load()
    k_ptr, group, pitch = _kv_destination("K", K, M, hd)
    v_ptr, group_v, pitch_v = _kv_destination("V", V, M, hd)
    if (group, pitch) != (group_v, pitch_v):
        raise ValueError("decoder_norm_qkv_rope: K and V must have the same layout")
    rope_rows = group or M
    ws, nb = _ws("dec_qkv_ws", lib.fvla_gemm_workspace_bytes(M, N, Kdim, 0), x.device)
    _lib.call("fvla_decoder_norm_qkv_rope", _chk("x", x, dtype=None), _is_f32("x", x), _shadow_of(x),
              _chk("weight_qkv", weight_qkv, (Kdim, N)),
              _chk("rope", rope[:rope_rows], (rope_rows, hd)), _chk("Q", Q, (M * heads, hd)), k_ptr, v_ptr,
              _chk("norm_factor", norm_factor[:M], (M,)), M, Kdim, heads, hd, group, pitch,
              ws, nb, _stream())


def decoder_attention(Q, K, V, scores, out, encoder_seq_len):
    """softmax(Q K^T / sqrt(hd)) V with the Pi0 mask, keys split across CTAs. `scores` is
    accepted for signature parity and left untouched, as in the reference's fused wrapper
    (fused_wrappers.py:88-115); `out` may be Q.

    Extension for batches of episodes: K and V as 3-D views (episodes, keys, hd) of the episodes' caches
    (evenly spaced), Q and out holding the episodes' flat query rows end to end."""
    del scores
    lib = _lib.load()
    hd = Q.shape[1]
    if K.ndim == 3:
        episodes, keys = K.shape[0], K.shape[1]
        if K.shape != V.shape or K.stride() != V.stride() or K.stride(2) != 1 or K.stride(1) != hd or K.shape[2] != hd:
            raise ValueError("decoder_attention: batched K / V must be equally laid out (episodes, keys, hd) views")
        if Q.shape[0] % episodes:
            raise ValueError("decoder_attention: Q rows are not a whole number of episodes")
        for name, t in (("K", K), ("V", V)):
            if not t.is_cuda or t.dtype != torch.bfloat16:
                raise ValueError(f"{name}: expected a bf16 CUDA tensor")
        queries = Q.shape[0] // episodes
        k_ptr, v_ptr, kv_stride = K.data_ptr(), V.data_ptr(), K.stride(0)
    else:
        episodes, keys, queries = 1, K.shape[0], Q.shape[0]
        k_ptr, v_ptr, kv_stride = _chk("K", K, (keys, hd)), _chk("V", V, (keys, hd)), 0
    ws, nb = _ws("dec_attn_ws", lib.fvla_decoder_attention_workspace_bytes(queries, keys), Q.device)
    _lib.call("fvla_decoder_attention", _chk("Q", Q), k_ptr, v_ptr,
              _chk("out", out, (queries * episodes, hd)), queries, keys, hd, DECODER_HEADS, int(encoder_seq_len),
              episodes, queries * hd, kv_stride, ws, nb, _stream())
    return out


def decoder_out_proj_residual(x, weight, out):
    """out += x @ weight (wrappers.py:176-181)."""
    return _linear_residual("dec_o_ws", x, weight, out)


def decoder_ffn_down_residual(x, weight, out):
    """out += x @ weight (wrappers.py:184-189)."""
    return _linear_residual("dec_down_ws", x, weight, out)


def _gated_ffn(x, gate_w, up_w, out, norm_factor):
    M, K = x.shape
    N = gate_w.shape[1]
    lib = _lib.load()
    ws, nb = _ws("dec_gate_ws", lib.fvla_gemm_workspace_bytes(M, N, K, 1), x.device)
    nf = None if norm_factor is None else _chk("norm_factor", norm_factor[:M], (M,))
    _lib.call("fvla_decoder_norm_gated_ffn", _chk("x", x, dtype=None), _is_f32("x", x), _shadow_of(x),
              _chk("gate_w", gate_w, (K, N)),
              _chk("up_w", up_w, (K, N)), _chk("out", out, (M, N)), nf, M, N, K, ws, nb, _stream())
    return out


def decoder_norm_gated_ffn(x, gate_w, up_w, out, norm_factor):
    """out = gelu(rms(x) @ gate_w) * (rms(x) @ up_w); stores the factor (wrappers.py:192-198)."""
    return _gated_ffn(x, gate_w, up_w, out, norm_factor)


def _action_out(x, weight, bias, out, norm_factor):
    M, K = x.shape
    N = weight.shape[1]
    nf = None if norm_factor is None else _chk("norm_factor", norm_factor[:M], (M,))
    _lib.call("fvla_decoder_action_out_proj", _chk("x", x, dtype=None), _is_f32("x", x),
              _chk("weight", weight, (K, N)), _chk("bias", bias, (N,)), _chk("out", out, (M, N), dtype=None),
              _is_f32("out", out), None, nf, M, N, K, _stream())
    return out


def decoder_action_out_proj(x, weight, bias, out, norm_factor):
    """out += bias + rms(x) @ weight, the Euler update; stores the factor (wrappers.py:201-208).
    `out` may be bf16 or the fp32 master copy of the noise."""
    return _action_out(x, weight, bias, out, norm_factor)


VISION_WRAPPERS = {f.__name__: f for f in (
    vision_patch_embed, vision_norm_qkv, vision_attention, vision_out_proj_residual,
    vision_norm_ffn_up, vision_ffn_down_residual)}
ENCODER_WRAPPERS = {f.__name__: f for f in (
    encoder_projector, encoder_norm_qkv_rope, encoder_attention, encoder_out_proj_residual,
    encoder_norm_gated_ffn, encoder_ffn_down_residual)}
DECODER_WRAPPERS = {f.__name__: f for f in (
    decoder_state_proj, decoder_action_in_proj, decoder_action_mlp, decoder_norm_qkv_rope,
    decoder_attention, decoder_out_proj_residual, decoder_ffn_down_residual,
    decoder_norm_gated_ffn, decoder_action_out_proj)}

# `sync_shadow` rides in the table so that orchestration code can reach it through `ops`.
ALL_WRAPPERS = {**VISION_WRAPPERS, **ENCODER_WRAPPERS, **DECODER_WRAPPERS, "sync_shadow": sync_shadow,
                "embed_prompt": embed_prompt, "copy_rows": copy_rows}
