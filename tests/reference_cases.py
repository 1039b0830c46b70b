"""Seeded inputs for every call site of the Pi0 op table, shared by three parties with the same positional
signatures: the reference's own TileLang wrappers (run once on a GPU by `tests/golden/make_reference_gpu_golden.py`,
whose strided output samples are the committed fixture `tests/golden/reference_gpu.pt`), the CPU oracle, and this
package's CUDA wrappers (`tests/test_reference_gpu_parity.py` compares both with the fixture).

A case builds its tensors on the CPU from a fixed seed (bf16 values), `run` calls the op on whatever copies of them
it is given (bf16 CUDA tensors for the two GPU back ends, fp32 CPU tensors for the oracle) and returns the tensors the
op wrote. `optional` names outputs that a fused table may leave unwritten (scratch the reference documents as such).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import torch

bf16 = torch.bfloat16


def rnd(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(bf16)


def sample(t: torch.Tensor, limit: int = 4096) -> torch.Tensor:
    """A strided sample of at most `limit` values of a tensor, the same for every party (fp32, 1-D): a stride coprime
    with the usual row lengths, so that it walks across rows, columns and tile edges."""
    flat = t.detach().float().cpu().reshape(-1)
    n = flat.numel()
    if n <= limit:
        return flat.clone()
    stride = n // limit
    if stride % 2 == 0:
        stride += 1
    while stride % 3 == 0 or stride % 5 == 0:
        stride += 2
    return flat[::stride][:limit].clone()


@dataclass
class Case:
    name: str
    inputs: Callable[[], dict]
    run: Callable[..., dict]
    fused_only: bool = False
    optional: tuple = field(default_factory=tuple)


def rope_table(rows: int, first_position: int, head_dim: int = 256) -> torch.Tensor:
    """The reference's RoPE table (buffers.py:15-23): interleaved (cos, sin) per frequency for positions
    first_position .. first_position + rows - 1; the committed fixture tests/golden/rope.pt pins the oracle's copy."""
    from oracle import pi0_ref as O
    return O.rope_table(rows, first_position).to(bf16)


def _vision_patch_embed():
    g = torch.Generator().manual_seed(101)
    return {"img": (torch.rand(3, 224, 224, 3, generator=g) * 2 - 1).to(bf16), "pw": rnd(g, 14, 14, 3, 1152, scale=0.02),
            "pb": rnd(g, 1152, scale=0.02), "pos": rnd(g, 256, 1152, scale=0.02), "out": torch.zeros(3, 256, 1152, dtype=bf16)}


def _vision_norm_linear(N, seed):
    def make():
        g = torch.Generator().manual_seed(seed)
        return {"x": rnd(g, 3, 256, 1152), "nw": rnd(g, 1152, scale=0.5) + 1, "nb": rnd(g, 1152, scale=0.1),
                "w": rnd(g, 1152, N, scale=0.02), "b": rnd(g, N, scale=0.02),
                "out": torch.zeros(3, 256, N, dtype=bf16), "x_norm": torch.zeros(3, 256, 1152, dtype=bf16)}
    return make


def _vision_bias_residual(K, seed):
    def make():
        g = torch.Generator().manual_seed(seed)
        return {"x": rnd(g, 3, 256, K), "w": rnd(g, K, 1152, scale=0.02), "b": rnd(g, 1152, scale=0.02), "res": rnd(g, 3, 256, 1152)}
    return make


def _encoder_projector():
    g = torch.Generator().manual_seed(106)
    return {"x": rnd(g, 3, 256, 1152), "nw": rnd(g, 1152, scale=0.5) + 1, "nb": rnd(g, 1152, scale=0.1),
            "w": rnd(g, 1152, 2048, scale=0.02), "b": rnd(g, 2048, scale=0.02),
            "out": torch.zeros(768, 2048, dtype=bf16), "x_norm": torch.zeros(3, 256, 1152, dtype=bf16)}


def _encoder_qkv():
    g = torch.Generator().manual_seed(107)
    S = 768
    return {"x": rnd(g, S, 2048), "w": rnd(g, 2048, 2560, scale=0.02), "rope": rope_table(S, 0),
            "Q": torch.zeros(S * 8, 256, dtype=bf16), "K": torch.zeros(S, 256, dtype=bf16), "V": torch.zeros(S, 256, dtype=bf16),
            "x_norm": torch.zeros(S, 2048, dtype=bf16)}


def _linear_residual(M, K, N, seed):
    def make():
        g = torch.Generator().manual_seed(seed)
        return {"x": rnd(g, M, K), "w": rnd(g, K, N, scale=0.02), "out": rnd(g, M, N)}
    return make


def _encoder_gated():
    g = torch.Generator().manual_seed(109)
    return {"x": rnd(g, 768, 2048), "wg": rnd(g, 2048, 16384, scale=0.02), "wu": rnd(g, 2048, 16384, scale=0.02),
            "out": torch.zeros(768, 16384, dtype=bf16), "x_norm": torch.zeros(768, 2048, dtype=bf16)}


def _decoder_small(M, K, seed):
    def make():
        g = torch.Generator().manual_seed(seed)
        return {"x": rnd(g, M, K) if M > 1 else rnd(g, K), "w": rnd(g, K, 1024, scale=0.02), "b": rnd(g, 1024, scale=0.02),
                "out": torch.zeros(M, 1024, dtype=bf16)}
    return make


def _decoder_qkv():
    g = torch.Generator().manual_seed(113)
    M, S = 51, 768
    return {"x": rnd(g, M, 1024, scale=3.0), "w": rnd(g, 1024, 2560, scale=0.02), "rope": rope_table(M, S),
            "Q": torch.zeros(M * 8, 256, dtype=bf16), "K": torch.zeros(M, 256, dtype=bf16), "V": torch.zeros(M, 256, dtype=bf16),
            "factor": torch.zeros(M, dtype=bf16)}


def _decoder_attention():
    g = torch.Generator().manual_seed(114)
    S, keys = 768, 819
    return {"Q": rnd(g, 408, 256), "K": rnd(g, keys, 256), "V": rnd(g, keys, 256), "scores": torch.zeros(408, keys, dtype=bf16),
            "out": torch.zeros(408, 256, dtype=bf16), "S": S}


def _decoder_gated():
    g = torch.Generator().manual_seed(115)
    return {"x": rnd(g, 51, 1024, scale=3.0), "wg": rnd(g, 1024, 4096, scale=0.02), "wu": rnd(g, 1024, 4096, scale=0.02),
            "out": torch.zeros(51, 4096, dtype=bf16), "factor": torch.zeros(51, dtype=bf16)}


def _decoder_action_out():
    g = torch.Generator().manual_seed(116)
    return {"x": rnd(g, 50, 1024, scale=3.0), "w": rnd(g, 1024, 32, scale=0.02), "b": rnd(g, 32, scale=0.02),
            "out": rnd(g, 50, 32), "factor": torch.zeros(50, dtype=bf16)}


CASES = [
    Case("vision_patch_embed", _vision_patch_embed,
         lambda ops, t, **kw: (ops.vision_patch_embed(t["img"], t["pw"], t["pb"], t["pos"], t["out"]), {"out": t["out"]})[1]),
    Case("vision_norm_qkv", _vision_norm_linear(3456, 102),
         lambda ops, t, **kw: (ops.vision_norm_qkv(t["x"], t["nw"], t["nb"], t["w"], t["b"], t["out"], t["x_norm"]),
                               {"out": t["out"], "x_norm": t["x_norm"]})[1], optional=("x_norm",)),
    Case("vision_out_proj_residual", _vision_bias_residual(1152, 103),
         lambda ops, t, **kw: (ops.vision_out_proj_residual(t["x"], t["w"], t["b"], t["res"], t["res"]), {"out": t["res"]})[1]),
    Case("vision_norm_ffn_up", _vision_norm_linear(4304, 104),
         lambda ops, t, **kw: (ops.vision_norm_ffn_up(t["x"], t["nw"], t["nb"], t["w"], t["b"], t["out"], t["x_norm"]),
                               {"out": t["out"], "x_norm": t["x_norm"]})[1], optional=("x_norm",)),
    Case("vision_ffn_down_residual", _vision_bias_residual(4304, 105),
         lambda ops, t, **kw: (ops.vision_ffn_down_residual(t["x"], t["w"], t["b"], t["res"], t["res"]), {"out": t["res"]})[1]),
    Case("encoder_projector", _encoder_projector,
         lambda ops, t, **kw: (ops.encoder_projector(t["x"], t["nw"], t["nb"], t["w"], t["b"], t["out"], t["x_norm"]),
                               {"out": t["out"], "x_norm": t["x_norm"]})[1]),
    Case("encoder_norm_qkv_rope", _encoder_qkv,
         lambda ops, t, **kw: (ops.encoder_norm_qkv_rope(t["x"], t["w"], t["rope"], t["Q"], t["K"], t["V"], t["x_norm"]),
                               {"Q": t["Q"], "K": t["K"], "V": t["V"], "x_norm": t["x_norm"]})[1], optional=("x_norm",)),
    Case("encoder_out_proj_residual", _linear_residual(768, 2048, 2048, 108),
         lambda ops, t, **kw: (ops.encoder_out_proj_residual(t["x"], t["w"], t["out"]), {"out": t["out"]})[1]),
    Case("encoder_norm_gated_ffn", _encoder_gated,
         lambda ops, t, **kw: (ops.encoder_norm_gated_ffn(t["x"], t["wg"], t["wu"], t["out"], t["x_norm"]),
                               {"out": t["out"], "x_norm": t["x_norm"]})[1]),
    Case("encoder_ffn_down_residual", _linear_residual(768, 16384, 2048, 110),
         lambda ops, t, **kw: (ops.encoder_ffn_down_residual(t["x"], t["w"], t["out"]), {"out": t["out"]})[1]),
    Case("decoder_state_proj", _decoder_small(1, 32, 111),
         lambda ops, t, **kw: (ops.decoder_state_proj(t["x"], t["w"], t["b"], t["out"]), {"out": t["out"]})[1]),
    Case("decoder_action_in_proj", _decoder_small(50, 32, 112),
         lambda ops, t, **kw: (ops.decoder_action_in_proj(t["x"], t["w"], t["b"], t["out"]), {"out": t["out"]})[1]),
    Case("decoder_action_mlp", _decoder_small(50, 1024, 117),
         lambda ops, t, **kw: (ops.decoder_action_mlp(t["x"], t["w"], t["b"], t["out"]), {"out": t["out"]})[1]),
    Case("decoder_norm_qkv_rope", _decoder_qkv,
         lambda ops, t, **kw: (ops.decoder_norm_qkv_rope(t["x"], t["w"], t["rope"], t["Q"], t["K"], t["V"], t["factor"]),
                               {"Q": t["Q"], "K": t["K"], "V": t["V"], "factor": t["factor"]})[1]),
    Case("decoder_attention", _decoder_attention,
         lambda ops, t, **kw: (ops.decoder_attention(t["Q"], t["K"], t["V"], t["scores"], t["out"], t["S"]), {"out": t["out"]})[1]),
    Case("decoder_out_proj_residual", _linear_residual(51, 2048, 1024, 118),
         lambda ops, t, **kw: (ops.decoder_out_proj_residual(t["x"], t["w"], t["out"]), {"out": t["out"]})[1]),
    Case("decoder_norm_gated_ffn", _decoder_gated,
         lambda ops, t, **kw: (ops.decoder_norm_gated_ffn(t["x"], t["wg"], t["wu"], t["out"], t["factor"]), {"out": t["out"]})[1]),
    Case("decoder_ffn_down_residual", _linear_residual(51, 4096, 1024, 119),
         lambda ops, t, **kw: (ops.decoder_ffn_down_residual(t["x"], t["w"], t["out"]), {"out": t["out"]})[1]),
    Case("decoder_action_out_proj", _decoder_action_out,
         lambda ops, t, **kw: (ops.decoder_action_out_proj(t["x"], t["w"], t["b"], t["out"], t["factor"]), {"out": t["out"]})[1]),
]
