"""Host-side logic that needs no GPU: schema, op table, scratch pool, buffer plan, the package
pipeline driven by the oracle's ops, and the C-ABI library's exported symbols."""
from __future__ import annotations

import ctypes
import re

import pytest
import torch

from conftest import ROOT
from oracle import pi0_ref as O


def test_weight_schema():
    from flash_vla_b200.models.pi0 import weight_shapes
    shapes = weight_shapes(48)
    assert len(shapes) == 38
    assert shapes["language_embeds"] == (48, 2048)
    assert shapes["vision_ffn_up_w"] == (27, 1152, 4304)
    assert shapes["decoder_attn_qkv_w"] == (18, 1024, 2560)
    total = sum(torch.Size(s).numel() for s in weight_shapes(0).values())
    assert abs(total - 2.709e9) < 2e6
    assert list(shapes)[0] == "vision_patch_embedding_w" and list(shapes)[-1] == "language_embeds"


def test_random_checkpoint_is_deterministic_and_filterable(decoder_checkpoint):
    from flash_vla_b200.models.pi0 import random_checkpoint
    a = random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cpu", only=("decoder_action", "decoder_state"))
    b = decoder_checkpoint                # an earlier draw of the same stream with a wider filter
    assert set(a) == {"decoder_state_in_proj_w", "decoder_state_in_proj_b", "decoder_action_fused_in_proj_w",
                      "decoder_action_fused_time_biases", "decoder_action_mlp_w", "decoder_action_mlp_b",
                      "decoder_action_fused_out_proj_w", "decoder_action_fused_out_proj_b"}
    assert all(torch.equal(a[k], b[k]) and a[k].dtype == torch.bfloat16 for k in a)
    assert 0.015 < a["decoder_action_mlp_w"].float().std().item() < 0.025


def test_op_table_contract():
    from flash_vla_b200 import op_table
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends import BACKENDS, DEFAULT_FUSED_OPS
    from flash_vla_b200.hardware.nvidia.b200.pi0.ops import op_names
    cuda = BACKENDS["cuda"]
    reference_names = {
        "vision_patch_embed", "vision_norm_qkv", "vision_out_proj_residual", "vision_norm_ffn_up",
        "vision_ffn_down_residual", "encoder_projector", "encoder_norm_qkv_rope", "encoder_out_proj_residual",
        "encoder_norm_gated_ffn", "encoder_ffn_down_residual", "decoder_state_proj", "decoder_action_in_proj",
        "decoder_action_mlp", "decoder_norm_qkv_rope", "decoder_attention", "decoder_out_proj_residual",
        "decoder_ffn_down_residual", "decoder_norm_gated_ffn", "decoder_action_out_proj"}
    assert reference_names <= set(cuda.ALL_WRAPPERS)
    assert set(cuda.ALL_WRAPPERS) - reference_names == {"vision_attention", "encoder_attention", "sync_shadow", "embed_prompt", "copy_rows"}
    # the reference's three fused decoder ops, plus three prefix ops whose row norm this backend folds into the GEMM
    reference_fused = {"decoder_norm_gated_ffn", "decoder_action_out_proj", "decoder_attention"}
    assert set(DEFAULT_FUSED_OPS) == reference_fused | {"vision_norm_qkv", "vision_norm_ffn_up", "encoder_norm_qkv_rope"}
    fused, unfused = op_table(True), op_table(False)
    assert fused.decoder_attention is cuda.FUSED_WRAPPERS["decoder_attention"]
    assert unfused.decoder_attention is cuda.ALL_WRAPPERS["decoder_attention"]
    assert fused.vision_norm_qkv is not unfused.vision_norm_qkv
    assert fused.vision_patch_embed is unfused.vision_patch_embed
    planned = op_table(True, plan={"decoder_attention": "cuda"})
    assert set(vars(planned)) == set(op_names(True))
    with pytest.raises(KeyError):
        op_table(True, plan={"decoder_attention": "tilelang"})
    # signatures are positional and match the oracle's (which follow the reference's wrappers)
    import inspect
    for name in reference_names:
        want = list(inspect.signature(getattr(O.op_table(True), name)).parameters)
        got = list(inspect.signature(getattr(fused, name)).parameters)
        assert got == want, name


def test_scratch_pool_freeze():
    from flash_vla_b200.runtime.cuda import ScratchPool
    pool = ScratchPool()
    a = pool.get("partials", (3, 4), torch.float32, "cpu")
    assert a.abs().sum() == 0 and pool.get("partials", (3, 4), torch.float32, "cpu") is a
    assert pool.get("partials", (3, 5), torch.float32, "cpu") is not a and len(pool) == 2
    pool.freeze()
    assert pool.get("partials", (3, 4), torch.float32, "cpu") is a
    with pytest.raises(RuntimeError, match="frozen"):
        pool.get("partials", (9,), torch.float32, "cpu")


def test_buffer_plan():
    from flash_vla_b200.hardware.nvidia.b200.pi0.buffers import allocate_static_buffers, rope_table
    b, S = allocate_static_buffers(3, 50, 49, "cpu")
    assert S == 817
    assert b["encoder_K"].shape == (18, 868, 256) and b["encoder_Q"].shape == (817 * 8, 256)
    assert b["decoder_attn_buf"].shape == (408, 868) and b["decoder_q_buf"].shape == (408, 256)
    assert b["diffusion_noise"].dtype == torch.bfloat16 and b["diffusion_noise_f32"].dtype == torch.float32
    assert b["decoder_x"].dtype == torch.float32
    assert torch.equal(b["decoder_rope_weights"], O.rope_table(51, 817))
    assert torch.equal(rope_table(13, 5, 256, "cpu"), O.rope_table(13, 5))


def test_batched_buffer_plan():
    from flash_vla_b200.hardware.nvidia.b200.pi0.buffers import allocate_batched_buffers
    prefix, episodes, S = allocate_batched_buffers(3, 50, 49, 2, "cpu")
    assert S == 817 and len(episodes) == 2
    assert prefix["vision_x"].shape == (6, 256, 1152) and prefix["encoder_x"].shape == (2 * 817, 2048)
    assert prefix["encoder_K"].shape == (2, 18, 868, 256) and prefix["encoder_rope_weights"].shape == (817, 256)
    for e, b in enumerate(episodes):
        assert b["encoder_K"].shape == (18, 868, 256) and b["encoder_K"].data_ptr() == prefix["encoder_K"][e].data_ptr()
        assert b["observation_images_normalized"].shape == (3, 224, 224, 3)
        assert b["decoder_x"].dtype == torch.float32 and "vision_x" not in b
        assert torch.equal(b["decoder_rope_weights"], O.rope_table(51, 817))
    # the K / V destination the batched QKV projection gets: evenly spaced (episodes, S, 256) blocks
    k = prefix["encoder_K"][:, 3, :S]
    assert k.shape == (2, 817, 256) and k.stride() == (18 * 868 * 256, 256, 1)


def test_package_pipeline_with_oracle_ops(monkeypatch):
    """The package's orchestration, driven by the oracle's op table on the CPU, must equal the
    oracle's own orchestration (which make_golden checks against the reference's pipeline.py).
    Layer counts are cut to 2 to keep this fast; stacked weights are drawn directly."""
    from flash_vla_b200.hardware.nvidia.b200.pi0 import pipeline
    from flash_vla_b200.models.pi0.spec import weight_shapes
    L = 2
    monkeypatch.setattr(pipeline, "VISION_LAYERS", L)
    monkeypatch.setattr(pipeline, "ENCODER_LAYERS", L)
    monkeypatch.setattr(O, "VISION_LAYERS", L)
    monkeypatch.setattr(O, "ENCODER_LAYERS", L)
    g = torch.Generator().manual_seed(0)
    w = {}
    for name, shape in weight_shapes(5).items():
        shape = tuple(L if (i == 0 and s in (27, 18) and len(shape) > 1 and name != "decoder_action_fused_time_biases") else s
                      for i, s in enumerate(shape))
        w[name] = torch.randn(shape, generator=g) * 0.02
    images = torch.rand(3, 224, 224, 3, generator=g) * 2 - 1
    state, noise = torch.randn(32, generator=g), torch.randn(50, 32, generator=g)

    want, ref_buffers = O.forward(w, images, state, noise, steps=3, layers=L)
    want = want.clone()

    b, S = O.allocate_buffers(3, 50, 5)
    b["diffusion_noise_f32"] = torch.zeros(50, 32)
    ops = O.op_table(True)
    b["observation_images_normalized"].copy_(images)
    b["observation_state_normalized"].copy_(state)
    b["diffusion_noise"].copy_(noise)
    b["encoder_x"][768:].copy_(w["language_embeds"])
    pipeline.vision_encoder(ops, w, b, 3)
    pipeline.transformer_encoder(ops, w, b, S)
    pipeline.transformer_decoder(ops, w, b, S, steps=3, layers=L)
    assert torch.allclose(b["diffusion_noise"], want, atol=1e-5)
    assert torch.allclose(b["encoder_K"][:L], ref_buffers["encoder_K"][:L], atol=1e-5)
    with pytest.raises(NotImplementedError):
        pipeline.vision_encoder(ops, w, b, 2)


def test_batched_prefix_pipeline_equals_independent_episodes(monkeypatch):
    """The throughput plan's orchestration (SigLIP and the prefix encoder once over all episodes' rows,
    K/V scattered into per-episode caches, decoders per episode) driven by the oracle's ops on the CPU must
    give, for every episode, what an independent single-episode pass gives."""
    from types import SimpleNamespace
    from flash_vla_b200.hardware.nvidia.b200.pi0 import pipeline
    from flash_vla_b200.models.pi0.spec import weight_shapes
    L, E, P = 2, 2, 5
    monkeypatch.setattr(pipeline, "VISION_LAYERS", L)
    monkeypatch.setattr(pipeline, "ENCODER_LAYERS", L)
    monkeypatch.setattr(O, "VISION_LAYERS", L)
    monkeypatch.setattr(O, "ENCODER_LAYERS", L)
    g = torch.Generator().manual_seed(1)
    w = {}
    for name, shape in weight_shapes(P).items():
        shape = tuple(L if (i == 0 and s in (27, 18) and len(shape) > 1 and name != "decoder_action_fused_time_biases") else s
                      for i, s in enumerate(shape))
        w[name] = torch.randn(shape, generator=g) * 0.02
    inputs = [(torch.rand(3, 224, 224, 3, generator=g) * 2 - 1, torch.randn(32, generator=g), torch.randn(50, 32, generator=g))
              for _ in range(E)]
    want = [O.forward(w, *inp, steps=2, layers=L)[0].clone() for inp in inputs]

    # the oracle's QKV op writes (M, hd) K / V; the batched plan hands it (episodes, S, hd) views of the caches
    base = O.op_table(True)

    def qkv(x, weight, rope, Q, K, V, x_norm):
        if K.ndim == 2:
            return base.encoder_norm_qkv_rope(x, weight, rope, Q, K, V, x_norm)
        n, S = K.shape[0], K.shape[1]
        for e in range(n):                      # rope is one sequence's table: apply per sequence
            rows = slice(e * S, (e + 1) * S)
            base.encoder_norm_qkv_rope(x[rows], weight, rope, Q[e * S * 8:(e + 1) * S * 8], K[e], V[e], x_norm[rows])

    ops = SimpleNamespace(**{**vars(base), "encoder_norm_qkv_rope": qkv})
    S, D = 768 + P, 51
    ref_b, _ = O.allocate_buffers(3, 50, P)
    prefix = {k: (torch.zeros((E * v.shape[0],) + tuple(v.shape[1:])) if k.startswith(("vision_", "observation_images"))
                  or k in ("encoder_x", "encoder_x_norm", "encoder_Q", "encoder_attn", "encoder_hidden") else v)
              for k, v in ref_b.items()}
    prefix["encoder_K"] = torch.zeros(E, L, S + D, 256)
    prefix["encoder_V"] = torch.zeros(E, L, S + D, 256)
    episodes = []
    for e, (images, state, noise) in enumerate(inputs):
        b, _ = O.allocate_buffers(3, 50, P)
        b["diffusion_noise_f32"] = torch.zeros(50, 32)
        b["observation_state_normalized"].copy_(state)
        b["diffusion_noise"].copy_(noise)
        b["encoder_K"], b["encoder_V"] = prefix["encoder_K"][e], prefix["encoder_V"][e]
        prefix["observation_images_normalized"][3 * e:3 * e + 3].copy_(images)
        prefix["encoder_x"][e * S + 768:(e + 1) * S].copy_(w["language_embeds"])
        episodes.append(b)
    pipeline.vision_encoder(ops, w, prefix, 3)
    seen = []
    pipeline.transformer_encoder_batched(ops, w, prefix, S, 3, E, after_qkv=seen.append)
    assert seen == list(range(L))
    for e, b in enumerate(episodes):
        pipeline.transformer_decoder(ops, w, b, S, steps=2, layers=L)
        assert torch.allclose(b["diffusion_noise"], want[e], atol=1e-5), f"episode {e}"

    # the decoder batched as well: one pass over all episodes' rows, K / V in the per-episode caches
    def dec_qkv(x, weight, rope, Q, K, V, nf):
        if K.ndim == 2:
            return base.decoder_norm_qkv_rope(x, weight, rope, Q, K, V, nf)
        n, Dr = K.shape[0], K.shape[1]
        for e in range(n):
            rows = slice(e * Dr, (e + 1) * Dr)
            base.decoder_norm_qkv_rope(x[rows], weight, rope, Q[e * Dr * 8:(e + 1) * Dr * 8], K[e], V[e], nf[rows])

    def dec_attn(Q, K, V, scores, out, S_):
        if K.ndim == 2:
            return base.decoder_attention(Q, K, V, scores, out, S_)
        n = K.shape[0]
        per = Q.shape[0] // n
        for e in range(n):
            rows = slice(e * per, (e + 1) * per)
            base.decoder_attention(Q[rows], K[e], V[e], torch.zeros(per, K.shape[1]), out[rows], S_)

    def state_proj(x, weight, bias, out):           # the oracle's form takes one state vector
        for e in range(x.shape[0]):
            base.decoder_state_proj(x[e], weight, bias, out[e:e + 1])

    ops2 = SimpleNamespace(**{**vars(ops), "decoder_norm_qkv_rope": dec_qkv, "decoder_attention": dec_attn,
                              "decoder_state_proj": state_proj})
    dec = {"observation_state_normalized": torch.stack([i[1] for i in inputs]),
           "diffusion_noise": torch.stack([i[2] for i in inputs]).clone(),
           "diffusion_noise_f32": torch.zeros(E * 50, 32), "decoder_rope_weights": ref_b["decoder_rope_weights"],
           "decoder_x": torch.zeros(E * D, 1024), "decoder_x_buf": torch.zeros(E * 50, 1024),
           "decoder_mlp_out": torch.zeros(E * 50, 1024), "decoder_x_rows": torch.zeros(E * 50, 1024),
           "decoder_state_buf": torch.zeros(E, 1024), "decoder_norm_factor_buf": torch.zeros(E * D),
           "decoder_q_buf": torch.zeros(E * D * 8, 256), "decoder_hidden": torch.zeros(E * D, 4096)}
    prefix["encoder_K"][:, :, S:] = 0
    prefix["encoder_V"][:, :, S:] = 0
    pipeline.decoder_prologue_batched(ops2, w, dec)
    for step in range(2):
        pipeline.decoder_step_batched(ops2, w, prefix, dec, S, step, E, layers=L)
    pipeline.decoder_epilogue_batched(dec)
    for e in range(E):
        assert torch.allclose(dec["diffusion_noise"][e], want[e], atol=1e-5), f"batched decoder, episode {e}"


def test_engine_refuses_to_run_without_cuda():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from flash_vla_b200 import Pi0Inference
    with pytest.raises(RuntimeError, match="CUDA"):
        Pi0Inference({"language_embeds": torch.zeros(0, 2048)}, num_views=3, chunk_size=50)


def declared_symbols():
    text = (ROOT / "include" / "flash_vla_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fvla_\w+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    from flash_vla_b200 import build
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib
    path = build.build()
    lib = ctypes.CDLL(str(path))
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), name
    assert set(_lib.SIGNATURES) | set(_lib.QUERIES) == set(names)
    loaded = _lib.load()
    assert loaded.fvla_abi_version() >= 1
    # pure host queries: sizes grow with the problem and are zero for empty problems
    assert loaded.fvla_gemm_workspace_bytes(0, 8, 8, 0) == 0
    assert loaded.fvla_gemm_workspace_bytes(51, 4096, 1024, 1) > loaded.fvla_gemm_workspace_bytes(51, 4096, 1024, 0) > 0
    assert loaded.fvla_decoder_attention_workspace_bytes(408, 868) >= 7 * 448 * 256 * 4
    assert loaded.fvla_patch_embed_workspace_bytes(3) == 3 * 256 * 592 * 2


def test_header_argument_counts_match_ctypes_table():
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib
    text = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "flash_vla_b200.h").read_text(), flags=re.S)
    for name, argtypes in {**_lib.SIGNATURES, **{k: v[0] for k, v in _lib.QUERIES.items()}}.items():
        m = re.search(rf"\b{name}\s*\((.*?)\)\s*;", text, flags=re.S)
        assert m, name
        args = m.group(1).strip()
        count = 0 if args in ("", "void") else args.count(",") + 1
        assert count == len(argtypes), f"{name}: header has {count} parameters, ctypes table {len(argtypes)}"


def test_graft_entry_build_passes():
    """The entry point the build check runs: compiles (or finds the up-to-date library), verifies that every
    declared symbol is exported and that the op table holds the reference's 19 call sites plus the extensions."""
    import importlib
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parents[1])
    if root not in sys.path:
        sys.path.insert(0, root)
    entry = importlib.import_module("__graft_entry__")
    entry.build()


def test_pinned_plan_table_validates_on_the_host():
    """fvla_gemm_plan_set accepts only (kind, engine, tile width, split) combinations that exist; the table
    is process-wide, replaceable and clearable. Pure host logic: no launch is made."""
    from flash_vla_b200.hardware.nvidia.b200.pi0 import autotune
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib
    lib = _lib.load()
    K, E = autotune.KIND, autotune.ENGINE
    assert lib.fvla_gemm_plan_clear() == 0 and lib.fvla_gemm_plan_count() == 0
    assert lib.fvla_gemm_plan_set(768, 1152, 4304, K["plain"], E["tc5_scratch"], 192, 2) == 0
    assert lib.fvla_gemm_plan_set(768, 1152, 4304, K["plain"], E["tc5_cluster"], 128, 3) == 0      # replaces, not adds
    assert lib.fvla_gemm_plan_count() == 1
    assert lib.fvla_gemm_plan_set(51, 4096, 1024, K["skinny_dual"], E["skinny"], 128, 2) == 0
    assert lib.fvla_gemm_plan_count() == 2
    for bad in ((768, 1152, 4304, K["plain"], E["tc5_scratch"], 160, 2),      # no such tile width
                (768, 1152, 4304, K["plain"], E["tc5_cluster"], 128, 5),      # clusters split K at most 4 ways
                (768, 1152, 4304, K["rope"], E["pair"], 256, 1),              # the RoPE epilogue has one kernel only
                (51, 4096, 1024, K["skinny"], E["skinny"], 128, 3),           # cluster sizes are powers of two
                (0, 1152, 4304, K["plain"], E["pair"], 256, 1)):
        assert lib.fvla_gemm_plan_set(*bad) == -1, bad
        assert b"gemm_plan_set" in lib.fvla_last_error()
    assert lib.fvla_gemm_plan_count() == 2
    assert lib.fvla_gemm_plan_clear() == 0 and lib.fvla_gemm_plan_count() == 0
    # the sweep's candidate lists only name plans the table accepts
    for site in autotune.SITES.values():
        for cand in autotune.candidates(site):
            assert lib.fvla_gemm_plan_set(*site.key(), E[cand["engine"]], cand["bn"], cand["splits"]) == 0, (site.name, cand)
    lib.fvla_gemm_plan_clear()
    assert autotune.grid(bn=[128, 256], splits=[1, 2]) == [{"bn": 128, "splits": 1}, {"bn": 128, "splits": 2},
                                                            {"bn": 256, "splits": 1}, {"bn": 256, "splits": 2}]
