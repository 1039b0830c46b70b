"""The oracle against independent torch expressions and against the committed fixtures that
were produced by the reference's own CPU-runnable code (tests/golden/make_golden.py)."""
from __future__ import annotations

import hashlib
import json
import math

import pytest
import torch
import torch.nn.functional as F

from conftest import GOLDEN
from oracle import pi0_ref as O

bf16 = torch.bfloat16


def test_gelu_silu_forms():
    v = torch.linspace(-8, 8, 4001)
    assert torch.allclose(O.gelu(v), F.gelu(v, approximate="tanh"), atol=2e-6)
    assert torch.allclose(O.silu(v), F.silu(v), atol=1e-6)


def test_layer_norm_and_rms():
    g = torch.Generator().manual_seed(0)
    x, w, b = torch.randn(7, 1152, generator=g), torch.randn(1152, generator=g), torch.randn(1152, generator=g)
    assert torch.allclose(O.layer_norm(x, w, b), F.layer_norm(x, (1152,), w, b, eps=1e-5), atol=1e-5)
    f = O.rms_factor(x)
    assert torch.allclose(f, 1.0 / torch.sqrt(x.pow(2).mean(-1) + 1e-6))


def test_layer_norm_folded_into_the_linear_layer_is_the_same_function():
    """The algebra behind the CUDA backend's fused LayerNorm + linear ops, checked against the oracle's own op
    (the reference's two-kernel form, wrappers.py:268-276) in fp64: with W' = diag(g) W, colsum = 1^T W' and
    bias' = s^T W + b,  LN(x) W + b  ==  rstd * (x W' - mean * colsum) + bias',  also for rows whose mean is many
    times their spread. And the RMS form: (x * rstd) W == rstd * (x W)."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(16, 1152, generator=g, dtype=torch.float64)
    x[:4] += 6.0
    gam, sh = torch.randn(1152, generator=g, dtype=torch.float64) * 0.5 + 1, torch.randn(1152, generator=g, dtype=torch.float64) * 0.1
    W, b = torch.randn(1152, 96, generator=g, dtype=torch.float64) * 0.02, torch.randn(96, generator=g, dtype=torch.float64) * 0.02
    ref = O.layer_norm(x.float(), gam.float(), sh.float()).double() @ W + b          # the oracle keeps fp32 inside the norm
    mean = x.mean(-1, keepdim=True)
    rstd = torch.rsqrt((x * x).mean(-1, keepdim=True) - mean * mean + 1e-5)
    Wf = gam[:, None] * W
    folded = rstd * (x @ Wf - mean * Wf.sum(0)) + (sh @ W + b)
    assert (folded - ref).abs().max().item() <= 2e-5 * ref.abs().max().item()
    r = O.rms_factor(x.float()).double()[:, None]
    assert torch.allclose((x * r) @ W, r * (x @ W), rtol=1e-12, atol=1e-12)


def test_rope_table_matches_reference_fixture():
    gold = torch.load(GOLDEN / "rope.pt")
    for S in (768, 816, 817):
        assert torch.equal(O.rope_table(51, S), gold[S])
    for S in (768, 817):
        assert torch.equal(O.rope_table(S, 0)[::37], gold[f"enc{S}"])


def test_rotation_is_complex_multiplication():
    """Adjacent pairs (2p, 2p+1) rotate as (x0 + i x1) * (cos + i sin)."""
    g = torch.Generator().manual_seed(1)
    M, heads, hd = 5, 8, 256
    proj = torch.randn(M, (heads + 2) * hd, generator=g)
    rope = O.rope_table(M, 768).float()
    Q, K, V = torch.zeros(M * heads, hd), torch.zeros(M, hd), torch.zeros(M, hd)
    O._rotate_scatter(proj, rope, Q, K, V)
    z = torch.view_as_complex(proj[:, :(heads + 1) * hd].reshape(M, heads + 1, hd // 2, 2).contiguous())
    r = torch.view_as_complex(rope.reshape(M, 1, hd // 2, 2).contiguous())
    want = torch.view_as_real(z * r).reshape(M, heads + 1, hd)
    assert torch.allclose(Q.view(M, heads, hd), want[:, :heads], atol=1e-6)
    assert torch.allclose(K, want[:, heads], atol=1e-6)
    assert torch.equal(V, proj[:, (heads + 1) * hd:])


def test_attention_matches_reference_torch_functions():
    """Outputs of the reference's own vision_attention / encoder_attention, stored by make_golden."""
    gold = torch.load(GOLDEN / "attention.pt")
    g = torch.Generator().manual_seed(gold["qkv_seed"])
    qkv = torch.randn(1, 256, 3456, generator=g)
    Q, K, V = torch.randn(64 * 8, 256, generator=g), torch.randn(300, 256, generator=g), torch.randn(300, 256, generator=g)
    ops = O.op_table()
    assert torch.allclose(ops.vision_attention(qkv)[:, ::8], gold["vision_out"], atol=2e-5)
    assert torch.allclose(ops.encoder_attention(Q, K, V, 256 ** -0.5), gold["encoder_out"], atol=2e-5)


@pytest.mark.parametrize("S", [768, 817])
@pytest.mark.parametrize("fused", [False, True])
def test_decoder_attention_mask_against_sdpa(S, fused):
    g = torch.Generator().manual_seed(2)
    keys = S + 51
    Q, K, V = torch.randn(408, 256, generator=g), torch.randn(keys, 256, generator=g), torch.randn(keys, 256, generator=g)
    out, scores = torch.zeros(408, 256), torch.zeros(408, keys)
    O.op_table(fused).decoder_attention(Q, K, V, scores, out, S)
    mask = torch.ones(408, keys, dtype=torch.bool)
    mask[:8, S + 1:] = False                       # the state token sees the prefix and itself only
    want = F.scaled_dot_product_attention(Q[None], K[None], V[None], attn_mask=mask[None])[0]
    assert torch.allclose(out, want, atol=2e-5)
    if not fused:
        assert torch.allclose(scores.sum(-1), torch.ones(408), atol=1e-5)
        assert (scores[:8, S + 1:] == 0).all()


def test_patch_embed_is_a_strided_convolution():
    g = torch.Generator().manual_seed(3)
    img = torch.rand(2, 224, 224, 3, generator=g)
    w, b, pos = torch.randn(14, 14, 3, 1152, generator=g) * 0.02, torch.randn(1152, generator=g), torch.randn(256, 1152, generator=g)
    out = torch.zeros(2, 256, 1152)
    O.op_table().vision_patch_embed(img, w, b, pos, out)
    conv = F.conv2d(img.permute(0, 3, 1, 2), w.permute(3, 2, 0, 1), b, stride=14)       # (2,1152,16,16)
    want = conv.flatten(2).transpose(1, 2) + pos
    assert torch.allclose(out, want, atol=2e-4)


def test_fused_and_unfused_tables_agree_in_fp32():
    g = torch.Generator().manual_seed(4)
    x, wg, wu = torch.randn(51, 1024, generator=g), torch.randn(1024, 4096, generator=g) * .02, torch.randn(1024, 4096, generator=g) * .02
    a, b = torch.zeros(51, 4096), torch.zeros(51, 4096)
    nf = torch.zeros(51)
    O.op_table(False).decoder_norm_gated_ffn(x, wg, wu, a, nf)
    O.op_table(True).decoder_norm_gated_ffn(x, wg, wu, b, torch.zeros(51))
    assert torch.allclose(a, b, atol=1e-5)
    assert torch.allclose(nf, O.rms_factor(x))


def test_bf16_faithful_mode_rounds_where_the_reference_does():
    g = torch.Generator().manual_seed(5)
    x, w = torch.randn(16, 2048, generator=g).to(bf16), (torch.randn(2048, 2560, generator=g) * .02).to(bf16)
    rope = O.rope_table(16, 0)
    outs = []
    for faithful in (False, True):
        Q, K, V, xn = torch.zeros(128, 256), torch.zeros(16, 256), torch.zeros(16, 256), torch.zeros(16, 2048)
        O.op_table(False, faithful).encoder_norm_qkv_rope(x, w, rope, Q, K, V, xn)
        outs.append((Q, V))
    # V is copied without rotation: in faithful mode it must be exactly bf16-representable
    assert torch.equal(outs[1][1], outs[1][1].to(bf16).float())
    assert not torch.equal(outs[0][1], outs[0][1].to(bf16).float())
    assert (outs[0][0] - outs[1][0]).abs().max() < 0.05


def test_checkpoint_generator_reproduces_reference_hashes(decoder_checkpoint):
    """SHA-256 of tensors drawn by the reference's random_checkpoint (stored by make_golden)."""
    gold = json.loads((GOLDEN / "checkpoint.json").read_text())
    assert gold["args"] == {"prompt_len": 0, "wscale": 0.02, "seed": 0, "device": "cpu"}
    ck = decoder_checkpoint
    checked = 0
    for name, digest in gold["sha256"].items():
        if name in ck:
            got = hashlib.sha256(ck[name].contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()
            assert got == digest, name
            checked += 1
    assert checked >= 6


def _decoder_step(w32, kv_scale, ops):
    from flash_vla_b200.synthetic import decoder_step_inputs
    K, V, st, nz = decoder_step_inputs(kv_scale)
    b, S = O.allocate_buffers(3, 50, 0)
    b["encoder_K"][:, :768] = K.float()
    b["encoder_V"][:, :768] = V.float()
    b["observation_state_normalized"].copy_(st)
    b["diffusion_noise"].copy_(nz)
    O.transformer_decoder(ops, w32, b, S, steps=1)
    return b["diffusion_noise"]


def test_decoder_step_fixture_reproduces(decoder_checkpoint):
    """The stored decoder-step result (made through the reference's transformer_decoder) is what
    the oracle's own orchestration gives today."""
    gold = torch.load(GOLDEN / "decoder_step.pt")["kv01"]
    w32 = {k: v.float() for k, v in decoder_checkpoint.items()}
    out = _decoder_step(w32, gold["kv_scale"], O.op_table(True))
    assert (out - gold["out"]).abs().max().item() < 1e-4


@pytest.mark.parametrize("tag", ["kv1", "kv01"])
def test_bf16_operand_floor_of_the_decoder_step(decoder_checkpoint, tag):
    """How close to fp32 can a bf16 tensor-core implementation get on the one-step decoder config?

    Run the step in fp32 with ONLY the tensor-core activation operands rounded to bf16 (weights are bf16
    already; residual stream, accumulators, norm factors, RoPE, softmax and the Euler update stay fp32).
    On a prefix K/V drawn from N(0, 1) that alone lands above the 2e-2 per-step tolerance the full
    forward meets: the tolerance is unreachable on this input for any implementation that feeds
    bf16 operands to the tensor cores. The GPU parity test bounds the CUDA path by 1.25 x this floor."""
    gold = torch.load(GOLDEN / "decoder_step.pt")[tag]
    w32 = {k: v.float() for k, v in decoder_checkpoint.items()}
    out = _decoder_step(w32, gold["kv_scale"], O.op_table(True, False, True))
    floor = (out - gold["out"]).abs().max().item()
    print(f"\n[{tag}] bf16-operand floor: {floor:.4g} (stored {gold['operand_bf16_max_abs']:.4g}; "
          f"reference numerics restated: {gold['bf16_faithful_max_abs']:.4g})")
    assert abs(floor - gold["operand_bf16_max_abs"]) <= 1e-3 * max(1.0, floor)
    assert floor > 2e-2, "if this ever drops below the step tolerance, tighten the GPU test to 2e-2"
    assert floor < gold["bf16_faithful_max_abs"]          # and it is still below the reference's own numerics


def test_error_metrics_fields():
    a = torch.randn(50, 32)
    m = O.error_metrics(a, a + 1e-3)
    assert set(m) == {"max_abs", "mean_abs", "rms_error", "p99_abs", "cosine_similarity"}
    assert math.isclose(m["max_abs"], 1e-3, rel_tol=1e-2) and m["cosine_similarity"] > 0.999999
