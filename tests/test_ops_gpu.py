"""Per-op parity: every CUDA call-site wrapper against the CPU fp32 oracle's op of the same
name, through the C ABI, on the model's real (ragged) shapes.

Tolerance (written in `conftest.assert_close`): |err| <= 1e-2 * rms(ref) + 1e-2 * |ref|. The
oracle keeps every intermediate in fp32; the CUDA ops store bf16 and, where the reference
rounds an intermediate to bf16 (the normalised activations), so do they.
"""
from __future__ import annotations

import pytest
import torch

from conftest import assert_close
from oracle import pi0_ref as O

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def rnd(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(bf16)


@pytest.fixture(scope="module")
def ops():
    from flash_vla_b200 import op_table
    return op_table(fused=False), op_table(fused=True)


@pytest.fixture(scope="module")
def ref_ops():
    return O.op_table(fused=False), O.op_table(fused=True)


def dev(*ts):
    return [t.cuda() for t in ts]


def f32(*ts):
    return [t.float() for t in ts]


@pytest.mark.parametrize("views", [1, 3])
def test_vision_patch_embed(ops, ref_ops, views):
    g = torch.Generator().manual_seed(1)
    img = (torch.rand(views, 224, 224, 3, generator=g) * 2 - 1).to(bf16)
    pw, pb, pos = rnd(g, 14, 14, 3, 1152, scale=0.02), rnd(g, 1152, scale=0.02), rnd(g, 256, 1152, scale=0.02)
    ref = torch.zeros(views, 256, 1152)
    ref_ops[0].vision_patch_embed(*f32(img, pw, pb, pos), ref)
    out = torch.zeros(views, 256, 1152, dtype=bf16, device="cuda")
    ops[0].vision_patch_embed(*dev(img, pw, pb, pos), out)
    assert_close(out, ref, what="vision_patch_embed")


@pytest.mark.parametrize("name,N,act", [("vision_norm_qkv", 3456, 0), ("vision_norm_ffn_up", 4304, 1)])
def test_vision_norm_linear(ops, ref_ops, name, N, act):
    g = torch.Generator().manual_seed(2)
    x = rnd(g, 3, 256, 1152)
    nw, nb = rnd(g, 1152, scale=0.5) + 1, rnd(g, 1152, scale=0.1)
    w, b = rnd(g, 1152, N, scale=0.02), rnd(g, N, scale=0.02)
    ref, ref_n = torch.zeros(3, 256, N), torch.zeros(3, 256, 1152)
    getattr(ref_ops[0], name)(*f32(x, nw, nb, w, b), ref, ref_n)
    out = torch.zeros(3, 256, N, dtype=bf16, device="cuda")
    xn = torch.zeros(3, 256, 1152, dtype=bf16, device="cuda")
    getattr(ops[0], name)(*dev(x, nw, nb, w, b), out, xn)
    assert_close(xn, ref_n, what=name + ".x_norm")
    assert_close(out, ref, what=name)


@pytest.mark.parametrize("views", [1, 3, 12])
@pytest.mark.parametrize("name,N,act", [("vision_norm_qkv", 3456, 0), ("vision_norm_ffn_up", 4304, 1)])
def test_vision_norm_linear_fused_table(ops, ref_ops, name, N, act, views):
    """The fused table folds the LayerNorm into the GEMM (row statistics inside the kernel, scale and shift folded
    into the weights once): same result as the oracle's op, `x_norm` left alone. 12 views give a CTA several
    tiles, where the library centres the rows with a kernel of its own and does write `x_norm`. Rows with a
    large common offset check the variance taken as E[x^2] - mean^2 in fp32."""
    g = torch.Generator().manual_seed(2)
    x = rnd(g, views, 256, 1152)
    x[0, :32] += 6.0                                      # mean several times the spread
    nw, nb = rnd(g, 1152, scale=0.5) + 1, rnd(g, 1152, scale=0.1)
    w, b = rnd(g, 1152, N, scale=0.02), rnd(g, N, scale=0.02)
    ref, ref_n = torch.zeros(views, 256, N), torch.zeros(views, 256, 1152)
    getattr(ref_ops[1], name)(*f32(x, nw, nb, w, b), ref, ref_n)
    out = torch.zeros(views, 256, N, dtype=bf16, device="cuda")
    xn = torch.full((views, 256, 1152), 5.0, dtype=bf16, device="cuda")
    args = dev(x, nw, nb, w, b)
    getattr(ops[1], name)(*args, out, xn)
    assert_close(out, ref, what=name + " (fused table)")
    if views <= 3:
        assert (xn == 5.0).all(), "the fused form must not write x_norm"
    # a second call reuses the folded operands; an in-place weight update refolds them
    out2 = torch.zeros_like(out)
    getattr(ops[1], name)(*args, out2, xn)
    assert torch.equal(out, out2)
    args[3].mul_(2.0)
    getattr(ref_ops[1], name)(*f32(x, nw, nb, w * 2, b), ref, ref_n)
    getattr(ops[1], name)(*args, out2, xn)
    assert_close(out2, ref, what=name + " (fused table, updated weight)")
    # and the two tables agree with each other to rounding
    args[3].div_(2.0)
    getattr(ops[0], name)(*args, out2, xn)
    # (both are bf16 roundings of nearly the same fp32 value: they may land on neighbouring bf16 numbers)
    assert_close(out, out2.float().cpu(), rtol=2e-2, what=name + " fused vs unfused table")


def test_vision_attention(ops, ref_ops):
    g = torch.Generator().manual_seed(3)
    qkv = rnd(g, 3, 256, 3456)
    ref = torch.zeros(3, 256, 1152)
    ref_ops[0].vision_attention(qkv.float(), ref)
    out = torch.zeros(3, 256, 1152, dtype=bf16, device="cuda")
    ops[0].vision_attention(qkv.cuda(), out)
    assert_close(out, ref, what="vision_attention")


@pytest.mark.parametrize("name,K", [("vision_out_proj_residual", 1152), ("vision_ffn_down_residual", 4304)])
def test_vision_linear_bias_residual_in_place(ops, ref_ops, name, K):
    g = torch.Generator().manual_seed(4)
    x, w, b = rnd(g, 3, 256, K), rnd(g, K, 1152, scale=0.02), rnd(g, 1152, scale=0.02)
    res = rnd(g, 3, 256, 1152)
    ref = res.float().clone()
    getattr(ref_ops[0], name)(*f32(x, w, b), ref, ref)
    out = res.cuda().clone()
    getattr(ops[0], name)(*dev(x, w, b), out, out)       # residual aliases the destination
    assert_close(out, ref, what=name)


def test_encoder_projector(ops, ref_ops):
    g = torch.Generator().manual_seed(5)
    x = rnd(g, 3, 256, 1152)
    nw, nb = rnd(g, 1152, scale=0.5) + 1, rnd(g, 1152, scale=0.1)
    w, b = rnd(g, 1152, 2048, scale=0.02), rnd(g, 2048, scale=0.02)
    S = 817                                               # prompt rows after the image rows stay untouched
    ref, ref_n = torch.full((S, 2048), 7.0), torch.zeros(3, 256, 1152)
    ref_ops[0].encoder_projector(*f32(x, nw, nb, w, b), ref, ref_n)
    out = torch.full((S, 2048), 7.0, dtype=bf16, device="cuda")
    xn = torch.zeros(3, 256, 1152, dtype=bf16, device="cuda")
    ops[0].encoder_projector(*dev(x, nw, nb, w, b), out, xn)
    assert_close(out, ref, what="encoder_projector")
    assert (out[768:] == 7.0).all()


@pytest.mark.parametrize("S", [768, 816, 817])
def test_encoder_norm_qkv_rope(ops, ref_ops, S):
    g = torch.Generator().manual_seed(6)
    x, w = rnd(g, S, 2048), rnd(g, 2048, 2560, scale=0.02)
    rope = O.rope_table(S, 0)
    refs = [torch.zeros(S * 8, 256), torch.zeros(S, 256), torch.zeros(S, 256), torch.zeros(S, 2048)]
    ref_ops[0].encoder_norm_qkv_rope(x.float(), w.float(), rope.float(), *refs)
    # the reference rounds x_norm and the projection to bf16 before rotating (wrappers.py:350-352);
    # the op does the same, so it is also held to the default bound against that restatement
    faithful = [torch.zeros_like(r) for r in refs]
    O.op_table(False, faithful=True).encoder_norm_qkv_rope(x.float(), w.float(), rope.float(), *faithful)
    cache_k = torch.zeros(S + 51, 256, dtype=bf16, device="cuda")
    cache_v = torch.zeros(S + 51, 256, dtype=bf16, device="cuda")
    Q = torch.zeros(S * 8, 256, dtype=bf16, device="cuda")
    xn = torch.zeros(S, 2048, dtype=bf16, device="cuda")
    ops[0].encoder_norm_qkv_rope(*dev(x, w, rope), Q, cache_k[:S], cache_v[:S], xn)
    for got, ref, fa, what in zip((Q, cache_k[:S], cache_v[:S], xn), refs, faithful, "Q K V x_norm".split()):
        # The op rounds the projection to bf16 BEFORE rotating, as the reference does. A projection value
        # whose fp32 sum falls on the other side of a rounding boundary moves by one bf16 ulp, and the
        # rotation spreads that over a pair. So: the DEFAULT bound for all but a tiny fraction of the
        # elements, and the wide bound (which a wrong row, column or tile edge would still break) for all.
        for other, tag in ((ref, "fp32"), (fa, "bf16-faithful")):
            o = other.float()
            err = (got.float().cpu() - o).abs()
            default_bound = 1e-2 * o.pow(2).mean().sqrt() + 1e-2 * o.abs()
            outliers = (err > default_bound).float().mean().item()
            print(f"\n[S={S}] {what} vs {tag}: fraction outside the default bound {outliers:.2e}, max-abs {err.max().item():.4g}")
            assert outliers <= 2e-3, f"encoder_norm_qkv_rope.{what} vs {tag}: {outliers:.2e} of the elements outside the default bound"
        assert_close(got, ref, rtol=2e-2, atol_rms=4e-2, what=f"encoder_norm_qkv_rope.{what} vs fp32")
        assert_close(got, fa, rtol=1e-2, atol_rms=3e-2, what=f"encoder_norm_qkv_rope.{what} vs bf16-faithful")
    # The fused table applies the RMS factor to the GEMM's accumulators instead of normalising the rows first:
    # same bounds against the oracle, x_norm left alone.
    Qf, kf, vf = torch.zeros_like(Q), torch.zeros_like(cache_k), torch.zeros_like(cache_v)
    xnf = torch.full((S, 2048), 5.0, dtype=bf16, device="cuda")
    ops[1].encoder_norm_qkv_rope(*dev(x, w, rope), Qf, kf[:S], vf[:S], xnf)
    assert (xnf == 5.0).all(), "the fused form must not write x_norm"
    assert (kf[S:] == 0).all() and (vf[S:] == 0).all()
    for got, ref, what in zip((Qf, kf[:S], vf[:S]), refs, "Q K V".split()):
        o = ref.float()
        err = (got.float().cpu() - o).abs()
        outliers = (err > 1e-2 * o.pow(2).mean().sqrt() + 1e-2 * o.abs()).float().mean().item()
        print(f"\n[S={S}] fused table {what} vs fp32: fraction outside the default bound {outliers:.2e}, max-abs {err.max().item():.4g}")
        assert outliers <= 2e-3, f"encoder_norm_qkv_rope (fused table).{what}: {outliers:.2e} of the elements outside the default bound"
        assert_close(got, ref, rtol=2e-2, atol_rms=4e-2, what=f"encoder_norm_qkv_rope (fused table).{what} vs fp32")
    assert (cache_k[S:] == 0).all() and (cache_v[S:] == 0).all()


@pytest.mark.parametrize("S", [768, 817])
def test_encoder_attention(ops, ref_ops, S):
    g = torch.Generator().manual_seed(7)
    Q, K, V = rnd(g, S * 8, 256), rnd(g, S, 256), rnd(g, S, 256)
    ref = torch.zeros(S, 2048)
    ref_ops[0].encoder_attention(*f32(Q, K, V), 256 ** -0.5, ref)
    out = torch.zeros(S, 2048, dtype=bf16, device="cuda")
    ops[0].encoder_attention(*dev(Q, K, V), 256 ** -0.5, out)
    assert_close(out, ref, what="encoder_attention")


@pytest.mark.parametrize("name,M,K,N", [
    ("encoder_out_proj_residual", 768, 2048, 2048), ("encoder_ffn_down_residual", 817, 16384, 2048),
    ("decoder_out_proj_residual", 51, 2048, 1024), ("decoder_ffn_down_residual", 51, 4096, 1024),
    ("decoder_ffn_down_residual", 204, 4096, 1024), ("decoder_out_proj_residual", 1, 2048, 1024)])
def test_linear_residual(ops, ref_ops, name, M, K, N):
    g = torch.Generator().manual_seed(8)
    x, w, res = rnd(g, M, K), rnd(g, K, N, scale=0.02), rnd(g, M, N)
    ref = res.float().clone()
    getattr(ref_ops[0], name)(x.float(), w.float(), ref)
    out = res.cuda().clone()
    for _ in range(2):                                    # twice: split-K semaphores must self-reset
        out.copy_(res)
        getattr(ops[0], name)(x.cuda(), w.cuda(), out)
    assert_close(out, ref, what=name)


@pytest.mark.parametrize("S", [768, 817])
def test_encoder_norm_gated_ffn(ops, ref_ops, S):
    g = torch.Generator().manual_seed(9)
    x = rnd(g, S, 2048)
    wg, wu = rnd(g, 2048, 16384, scale=0.02), rnd(g, 2048, 16384, scale=0.02)
    ref, ref_n = torch.zeros(S, 16384), torch.zeros(S, 2048)
    ref_ops[0].encoder_norm_gated_ffn(*f32(x, wg, wu), ref, ref_n)
    fa, fa_n = torch.zeros(S, 16384), torch.zeros(S, 2048)
    O.op_table(False, faithful=True).encoder_norm_gated_ffn(*f32(x, wg, wu), fa, fa_n)
    out = torch.zeros(S, 16384, dtype=bf16, device="cuda")
    xn = torch.zeros(S, 2048, dtype=bf16, device="cuda")
    ops[0].encoder_norm_gated_ffn(*dev(x, wg, wu), out, xn)
    # the reference feeds the GEMM the bf16-rounded x_norm (wrappers.py:374-380); against that
    # restatement only the output rounding remains, against pure fp32 the input rounding shows
    assert_close(out, fa, what="encoder_norm_gated_ffn vs bf16-faithful")
    assert_close(out, ref, rtol=2e-2, atol_rms=5e-2, what="encoder_norm_gated_ffn vs fp32")
    assert_close(xn, ref_n, what="encoder_norm_gated_ffn.x_norm")


def test_decoder_small_projections(ops, ref_ops):
    g = torch.Generator().manual_seed(10)
    state, noise = rnd(g, 32), torch.randn(50, 32, generator=g)
    ws, bs = rnd(g, 32, 1024, scale=0.02), rnd(g, 1024, scale=0.02)
    for x_gpu, x_ref, M, name in ((state.cuda(), state.float(), 1, "decoder_state_proj"),
                                  (noise.cuda(), noise, 50, "decoder_action_in_proj"),
                                  (noise.to(bf16).cuda(), noise.to(bf16).float(), 50, "decoder_action_in_proj")):
        ref = torch.zeros(M, 1024)
        getattr(ref_ops[0], name)(x_ref, ws.float(), bs.float(), ref)
        out = torch.zeros(M, 1024, dtype=bf16, device="cuda")
        getattr(ops[0], name)(x_gpu, ws.cuda(), bs.cuda(), out)
        assert_close(out, ref, what=name)
    x, w = rnd(g, 50, 1024), rnd(g, 1024, 1024, scale=0.02)
    ref = torch.zeros(50, 1024)
    ref_ops[0].decoder_action_mlp(x.float(), w.float(), bs.float(), ref)
    dx = torch.zeros(51, 1024, dtype=bf16, device="cuda")
    ops[0].decoder_action_mlp(x.cuda(), w.cuda(), bs.cuda(), dx[1:])     # destination is a row-offset view
    assert_close(dx[1:], ref, what="decoder_action_mlp")
    assert (dx[0] == 0).all()


@pytest.mark.parametrize("S,M", [(768, 51), (816, 51), (817, 51), (768, 1)])
def test_decoder_norm_qkv_rope(ops, ref_ops, S, M):
    g = torch.Generator().manual_seed(11)
    x, w = rnd(g, M, 1024, scale=3.0), rnd(g, 1024, 2560, scale=0.02)
    rope = O.rope_table(M, S)
    refs = [torch.zeros(M * 8, 256), torch.zeros(M, 256), torch.zeros(M, 256), torch.zeros(M)]
    ref_ops[0].decoder_norm_qkv_rope(x.float(), w.float(), rope.float(), *refs)
    K = torch.zeros(S + M, 256, dtype=bf16, device="cuda")
    V = torch.zeros(S + M, 256, dtype=bf16, device="cuda")
    Q = torch.zeros(M * 8, 256, dtype=bf16, device="cuda")
    nf = torch.zeros(M, dtype=bf16, device="cuda")
    for _ in range(2):
        ops[0].decoder_norm_qkv_rope(*dev(x, w, rope), Q, K[S:], V[S:], nf)
    for got, ref, what in zip((Q, K[S:], V[S:], nf), refs, "Q K V factor".split()):
        assert_close(got, ref, what=f"decoder_norm_qkv_rope.{what}")
    assert (K[:S] == 0).all()


# 256 and 64: one view / a short prefix, where most key splits lie wholly behind the prefix (their tensor loads are
# entirely out of range and must still complete)
@pytest.mark.parametrize("S,kv_scale", [(768, 1.0), (768, 0.1), (816, 1.0), (817, 1.0), (1024, 0.1), (256, 1.0), (64, 1.0)])
@pytest.mark.parametrize("fused", [False, True])
def test_decoder_attention(ops, ref_ops, S, kv_scale, fused):
    g = torch.Generator().manual_seed(12)
    keys = S + 51
    Q, K, V = rnd(g, 408, 256), rnd(g, keys, 256, scale=kv_scale), rnd(g, keys, 256, scale=kv_scale)
    ref, ref_scores = torch.zeros(408, 256), torch.zeros(408, keys)
    ref_ops[fused].decoder_attention(*f32(Q, K, V), ref_scores, ref, S)
    q = Q.cuda().clone()
    scores = torch.full((408, keys), 3.0, dtype=bf16, device="cuda")
    ops[fused].decoder_attention(q, K.cuda(), V.cuda(), scores, q, S)        # out aliases Q
    assert_close(q, ref, what="decoder_attention")
    assert (scores == 3.0).all()
    # mask property: the state token's rows must not depend on keys past S
    K2, V2 = K.clone(), V.clone()
    K2[S + 1:] += 1.0
    V2[S + 1:] -= 1.0
    q2 = Q.cuda().clone()
    ops[fused].decoder_attention(q2, K2.cuda(), V2.cuda(), scores, q2, S)
    assert torch.equal(q2[:8], q[:8])


@pytest.mark.parametrize("S,episodes", [(768, 4), (817, 3), (1024, 2)])
def test_decoder_attention_for_a_batch_of_episodes(ops, ref_ops, S, episodes):
    """The batched decoder's attention: E episodes in one call (3-D Q, K / V views of per-episode caches that also
    hold other rows), each against its own keys, the state token's mask included. Every episode is compared with
    the oracle's single-episode op; 1 075 keys (S = 1024) go beyond what the cluster kernel takes for a batch."""
    g = torch.Generator().manual_seed(31)
    keys = S + 51
    Q = rnd(g, episodes, 408, 256)
    cache_k = rnd(g, episodes, keys + 13, 256)             # each episode's cache holds rows that are not keys of this call
    cache_v = rnd(g, episodes, keys + 13, 256)
    q = Q.cuda().clone()
    k_all, v_all = cache_k.cuda()[:, :keys], cache_v.cuda()[:, :keys]
    ops[1].decoder_attention(q.view(-1, 256), k_all, v_all, None, q.view(-1, 256), S)      # flat rows, out aliases Q
    for e in range(episodes):
        ref = torch.zeros(408, 256)
        ref_ops[1].decoder_attention(Q[e].float(), cache_k[e, :keys].float(), cache_v[e, :keys].float(), None, ref, S)
        assert_close(q[e], ref, what=f"decoder_attention, episode {e} of {episodes}")
    # mask property per episode: the state token's rows must not depend on keys past S
    k2, v2 = cache_k.clone(), cache_v.clone()
    k2[:, S + 1:] += 1.0
    v2[:, S + 1:] -= 1.0
    q2 = Q.cuda().clone()
    ops[1].decoder_attention(q2.view(-1, 256), k2.cuda()[:, :keys], v2.cuda()[:, :keys], None, q2.view(-1, 256), S)
    assert torch.equal(q2[:, :8], q[:, :8])
    assert not torch.equal(q2[:, 8:], q[:, 8:])


@pytest.mark.parametrize("M", [51, 1])
@pytest.mark.parametrize("fused", [False, True])
def test_decoder_norm_gated_ffn(ops, ref_ops, M, fused):
    g = torch.Generator().manual_seed(13)
    x = rnd(g, M, 1024, scale=3.0)
    wg, wu = rnd(g, 1024, 4096, scale=0.02), rnd(g, 1024, 4096, scale=0.02)
    ref, ref_f = torch.zeros(M, 4096), torch.zeros(M)
    ref_ops[fused].decoder_norm_gated_ffn(*f32(x, wg, wu), ref, ref_f)
    out = torch.zeros(M, 4096, dtype=bf16, device="cuda")
    nf = torch.full((M,), 5.0, dtype=bf16, device="cuda")
    for _ in range(2):
        ops[fused].decoder_norm_gated_ffn(*dev(x, wg, wu), out, nf)
    assert_close(out, ref, what="decoder_norm_gated_ffn")
    if fused:
        assert (nf == 5.0).all()                          # fused form leaves norm_factor untouched
    else:
        assert_close(nf, ref_f, what="norm_factor")


@pytest.mark.parametrize("out_dtype", [bf16, torch.float32])
@pytest.mark.parametrize("fused", [False, True])
def test_decoder_action_out_proj(ops, ref_ops, out_dtype, fused):
    g = torch.Generator().manual_seed(14)
    x, w, b = rnd(g, 50, 1024, scale=3.0), rnd(g, 1024, 32, scale=0.02), rnd(g, 32, scale=0.02)
    noise = rnd(g, 50, 32)
    ref = noise.float().clone()
    ref_ops[fused].decoder_action_out_proj(*f32(x, w, b), ref, torch.zeros(50))
    dx = torch.zeros(51, 1024, dtype=bf16, device="cuda")
    dx[1:] = x.cuda()
    out = noise.cuda().to(out_dtype)
    nf = torch.zeros(51, dtype=bf16, device="cuda")
    ops[fused].decoder_action_out_proj(dx[1:], w.cuda(), b.cuda(), out, nf)
    assert_close(out, ref, rtol=(1e-2 if out_dtype == bf16 else 2e-3), atol_rms=(1e-2 if out_dtype == bf16 else 2e-3),
                 what="decoder_action_out_proj")


def test_bad_arguments_raise_before_launch(ops):
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda._lib import FvlaError
    x = torch.zeros(51, 1024, dtype=bf16, device="cuda")
    w = torch.zeros(1024, 1024, dtype=bf16, device="cuda")
    with pytest.raises(ValueError):
        ops[0].decoder_out_proj_residual(x.float(), w, x)            # wrong dtype
    with pytest.raises(ValueError):
        ops[0].decoder_out_proj_residual(x.t(), w, x)                # not contiguous
    with pytest.raises(ValueError):
        ops[0].decoder_out_proj_residual(x.cpu(), w, x)              # host tensor
    with pytest.raises(FvlaError):
        q = torch.zeros(408, 128, dtype=bf16, device="cuda")         # head_dim the library does not build
        k = torch.zeros(819, 128, dtype=bf16, device="cuda")
        ops[0].decoder_attention(q, k, k, None, q, 768)
    torch.cuda.synchronize()


@pytest.mark.parametrize("rows", [1, 48, 49])
def test_embed_prompt_is_a_row_gather(ops, rows):
    """Prompt embedding lookup against the oracle's gather, ids at both ends of the vocabulary included."""
    g = torch.Generator().manual_seed(5)
    vocab, dim = 4096, 2048
    table = rnd(g, vocab, dim, scale=0.02)
    ids = torch.randint(0, vocab, (rows,), generator=g)
    ids[0], ids[-1] = vocab - 1, 0
    want = O.embed_prompt(table, ids)
    out = torch.zeros(rows, dim, dtype=bf16, device="cuda")
    ops[1].embed_prompt(table.cuda(), ids.cuda(), out)
    assert torch.equal(out.cpu(), want.to(bf16))


def test_embed_prompt_reports_a_bad_id(ops):
    """An id outside the vocabulary gives a zero row and is reported through the device status word."""
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(6)
    table = rnd(g, 100, 64).cuda()
    ids = torch.tensor([3, 100, 7, -1], dtype=torch.int64).cuda()
    out = torch.full((4, 64), 9.0, dtype=bf16, device="cuda")
    assert lib.fvla_device_status(None) == 0
    ops[1].embed_prompt(table, ids, out)
    assert lib.fvla_device_status(None) == 7          # reading clears it
    assert lib.fvla_device_status(None) == 0
    assert torch.equal(out[0], table[3]) and torch.equal(out[2], table[7])
    assert (out[1] == 0).all() and (out[3] == 0).all()


@pytest.mark.parametrize("src_dtype,dst_dtype", [(bf16, torch.float32), (torch.float32, bf16), (torch.float32, torch.float32), (bf16, bf16)])
def test_copy_rows_converts_and_refreshes_the_shadow(ops, src_dtype, dst_dtype):
    """The library's own copy kernel (used for the decoder's small copies): any bf16 / fp32 pairing, a row-offset
    view as destination, and the bf16 shadow of a registered fp32 destination kept current."""
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import wrappers
    g = torch.Generator().manual_seed(12)
    src = torch.randn(3, 1024, generator=g).to(src_dtype).cuda()
    owner = torch.zeros(7, 1024, dtype=dst_dtype, device="cuda")
    shadow = None
    if dst_dtype == torch.float32:
        shadow = torch.full((7, 1024), 5.0, dtype=bf16, device="cuda")
        wrappers.register_bf16_shadow(owner, shadow)
    ops[1].copy_rows(owner[2:5], src)
    torch.cuda.synchronize()
    assert torch.equal(owner[2:5], src.to(dst_dtype)) and (owner[:2] == 0).all() and (owner[5:] == 0).all()
    if shadow is not None:
        assert torch.equal(shadow[2:5], src.to(bf16)) and (shadow[:2] == 0).all()
    with pytest.raises(ValueError):
        ops[1].copy_rows(owner[2:4], src)
