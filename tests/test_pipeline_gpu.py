"""Stage- and pipeline-level parity on the GPU against committed oracle fixtures.

Tolerances are the ones the benchmark definition states: per Euler step (teacher-forced, i.e.
both sides start the step from the oracle's noise) max-abs <= 2e-2; on the final action chunk
of the free-running 10-step pass cosine >= 0.999.

On the synthetic-prefix decoder step (prefix K/V drawn from N(0,1) or N(0,0.1) instead of coming
from the encoder) the 2e-2 step tolerance is not reachable by a bf16 tensor-core implementation:
fp32 arithmetic with nothing but the tensor-core activation operands rounded to bf16 already lands
3e-2 to 4e-2 from the fp32 result (`operand_bf16_max_abs` in the fixture, reproduced on the CPU by
tests/test_oracle.py::test_bf16_operand_floor_of_the_decoder_step). That case is therefore bounded
by 1.25 x that floor, and must also stay below the restated numerics of the reference itself.
"""
from __future__ import annotations

import pytest
import torch

from conftest import GOLDEN
from flash_vla_b200.synthetic import bench_inputs, decoder_step_inputs, prompt_embeds

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16

STEP_MAX_ABS = 2e-2
FINAL_COSINE = 0.999


def cosine(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten().cpu(), b.float().flatten().cpu(), dim=0).item()


@pytest.fixture(scope="module")
def device_weights(full_checkpoint):
    return {k: v.cuda() for k, v in full_checkpoint.items()}


@pytest.mark.parametrize("tag", ["kv1", "kv01"])
@pytest.mark.parametrize("fused", [True, False])
def test_one_decoder_step(device_weights, tag, fused):
    """18 layers, M = 51, 819 keys, timestep t = 1.0 on a synthetic prefix KV."""
    from flash_vla_b200 import op_table
    from flash_vla_b200.hardware.nvidia.b200.pi0 import pipeline
    from flash_vla_b200.hardware.nvidia.b200.pi0.buffers import allocate_static_buffers
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import wrappers
    from flash_vla_b200.runtime.cuda import ScratchPool

    gold = torch.load(GOLDEN / "decoder_step.pt")[tag]
    K, V, state, noise = decoder_step_inputs(gold["kv_scale"])
    b, S = allocate_static_buffers(3, 50, 0, "cuda")
    b["encoder_K"][:, :768].copy_(K)
    b["encoder_V"][:, :768].copy_(V)
    b["observation_state_normalized"].copy_(state)
    b["diffusion_noise"].copy_(noise)
    with wrappers.use_pool(ScratchPool()):
        pipeline.transformer_decoder(op_table(fused), device_weights, b, S, steps=1)
    torch.cuda.synchronize()
    err = (b["diffusion_noise_f32"].cpu() - gold["out"]).abs().max().item()
    err_x = (b["decoder_x"].float().cpu() - gold["decoder_x"]).abs()
    print(f"\n[{tag} fused={fused}] step max-abs {err:.4g}; decoder_x max-abs {err_x.max().item():.4g} "
          f"(|x| max {gold['decoder_x'].abs().max().item():.3g})")
    floor = gold["operand_bf16_max_abs"]
    bound = STEP_MAX_ABS if 1.25 * floor <= STEP_MAX_ABS else 1.25 * floor
    assert err <= bound, f"step max-abs {err:.4g} exceeds {bound:.4g} (bf16-operand floor {floor:.4g})"
    assert err <= gold["bf16_faithful_max_abs"]
    # the bf16 view differs from the master only by its own rounding
    assert (b["diffusion_noise"].float() - b["diffusion_noise_f32"]).abs().max().item() <= \
        b["diffusion_noise_f32"].abs().max().item() * 2 ** -8


# Bounds on the strided stage probes of a full forward, against the fp32 oracle: (relative RMS error,
# max-abs error as a fraction of max |ref|). Cosine alone would hide one wrong row or tile edge in 10^4
# values; a max-abs bound does not. The figures are 1.5 to 2 times what the kernels measure (vision_x 1.1e-2 / 2.7e-2,
# encoder_x 1.6e-2 / 3.1e-2).
PROBE_BOUNDS = {"vision_x": (2e-2, 5e-2), "encoder_x": (2.5e-2, 5e-2), "encoder_K": (3e-2, 1e-1), "encoder_V": (3e-2, 1e-1)}


@pytest.mark.parametrize("prompt_len", [0, 48, 49, 256])
def test_full_forward(full_checkpoint, prompt_len):
    """Whole pass in one CUDA graph: vision + prefix encoder + 10 decoder steps. Prompt 256 (prefix
    1024, 1075 decoder keys) is the reference's second benchmark workload (benchmarks/e2e.py:8-11)."""
    from flash_vla_b200 import Pi0Inference
    from flash_vla_b200.hardware.nvidia.b200.pi0 import pipeline
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import wrappers

    gold = torch.load(GOLDEN / f"forward_p{prompt_len}.pt")
    ck = dict(full_checkpoint)
    if prompt_len:
        rows = prompt_embeds(prompt_len)[1]
        ck["language_embeds"] = torch.zeros_like(rows)           # the prompt arrives through set_prompt below
    images, state, noise = bench_inputs()
    # a small table holding the prompt's rows in shuffled order; the ids undo the shuffle
    perm = torch.randperm(max(prompt_len, 1), generator=torch.Generator().manual_seed(9))
    in_graph = prompt_len in (49, 256)            # these two gather inside the captured pass from a static id buffer
    engine = Pi0Inference(ck, num_views=3, chunk_size=50, embedding_table=rows[perm] if in_graph else None)
    assert engine.encoder_seq_len == 768 + prompt_len
    if prompt_len:
        if in_graph:
            engine.set_prompt(torch.argsort(perm))
            with pytest.raises(ValueError):
                engine.set_prompt(torch.argsort(perm), rows[perm])
        else:
            engine.set_prompt(torch.argsort(perm), rows[perm])
        with pytest.raises(ValueError):
            engine.set_prompt(torch.arange(prompt_len + 1), rows)
    with pytest.raises(ValueError):
        engine.forward(images[:1], state, noise)           # a wrong input shape must not broadcast
    out = engine.forward(images, state, noise).clone()
    out2 = engine.forward(images, state, noise).clone()
    torch.cuda.synchronize()
    assert torch.equal(out, out2), "two replays of the same inputs must be bit-identical"

    b = engine.buffers
    S = engine.encoder_seq_len
    probes = {"vision_x": b["vision_x"][:, ::16, ::9], "encoder_x": b["encoder_x"][::16, ::16],
              "encoder_K": b["encoder_K"][:, ::32, ::8], "encoder_V": b["encoder_V"][:, ::32, ::8]}
    for name, got in probes.items():
        ref = gold[name]
        if name in ("encoder_K", "encoder_V"):      # decoder rows hold the last step's K/V on both sides
            got, ref = got[:, : S // 32], ref[:, : S // 32]
        e = (got.float().cpu() - ref).abs()
        rel_rms = (e.pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
        rel_max = e.max().item() / ref.abs().max().item()
        print(f"\n[p{prompt_len}] {name}: max-abs {e.max().item():.4g} ({rel_max:.4g} of max |ref|), rel-rms "
              f"{rel_rms:.4g}, cos {cosine(got, ref):.6f}")
        assert cosine(got, ref) >= 0.999, name
        assert rel_rms <= PROBE_BOUNDS[name][0] and rel_max <= PROBE_BOUNDS[name][1], (name, rel_rms, rel_max)

    cos = cosine(out, gold["actions"])
    print(f"\n[p{prompt_len}] final actions: cosine {cos:.6f}, max-abs "
          f"{(out.float().cpu() - gold['actions']).abs().max().item():.4g} (|a| max {gold['actions'].abs().max().item():.3g})")
    assert cos >= FINAL_COSINE

    # teacher-forced per-step error: start each step from the oracle's noise, on this engine's KV
    master = b["diffusion_noise_f32"]
    worst = 0.0
    with wrappers.use_pool(engine.pool):
        for step in range(10):
            start = noise if step == 0 else gold["trace"][step - 1]
            master.copy_(start)
            pipeline.decoder_step(engine.ops, engine.weights, b, S, step)
            torch.cuda.synchronize()
            err = (master.cpu() - gold["trace"][step]).abs().max().item()
            worst = max(worst, err)
    print(f"[p{prompt_len}] teacher-forced per-step max-abs: worst {worst:.4g}")
    assert worst <= STEP_MAX_ABS
    del engine
    torch.cuda.empty_cache()


def test_fused_and_unfused_tables_agree(full_checkpoint):
    """The reference's bisection gate (eval/correctness/pi0/fused_vs_unfused.py:34-60): the same forward through
    the fused and the unfused op table. Here the two tables differ in how three prefix ops apply their row norm
    (inside the GEMM against a kernel of its own), so this compares two implementations; both are also held to
    the oracle's actions."""
    from flash_vla_b200 import Pi0Inference

    gold = torch.load(GOLDEN / "forward_p0.pt")
    images, state, noise = bench_inputs()
    outs, probes = {}, {}
    for fused in (True, False):
        engine = Pi0Inference(full_checkpoint, num_views=3, chunk_size=50, fused=fused)
        outs[fused] = engine.forward(images, state, noise).float().cpu()
        b = engine.buffers
        probes[fused] = {k: b[k].float().cpu().clone() for k in ("vision_x", "encoder_x")}
        # the fused table leaves the row-norm scratch of the prefix ops it fuses untouched
        touched = b["vision_x_norm"].abs().sum().item() != 0
        assert touched, "encoder_projector (unfused in both tables) writes vision_x_norm"
        del engine
    for name in ("vision_x", "encoder_x"):
        f, u = probes[True][name], probes[False][name]
        rel_rms = ((f - u).pow(2).mean().sqrt() / u.pow(2).mean().sqrt()).item()
        print(f"\n{name}: fused vs unfused table rel-rms {rel_rms:.4g}, cos {cosine(f, u):.6f}")
        assert rel_rms <= 2e-2 and cosine(f, u) >= 0.9995, name
    diff = (outs[True] - outs[False]).abs().max().item()
    print(f"\nactions: fused vs unfused table max-abs {diff:.4g}, cosine {cosine(outs[True], outs[False]):.6f}")
    assert cosine(outs[True], outs[False]) >= FINAL_COSINE
    for fused in (True, False):
        assert cosine(outs[fused], gold["actions"]) >= FINAL_COSINE, fused


def test_many_replays_stay_identical_and_healthy(full_checkpoint):
    """The kernels' inter-CTA hand-offs (cluster exchanges, the shared-out split-K sum, self-resetting counters)
    must leave no state behind: 150 replays of the captured forward give the first result bit for bit, and no
    bounded device wait has expired."""
    from flash_vla_b200 import Pi0Inference
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib

    engine = Pi0Inference(full_checkpoint, num_views=3, chunk_size=50)
    images, state, noise = bench_inputs()
    first = engine.forward(images, state, noise).clone()
    for _ in range(150):
        engine.graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(engine.forward(images, state, noise), first)
    assert _lib.load().fvla_device_status(None) == 0


def test_one_view_forward(full_checkpoint):
    """One camera view (prefix 256, decoder keys 307): the M = 256 shapes of every prefix kernel and a decoder
    attention whose later key splits lie wholly behind the prefix, against the oracle's forward on the same
    inputs (computed here: about two seconds of CPU)."""
    from flash_vla_b200 import Pi0Inference
    from oracle import pi0_ref as O

    images, state, noise = bench_inputs()
    images = images[:1]
    ref, _ = O.forward({k: v.float() for k, v in full_checkpoint.items()}, images.float(), state.float(), noise.float(), num_views=1)
    engine = Pi0Inference(full_checkpoint, num_views=1, chunk_size=50)
    assert engine.encoder_seq_len == 256
    out = engine.forward(images, state, noise)
    cos = cosine(out, ref)
    print(f"\none view: final actions cosine {cos:.6f}, max-abs {(out.float().cpu() - ref.float()).abs().max().item():.4g}")
    assert cos >= FINAL_COSINE


def test_frozen_pool_refuses_new_scratch(full_checkpoint):
    """After capture a scratch request that warm-up never made raises instead of allocating."""
    from flash_vla_b200.runtime.cuda import ScratchPool
    pool = ScratchPool()
    pool.get("a", (4,), torch.float32, "cuda")
    pool.freeze()
    pool.get("a", (4,), torch.float32, "cuda")
    with pytest.raises(RuntimeError):
        pool.get("a", (8,), torch.float32, "cuda")


@pytest.mark.parametrize("batch_prefix,batch_decoder", [(False, False), (True, False), (True, True)],
                         ids=["streams", "batched-prefix", "batched-prefix-and-decoder"])
def test_concurrent_episodes_match_the_single_episode_engine(full_checkpoint, batch_prefix, batch_decoder):
    """The throughput profile: E episodes inside one graph, shared weights, own KV caches and decoder buffers.
    batch_prefix=False runs E complete single-episode passes on E streams, the same kernels per episode as
    the single-episode engine: results must be bit-identical to it. batch_prefix=True runs SigLIP and the
    prefix encoder once over all episodes' rows (differently shaped launches of the same kernels, so the
    results agree to rounding, not bit for bit); batch_decoder=True also runs the action expert once over
    all episodes' rows (M = 153 here), on the general GEMM kernels with per-episode attention inside one
    launch. Either way every episode is checked against the oracle's result for its own inputs."""
    from flash_vla_b200 import Pi0Inference

    E = 3
    sets = [bench_inputs(seed=e) for e in range(E)]
    single = Pi0Inference(full_checkpoint, num_views=3, chunk_size=50)
    want = [single.forward(*s).clone() for s in sets]
    del single
    torch.cuda.empty_cache()
    multi = Pi0Inference(full_checkpoint, num_views=3, chunk_size=50, episodes=E, batch_prefix=batch_prefix,
                         batch_decoder=batch_decoder)
    assert multi.batch_prefix == batch_prefix and multi.batch_decoder == batch_decoder
    batched = [torch.stack([s[i] for s in sets]) for i in range(3)]
    got = multi.forward(*batched).clone()
    got2 = multi.forward(*batched).clone()
    torch.cuda.synchronize()
    assert got.shape == (E, 50, 32)
    assert torch.equal(got, got2), "two replays of the same inputs must be bit-identical"
    for e in range(E):
        if batch_prefix:
            diff = (got[e].float() - want[e].float()).abs().max().item()
            print(f"\n[episode {e}] batched prefix vs single-episode engine: max-abs {diff:.4g}")
            assert cosine(got[e], want[e]) >= 0.9999
        else:
            assert torch.equal(got[e], want[e]), f"episode {e} differs from the single-episode engine"
    # and every episode is right on its own inputs, not merely equal to another CUDA run: the oracle's
    # result for the inputs of seeds 1 and 2 is a committed fixture (seed 0 is forward_p0.pt)
    for e in range(E):
        gold = torch.load(GOLDEN / ("forward_p0.pt" if e == 0 else f"forward_p0_seed{e}.pt"))
        cos = cosine(got[e], gold["actions"])
        err = (got[e].float().cpu() - gold["actions"]).abs().max().item()
        print(f"\n[episode {e}] cosine {cos:.6f}, max-abs {err:.4g}")
        assert cos >= FINAL_COSINE
    with pytest.raises(ValueError):
        Pi0Inference(full_checkpoint, num_views=3, chunk_size=50, episodes=0, capture=False)


def test_engine_with_a_chunk_beyond_the_cluster_gemm(full_checkpoint):
    """chunk_size 64 gives M = 65 decoder rows, one more than the cluster GEMM's 64 token slots: the
    decoder GEMMs then run on the general kernels, which cannot refresh the bf16 shadow of the fp32
    residual stream in their epilogue (a conversion kernel follows them instead). The engine must still
    build and agree with the oracle (one step, two layers, as the reference's own bisection runs do)."""
    from flash_vla_b200 import Pi0Inference
    from oracle import pi0_ref as O

    images, state, noise = bench_inputs(chunk_size=64)
    engine = Pi0Inference(full_checkpoint, num_views=3, chunk_size=64, steps=1, layers=2)
    out = engine.forward(images, state, noise).float().cpu()
    w32 = {k: v.float() for k, v in full_checkpoint.items()}
    ref, _ = O.forward(w32, images, state, noise, chunk_size=64, steps=1, layers=2)
    err = (out - ref).abs().max().item()
    print(f"\n[chunk 64] one step, two layers: max-abs {err:.4g}")
    assert err <= STEP_MAX_ABS
    del engine
    torch.cuda.empty_cache()


def test_two_devices_in_one_process(full_checkpoint):
    """One process driving two GPUs: kernel attributes, SM counts and the status word are per device, so
    the second engine must work as well as the first and both must match the fixture."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from flash_vla_b200 import Pi0Inference

    gold = torch.load(GOLDEN / "forward_p0.pt")
    images, state, noise = bench_inputs()
    outs = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            engine = Pi0Inference(full_checkpoint, num_views=3, chunk_size=50, device=f"cuda:{dev}")
            outs.append(engine.forward(images, state, noise).float().cpu())
            torch.cuda.synchronize(dev)
            del engine
            torch.cuda.empty_cache()
    assert torch.equal(outs[0], outs[1])
    assert cosine(outs[0], gold["actions"]) >= FINAL_COSINE
