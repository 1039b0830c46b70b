"""Parity with the reference's own GPU code. `tests/golden/reference_gpu.pt` holds what the reference's TileLang
kernels, op table, pipeline and engine produced on a B200 (made by `tests/golden/make_reference_gpu_golden.py`
from an installed copy of the reference; inputs are regenerated here from their seeds). Two parties are held to it:

  * the CPU oracle (`-m "not gpu"`): every op of the table, the whole forward and the one-decoder-step
    configuration. This pins the oracle's GEMM / norm / GeGLU / RoPE arithmetic to the reference's kernels.
  * this package's CUDA path (`-m gpu`), through the C ABI: the same ops (both op tables), forward and step.

Tolerance for the ops: the default bound of `conftest.assert_close`, |err| <= 1e-2 rms(ref) + 1e-2 |ref|, on the
fixture's strided sample of each output (both sides are bf16 roundings of nearly the same fp32 value).
"""
from __future__ import annotations

import pytest
import torch

import reference_cases as RC
from conftest import GOLDEN, assert_close
from flash_vla_b200.synthetic import bench_inputs, decoder_step_inputs

bf16 = torch.bfloat16


@pytest.fixture(scope="module")
def reference():
    return torch.load(GOLDEN / "reference_gpu.pt")


def cosine(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten().cpu(), b.float().flatten().cpu(), dim=0).item()


def check_outputs(case, outs, ref_samples, who, skip=()):
    for name, tensor in outs.items():
        if name in skip:
            continue
        got = RC.sample(tensor)
        assert_close(got, ref_samples[name].float(), what=f"{who} {case.name}.{name} vs the reference's kernel")


# ---------------------------------------------------------------- the oracle against the reference (CPU)

@pytest.mark.parametrize("case", RC.CASES, ids=lambda c: c.name)
def test_oracle_op_matches_the_reference_kernel(reference, case):
    from oracle import pi0_ref as O
    tensors = {k: (v.float() if torch.is_tensor(v) else v) for k, v in case.inputs().items()}
    outs = case.run(O.op_table(True), tensors)
    check_outputs(case, outs, reference["ops"][case.name + "/fused"], "oracle")


def ref_forward(reference, prompt_len):
    return reference["forward_fused" if prompt_len == 0 else f"forward_fused_p{prompt_len}"]


@pytest.mark.parametrize("prompt_len", [0, 48, 49, 256])
def test_oracle_forward_matches_the_reference_engine(reference, prompt_len):
    """The oracle's forward fixtures (fp32, `forward_p{0,48,49,256}.pt`; 49 gives the ragged prefix 817) against the reference engine's forward on the
    same checkpoint, prompt rows and inputs: final actions and the stage probes. Bounds are twice what was measured
    (actions 1.0 - 1.1e-2 of max |a|, rel-rms 0.6 - 0.8e-2; probes rel-rms 1.1 - 1.6e-2, max 1.5 - 2.9e-2 of max |ref|)."""
    ours, ref = torch.load(GOLDEN / f"forward_p{prompt_len}.pt"), ref_forward(reference, prompt_len)
    if prompt_len == 0:
        assert ref["replay_identical"]
    rows = (768 + prompt_len) // 32
    for name in ("actions", "vision_x", "encoder_x", "encoder_K", "encoder_V"):
        a, b = ours[name].float(), ref[name].float()
        if name in ("encoder_K", "encoder_V"):       # decoder rows hold the last step's K / V: prefix rows only
            a, b = a[:, :rows], b[:, :rows]
        e = (a - b).abs()
        rel_rms = (e.pow(2).mean().sqrt() / b.pow(2).mean().sqrt()).item()
        rel_max = (e.max() / b.abs().max()).item()
        print(f"\n[p{prompt_len}] oracle vs reference engine, {name}: rel-rms {rel_rms:.4g}, max-abs {e.max().item():.4g} ({rel_max:.4g} of max |ref|), cos {cosine(a, b):.6f}")
        assert cosine(a, b) >= 0.9995 and rel_rms <= 3.2e-2 and rel_max <= 6e-2, name


@pytest.mark.parametrize("seed", [1, 2])
def test_oracle_forward_of_other_episodes_matches_the_reference_engine(reference, seed):
    """The inputs of episodes 1 and 2 of the throughput profile through the reference engine, against the oracle."""
    ours, ref = torch.load(GOLDEN / f"forward_p0_seed{seed}.pt")["actions"].float(), reference[f"forward_fused_seed{seed}"]["actions"].float()
    e = (ours - ref).abs()
    print(f"\n[seed {seed}] oracle vs reference engine: max-abs {e.max().item():.4g} ({(e.max() / ref.abs().max()).item():.4g} of max |a|), cos {cosine(ours, ref):.6f}")
    assert cosine(ours, ref) >= 0.9995 and (e.max() / ref.abs().max()).item() <= 3e-2


def test_reference_decoder_step_against_the_oracle(reference):
    """The "one decoder diffusion step" configuration: how far the reference's own kernels are from the fp32 oracle.
    They are further away (7.9e-2 / 6.3e-2 max-abs) than the bf16-operand floor the CUDA path is held to, and close
    to the oracle's bf16-faithful restatement of the reference's numerics (6.4e-2)."""
    gold = torch.load(GOLDEN / "decoder_step.pt")
    for tag in ("kv1", "kv01"):
        ref, fp32 = reference["decoder_step"][tag + "_fused"], gold[tag]
        err = (ref["out"].float() - fp32["out"]).abs().max().item()
        print(f"\n[{tag}] reference's step vs fp32 oracle: max-abs {err:.4g} (oracle's bf16-faithful restatement: {fp32['bf16_faithful_max_abs']:.4g})")
        assert err <= 2.0 * fp32["bf16_faithful_max_abs"]
        assert cosine(ref["out"], fp32["out"]) >= 0.999


# ---------------------------------------------------------------- the CUDA path against the reference (GPU)

@pytest.mark.gpu
@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("case", RC.CASES, ids=lambda c: c.name)
def test_cuda_op_matches_the_reference_kernel(reference, case, fused):
    from flash_vla_b200 import op_table
    tensors = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in case.inputs().items()}
    outs = case.run(op_table(fused), tensors)
    torch.cuda.synchronize()
    # this package's fused table folds some row norms into the GEMM and leaves their scratch output unwritten
    check_outputs(case, outs, reference["ops"][case.name + "/fused"], f"CUDA (fused={fused})", skip=case.optional if fused else ())


@pytest.mark.gpu
@pytest.mark.parametrize("prompt_len", [0, 49, 256])
def test_cuda_forward_matches_the_reference_engine(reference, full_checkpoint, prompt_len):
    """This engine's forward against the reference engine's on the same checkpoint and inputs; prompt 256 (prefix
    1024, 1 075 decoder keys) is the reference's second benchmark workload."""
    from flash_vla_b200 import Pi0Inference
    from flash_vla_b200.synthetic import prompt_embeds
    ref = ref_forward(reference, prompt_len)
    images, state, noise = bench_inputs()
    ck = dict(full_checkpoint)
    if prompt_len:
        ck["language_embeds"] = prompt_embeds(prompt_len)[1]
    engine = Pi0Inference(ck, num_views=3, chunk_size=50)
    out = engine.forward(images, state, noise).float().cpu()
    b = engine.buffers
    rows = (768 + prompt_len) // 32
    probes = {"actions": out, "vision_x": b["vision_x"][:, ::16, ::9], "encoder_x": b["encoder_x"][::16, ::16],
              "encoder_K": b["encoder_K"][:, ::32, ::8][:, :rows], "encoder_V": b["encoder_V"][:, ::32, ::8][:, :rows]}
    for name, got in probes.items():
        want = ref[name].float()
        if name in ("encoder_K", "encoder_V"):
            want = want[:, :rows]
        e = (got.float().cpu() - want).abs()
        rel_rms = (e.pow(2).mean().sqrt() / want.pow(2).mean().sqrt()).item()
        rel_max = (e.max() / want.abs().max()).item()
        print(f"\n[p{prompt_len}] CUDA vs reference engine, {name}: rel-rms {rel_rms:.4g}, max-abs {e.max().item():.4g} ({rel_max:.4g} of max |ref|), cos {cosine(got, want):.6f}")
        assert cosine(got, want) >= 0.999 and rel_rms <= 4e-2 and rel_max <= 1e-1, name
    # this engine's time for the same pass, beside the reference's recorded one
    for _ in range(3):
        engine.graph.replay()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        engine.graph.replay()
    e.record()
    torch.cuda.synchronize()
    ref_ms = reference["timing"]["ms_per_replay"] if prompt_len == 0 else ref["ms_per_replay"]
    print(f"\n[p{prompt_len}] ms per forward: this engine {s.elapsed_time(e) / 10:.2f}, reference engine (recorded) {float(ref_ms):.2f}")


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["kv1", "kv01"])
def test_cuda_decoder_step_matches_the_reference(reference, full_checkpoint, tag):
    """One decoder step on a synthetic prefix KV: two bf16 implementations of the same step. Each is within its
    own floor of the fp32 result; the bound between them is the sum of the two floors."""
    from flash_vla_b200 import op_table
    from flash_vla_b200.hardware.nvidia.b200.pi0 import pipeline
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import wrappers
    from flash_vla_b200.hardware.nvidia.b200.pi0.buffers import allocate_static_buffers
    from flash_vla_b200.runtime.cuda import ScratchPool

    ref = reference["decoder_step"][tag + "_fused"]
    gold = torch.load(GOLDEN / "decoder_step.pt")[tag]
    weights = {k: v.cuda() for k, v in full_checkpoint.items() if k.startswith("decoder_")}
    K, V, state, noise = decoder_step_inputs(ref["kv_scale"])
    b, S = allocate_static_buffers(3, 50, 0, "cuda")
    b["encoder_K"][:, :768].copy_(K)
    b["encoder_V"][:, :768].copy_(V)
    b["observation_state_normalized"].copy_(state)
    b["diffusion_noise"].copy_(noise)
    with wrappers.use_pool(ScratchPool()):
        pipeline.transformer_decoder(op_table(True), weights, b, S, steps=1)
    torch.cuda.synchronize()
    got = b["diffusion_noise_f32"].cpu()
    err_ref = (got - ref["out"].float()).abs().max().item()
    err_fp32 = (got - gold["out"]).abs().max().item()
    ref_fp32 = (ref["out"].float() - gold["out"]).abs().max().item()
    print(f"\n[{tag}] CUDA vs reference {err_ref:.4g}; CUDA vs fp32 oracle {err_fp32:.4g}; reference vs fp32 oracle {ref_fp32:.4g}")
    assert err_ref <= gold["operand_bf16_max_abs"] * 1.25 + ref_fp32
    assert cosine(got, ref["out"]) >= 0.999
