"""Generate the committed fixtures under tests/golden/ from the reference's CPU-runnable code.

Run once, in a container that has the reference checkout (it cannot travel to the GPU box):

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py /path/to/reference [part ...]

Parts (default: all): rope checkpoint attention forward[=prompt_len,...] episodes decoder_step openpi.

What is pinned, and against what:
  * rope.pt            - the reference's own `rope_table` (buffers.py:15-23) for the three
                         prefix lengths used by the tests.
  * checkpoint.json    - SHA-256 of selected tensors of the reference's own
                         `random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cpu")`
                         (weights.py:10-24); the package's generator must reproduce them.
  * attention.pt       - the reference's own torch attention functions
                         (kernels/attention.py:20-34) on small seeded inputs.
  * forward_p{0,48,49,256}.pt - final actions, per-step trace and probes of the CPU fp32 oracle on
                         the benchmark inputs, after checking that driving the REFERENCE'S OWN
                         `pipeline.py` with the oracle's op table (and the reference's own
                         attention functions) gives the same result. The reference's kernels
                         cannot run on a CPU, so these vectors pin the oracle's orchestration
                         and the torch-level pieces, not the TileLang kernels: the arithmetic
                         of the GEMM/norm/RoPE ops stays "parity unpinned" by the reference.
                         prompt 256 (prefix 1024, 1075 decoder keys) is the reference's second
                         benchmark workload (benchmarks/e2e.py:8-11).
  * forward_p0_seed{1,2,3}.pt - the same for the inputs of episodes 1..3 of the throughput profile
                         (actions and per-step trace only).
  * decoder_step.pt    - results of the "one decoder diffusion step" configuration (decoder
                         weights of the same checkpoint; prefix KV ~ N(0,1) and ~ N(0,0.1)),
                         from the reference's own `transformer_decoder` driven with oracle ops;
                         plus two noise floors of that step against the fp32 result: the
                         restatement of the reference's numerics, and fp32 arithmetic with only
                         the tensor-core activation operands rounded to bf16.
  * openpi_checkpoint.json - SHA-256 of all 38 tensors the reference's own OpenPI converter
                         (eval/baselines/openpi.py:129-313 `target_checkpoint`) produces from a
                         seeded synthetic full-shape state dict. `openpi` itself is absent, so its
                         `create_sinusoidal_pos_embedding` is supplied by a stub module; the one
                         tensor that depends on it (`decoder_action_fused_time_biases`) is marked
                         "unpinned" in the file.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py /path/to/reference (the flash-vla checkout)")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF / "src"))
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from oracle import pi0_ref as O  # noqa: E402
from flash_vla_b200.synthetic import bench_inputs, decoder_step_inputs, prompt_embeds  # noqa: E402
from flash_vla.hardware.nvidia.h100.pi0 import pipeline as ref_pipeline  # noqa: E402
from flash_vla.hardware.nvidia.h100.pi0.backends.tilelang.kernels import attention as ref_attention  # noqa: E402
from flash_vla.hardware.nvidia.h100.pi0.buffers import rope_table as ref_rope_table  # noqa: E402
from flash_vla.models.pi0 import random_checkpoint as ref_random_checkpoint  # noqa: E402

bf16 = torch.bfloat16
PINNED = ["vision_patch_embedding_w", "vision_position_embedding", "vision_attn_qkv_b", "vision_final_norm_w",
          "encoder_multi_modal_projector_w", "decoder_state_in_proj_w", "decoder_action_fused_time_biases",
          "decoder_action_mlp_w", "decoder_attn_qkv_w", "decoder_ffn_down_w",
          "decoder_action_fused_out_proj_w", "decoder_action_fused_out_proj_b"]


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def part_rope():
    torch.save({S: ref_rope_table(51, S, 256, "cpu") for S in (768, 816, 817)} |
               {f"enc{S}": ref_rope_table(S, 0, 256, "cpu")[::37].clone() for S in (768, 817)}, HERE / "rope.pt")


_CK = {}


def checkpoint():
    if not _CK:
        _CK["bf16"] = ref_random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cpu")
        _CK["f32"] = {k: v.float() for k, v in _CK["bf16"].items()}
    return _CK["bf16"], _CK["f32"]


def part_checkpoint():
    ck, _ = checkpoint()
    (HERE / "checkpoint.json").write_text(json.dumps(
        {"args": {"prompt_len": 0, "wscale": 0.02, "seed": 0, "device": "cpu"}, "torch": torch.__version__,
         "sha256": {k: sha(ck[k]) for k in PINNED}}, indent=1))


def part_attention():
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(1, 256, 3456, generator=g)
    Q, K, V = torch.randn(64 * 8, 256, generator=g), torch.randn(300, 256, generator=g), torch.randn(300, 256, generator=g)
    torch.save({"qkv_seed": 5, "vision_out": ref_attention.vision_attention(qkv)[:, ::8].clone(),
                "encoder_out": ref_attention.encoder_attention(Q, K, V, 256 ** -0.5).clone()}, HERE / "attention.pt")



def oracle_forward(w32, prompt_len, seed):
    """Oracle forward on the benchmark inputs of `seed`, cross-checked against the reference's own
    orchestration and attention functions driven with the oracle's ops."""
    images, state, noise = bench_inputs(seed=seed)
    w32 = dict(w32)
    w32["language_embeds"] = prompt_embeds(prompt_len)[1].float() if prompt_len else torch.zeros(0, 2048)
    trace = []
    out, b = O.forward(w32, images, state, noise, trace=trace)
    out = out.clone()
    b2, S = O.allocate_buffers(3, 50, prompt_len)
    ops = O.op_table(True, False)
    b2["observation_images_normalized"].copy_(images)
    b2["observation_state_normalized"].copy_(state)
    b2["diffusion_noise"].copy_(noise)
    b2["encoder_x"][768:].copy_(w32["language_embeds"])
    ref_pipeline.vision_encoder(ops, w32, b2, 3)
    ref_pipeline.transformer_encoder(ops, w32, b2, S)
    ref_pipeline.transformer_decoder(ops, w32, b2, S)
    replay_diff = (b2["diffusion_noise"] - out).abs().max().item()
    assert replay_diff < 1e-4, replay_diff
    return out, torch.stack(trace), replay_diff, b


def part_forward(prompts=(0, 48, 49, 256)):
    _, w32 = checkpoint()
    for prompt_len in prompts:
        out, trace, replay_diff, b = oracle_forward(w32, prompt_len, 0)
        torch.save({"actions": out, "trace": trace, "replay_max_abs_diff": replay_diff,
                    "vision_x": b["vision_x"][:, ::16, ::9].clone(), "encoder_x": b["encoder_x"][::16, ::16].clone(),
                    "encoder_K": b["encoder_K"][:, ::32, ::8].clone(), "encoder_V": b["encoder_V"][:, ::32, ::8].clone()},
                   HERE / f"forward_p{prompt_len}.pt")
        print("forward", prompt_len, "replay diff", replay_diff, "out absmax", out.abs().max().item())


def part_episodes():
    _, w32 = checkpoint()
    for seed in (1, 2, 3):
        out, trace, replay_diff, _ = oracle_forward(w32, 0, seed)
        torch.save({"actions": out, "trace": trace, "replay_max_abs_diff": replay_diff}, HERE / f"forward_p0_seed{seed}.pt")
        print("episode seed", seed, "replay diff", replay_diff)


def part_decoder_step():
    _, w32 = checkpoint()
    # one decoder step (step 0, t = 1.0) on a synthetic prefix KV; inputs are regenerated from
    # their seed by `flash_vla_b200.synthetic.decoder_step_inputs`, only results are stored
    cases = {}
    for tag, kv_scale in (("kv1", 1.0), ("kv01", 0.1)):
        K, V, st, nz = decoder_step_inputs(kv_scale)
        b, S = O.allocate_buffers(3, 50, 0)
        b["encoder_K"][:, :768] = K.float()
        b["encoder_V"][:, :768] = V.float()
        b["observation_state_normalized"].copy_(st)
        b["diffusion_noise"].copy_(nz)
        ref_pipeline.transformer_decoder(O.op_table(True, False), w32, b, 768, steps=1)
        mine, _ = O.allocate_buffers(3, 50, 0)
        mine["encoder_K"][:, :768] = K.float()
        mine["encoder_V"][:, :768] = V.float()
        mine["observation_state_normalized"].copy_(st)
        mine["diffusion_noise"].copy_(nz)
        O.transformer_decoder(O.op_table(True, False), w32, mine, 768, steps=1)
        assert (mine["diffusion_noise"] - b["diffusion_noise"]).abs().max().item() < 1e-5
        # the same step with the reference's numerics (bf16 buffers, every kernel-internal
        # rounding): its distance from the fp32 result is the noise floor of the reference itself
        fa, _ = O.allocate_buffers(3, 50, 0, bf16)
        fa["encoder_K"][:, :768] = K
        fa["encoder_V"][:, :768] = V
        fa["observation_state_normalized"].copy_(st)
        fa["diffusion_noise"].copy_(nz)
        O.transformer_decoder(O.op_table(True, True), w32, fa, 768, steps=1)
        faithful_err = (fa["diffusion_noise"].float() - b["diffusion_noise"]).abs().max().item()
        # fp32 everywhere except the activation operands a tensor core must take in bf16
        op, _ = O.allocate_buffers(3, 50, 0)
        op["encoder_K"][:, :768] = K.float()
        op["encoder_V"][:, :768] = V.float()
        op["observation_state_normalized"].copy_(st)
        op["diffusion_noise"].copy_(nz)
        O.transformer_decoder(O.op_table(True, False, True), w32, op, 768, steps=1)
        operand_err = (op["diffusion_noise"] - b["diffusion_noise"]).abs().max().item()
        cases[tag] = {"kv_scale": kv_scale, "out": b["diffusion_noise"].clone(), "decoder_x": b["decoder_x"].clone(),
                      "bf16_faithful_max_abs": faithful_err, "operand_bf16_max_abs": operand_err}
        print("decoder step", tag, "bf16-faithful restatement vs fp32: max-abs", faithful_err,
              "; bf16 operands only:", operand_err)
    torch.save(cases, HERE / "decoder_step.pt")


def part_openpi():
    """Hashes of the reference converter's output on a synthetic OpenPI state dict."""
    import types
    from flash_vla_b200.models.pi0 import openpi as mine
    stub = types.ModuleType("openpi.models_pytorch.pi0_pytorch")
    stub.create_sinusoidal_pos_embedding = (
        lambda time, dimension, min_period, max_period, device="cpu": mine.sinusoidal_time_embedding(
            time, dimension, min_period, max_period))
    for name in ("openpi", "openpi.models_pytorch"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["openpi.models_pytorch.pi0_pytorch"] = stub
    sys.path.insert(0, str(REF))
    from eval.baselines import openpi as ref_openpi

    state = mine.synthetic_openpi_state(seed=0, scale=0.02)

    class Model:
        def state_dict(self):
            return state

    out = ref_openpi.target_checkpoint(Model())
    (HERE / "openpi_checkpoint.json").write_text(json.dumps(
        {"state": {"seed": 0, "scale": 0.02, "generator": "flash_vla_b200.models.pi0.openpi.synthetic_openpi_state"},
         "torch": torch.__version__,
         "unpinned": ["decoder_action_fused_time_biases"],
         "sha256": {k: sha(v) for k, v in out.items()}}, indent=1))
    print("openpi: hashed", len(out), "tensors")


PARTS = {"rope": part_rope, "checkpoint": part_checkpoint, "attention": part_attention, "forward": part_forward,
         "episodes": part_episodes, "decoder_step": part_decoder_step, "openpi": part_openpi}


def main():
    torch.set_num_threads(os.cpu_count())
    wanted = sys.argv[2:] or list(PARTS)
    for item in wanted:                       # `forward=256` regenerates only that prompt length
        name, _, arg = item.partition("=")
        if arg:
            PARTS[name](tuple(int(v) for v in arg.split(",")))
        else:
            PARTS[name]()
    print("done")


if __name__ == "__main__":
    main()
