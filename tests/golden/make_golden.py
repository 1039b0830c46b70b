"""Generate the committed fixtures under tests/golden/ from the reference's CPU-runnable code.

Run once, in a container that has the reference checkout (it cannot travel to the GPU box):

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py /path/to/reference

What is pinned, and against what:
  * rope.pt            - the reference's own `rope_table` (buffers.py:15-23) for the three
                         prefix lengths used by the tests.
  * checkpoint.json    - SHA-256 of selected tensors of the reference's own
                         `random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cpu")`
                         (weights.py:10-24); the package's generator must reproduce them.
  * attention.pt       - the reference's own torch attention functions
                         (kernels/attention.py:20-34) on small seeded inputs.
  * forward_p{0,48,49}.pt - final actions, per-step trace and probes of the CPU fp32 oracle on
                         the benchmark inputs, after checking that driving the REFERENCE'S OWN
                         `pipeline.py` with the oracle's op table (and the reference's own
                         attention functions) gives the same result. The reference's kernels
                         cannot run on a CPU, so these vectors pin the oracle's orchestration
                         and the torch-level pieces, not the TileLang kernels: the arithmetic
                         of the GEMM/norm/RoPE ops stays "parity unpinned" by the reference.
  * decoder_step.pt    - results of the "one decoder diffusion step" configuration (decoder
                         weights of the same checkpoint; prefix KV ~ N(0,1) and ~ N(0,0.1)),
                         from the reference's own `transformer_decoder` driven with oracle ops.
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


def main():
    torch.set_num_threads(os.cpu_count())
    torch.save({S: ref_rope_table(51, S, 256, "cpu") for S in (768, 816, 817)} |
               {f"enc{S}": ref_rope_table(S, 0, 256, "cpu")[::37].clone() for S in (768, 817)}, HERE / "rope.pt")

    ck = ref_random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cpu")
    (HERE / "checkpoint.json").write_text(json.dumps(
        {"args": {"prompt_len": 0, "wscale": 0.02, "seed": 0, "device": "cpu"}, "torch": torch.__version__,
         "sha256": {k: sha(ck[k]) for k in PINNED}}, indent=1))

    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(1, 256, 3456, generator=g)
    Q, K, V = torch.randn(64 * 8, 256, generator=g), torch.randn(300, 256, generator=g), torch.randn(300, 256, generator=g)
    torch.save({"qkv_seed": 5, "vision_out": ref_attention.vision_attention(qkv)[:, ::8].clone(),
                "encoder_out": ref_attention.encoder_attention(Q, K, V, 256 ** -0.5).clone()}, HERE / "attention.pt")

    w32 = {k: v.float() for k, v in ck.items()}
    images, state, noise = bench_inputs()
    for prompt_len in (0, 48, 49):
        if prompt_len:
            w32["language_embeds"] = prompt_embeds(prompt_len)[1].float()
        trace = []
        out, b = O.forward(w32, images, state, noise, trace=trace)
        out = out.clone()
        # the reference's own orchestration and attention functions, driven with the oracle's ops
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
        torch.save({"actions": out, "trace": torch.stack(trace), "replay_max_abs_diff": replay_diff,
                    "vision_x": b["vision_x"][:, ::16, ::9].clone(), "encoder_x": b["encoder_x"][::16, ::16].clone(),
                    "encoder_K": b["encoder_K"][:, ::32, ::8].clone(), "encoder_V": b["encoder_V"][:, ::32, ::8].clone()},
                   HERE / f"forward_p{prompt_len}.pt")
        print("forward", prompt_len, "replay diff", replay_diff, "out absmax", out.abs().max().item())

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
        cases[tag] = {"kv_scale": kv_scale, "out": b["diffusion_noise"].clone(), "decoder_x": b["decoder_x"].clone(),
                      "bf16_faithful_max_abs": faithful_err}
        print("decoder step", tag, "bf16-faithful restatement vs fp32: max-abs", faithful_err)
    torch.save(cases, HERE / "decoder_step.pt")
    print("done")


if __name__ == "__main__":
    main()
