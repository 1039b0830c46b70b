"""Generate tests/golden/reference_gpu.pt by running the REFERENCE ITSELF on a CUDA GPU: its TileLang
kernels, its op table, its pipeline and its engine, unmodified, from an installed copy of the package.

    python tests/golden/make_reference_gpu_golden.py <dir holding the installed `flash_vla` package> <output.pt> [part ...]

    (install: python -m pip install --no-deps --target <dir> <reference checkout>; the installed copy is not part
     of this repository. The reference pins tilelang 0.1.11 for Hopper; its kernels also compile and run with
     tilelang 0.1.9 on a B200, which is how the committed fixture was made; the fixture records both versions.)

Parts (default: forward decoder_step ops): forward decoder_step ops prompts episodes.

What the fixture pins, all of it output of the reference's own GPU code on seeded inputs that the tests
regenerate (`flash_vla_b200.synthetic`, `tests/reference_cases.py`):
  * forward       - `flash_vla.Pi0Inference(checkpoint, 3, 50).forward(images, state, noise)` on the benchmark
                    checkpoint (seed 0, scale 0.02, no prompt; drawn by the reference's own generator on the CPU)
                    and inputs: final actions, the same strided probes of vision_x / encoder_x / encoder_K /
                    encoder_V the oracle fixtures hold. Only the reference's fused op table (its engine's default) is
                    run: with its unfused table the first attempt on a B200 made no progress for 17 minutes after the
                    kernels had compiled and was ended by its time limit, so that table stays off the GPU.
  * episodes      - the forward on the inputs of episodes 1 and 2 of the throughput profile (`bench_inputs(seed)`),
                    final actions only.
  * prompts       - the same forward with a prompt of 48, 49 and 256 tokens (prefix 816, 817 and 1024, the last being the
                    reference's other benchmark workload, benchmarks/e2e.py:8-11): `language_embeds` are the rows
                    `flash_vla_b200.synthetic.prompt_embeds` draws, as in the oracle's fixtures.
  * decoder_step  - the "one decoder diffusion step" configuration (prefix K/V ~ N(0,1) and N(0,0.1)) through the
                    reference's `transformer_decoder(steps=1)`, fused table.
  * ops           - every call-site wrapper of the reference's (fused) op table on the inputs of
                    `tests/reference_cases.py`: a strided sample of each output.
  (with the forward: milliseconds per graph replay of the reference engine on this GPU, for information.)
"""
from __future__ import annotations

import os
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
if len(sys.argv) < 3:
    raise SystemExit(__doc__)
sys.path.insert(0, str(Path(sys.argv[1]).resolve()))
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
OUT = Path(sys.argv[2])
PARTS = sys.argv[3:] or ["forward", "decoder_step", "ops"]

import torch  # noqa: E402
import tilelang  # noqa: E402

import flash_vla  # noqa: E402  (the reference)
from flash_vla.hardware.nvidia.h100.pi0 import pipeline as ref_pipeline  # noqa: E402
from flash_vla.hardware.nvidia.h100.pi0.backends.tilelang import wrappers as ref_wrappers  # noqa: E402
from flash_vla.hardware.nvidia.h100.pi0.buffers import allocate_static_buffers as ref_allocate  # noqa: E402
from flash_vla.hardware.nvidia.h100.pi0.ops import op_table as ref_op_table  # noqa: E402
from flash_vla.runtime.cuda import ScratchPool as RefScratchPool  # noqa: E402

from flash_vla_b200.synthetic import bench_inputs, decoder_step_inputs, prompt_embeds  # noqa: E402

bf16 = torch.bfloat16
result = {"meta": {"tilelang": tilelang.__version__, "torch": str(torch.__version__), "gpu": torch.cuda.get_device_name(0),
                   "reference_pins_tilelang": "0.1.11"}}
if OUT.exists():
    result.update(torch.load(OUT))
    result["meta"].update({"tilelang": tilelang.__version__, "gpu": torch.cuda.get_device_name(0)})

_ck = None
PROMPTS = tuple(int(x) for x in os.environ.get("REFERENCE_PROMPTS", "48,49,256").split(","))


def save():
    """The reference's outputs are bf16 values: stored as bf16, which loses nothing and halves the file."""
    def pack(o):
        if torch.is_tensor(o):
            return o.to(bf16)
        return {k: pack(v) for k, v in o.items()} if isinstance(o, dict) else o
    torch.save(pack(result), OUT)


def checkpoint():
    """The benchmark checkpoint from the reference's own generator (CPU draw: CPU and CUDA generators differ)."""
    global _ck
    if _ck is None:
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        cpu = flash_vla.random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cpu")
        _ck = {k: v.cuda() for k, v in cpu.items()}
    return _ck


def probes(b):
    return {"vision_x": b["vision_x"][:, ::16, ::9].float().cpu().clone(), "encoder_x": b["encoder_x"][::16, ::16].float().cpu().clone(),
            "encoder_K": b["encoder_K"][:, ::32, ::8].float().cpu().clone(), "encoder_V": b["encoder_V"][:, ::32, ::8].float().cpu().clone()}


def part_forward():
    images, state, noise = [t.cuda() for t in bench_inputs()]
    for fused in (True,):
        t0 = time.time()
        engine = flash_vla.Pi0Inference(checkpoint(), num_views=3, chunk_size=50, fused=fused)
        out = engine.forward(images.to(bf16), state.to(bf16), noise.to(bf16)).float().cpu().clone()
        out2 = engine.forward(images.to(bf16), state.to(bf16), noise.to(bf16)).float().cpu().clone()
        torch.cuda.synchronize()
        entry = {"actions": out, "replay_identical": bool(torch.equal(out, out2)), **probes(engine.buffers)}
        if fused:
            for _ in range(5):
                engine.graph.replay()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(20):
                engine.graph.replay()
            e.record()
            torch.cuda.synchronize()
            result["timing"] = {"ms_per_replay": s.elapsed_time(e) / 20, "what": "reference engine, one CUDA graph, 3 views, empty prompt, chunk 50, 10 steps"}
            print("reference engine ms per replay", result["timing"]["ms_per_replay"], flush=True)
        result["forward_fused" if fused else "forward_unfused"] = entry
        save()
        print(f"forward fused={fused}: {time.time() - t0:.0f}s, |a| max {out.abs().max().item():.4g}, replays identical {entry['replay_identical']}", flush=True)
        del engine
        torch.cuda.empty_cache()


def part_prompts():
    images, state, noise = [t.cuda().to(bf16) for t in bench_inputs()]
    for prompt_len in PROMPTS:
        t0 = time.time()
        ck = dict(checkpoint())
        ck["language_embeds"] = prompt_embeds(prompt_len)[1].cuda()
        engine = flash_vla.Pi0Inference(ck, num_views=3, chunk_size=50)
        out = engine.forward(images, state, noise).float().cpu().clone()
        torch.cuda.synchronize()
        entry = {"actions": out, **probes(engine.buffers)}
        for _ in range(5):
            engine.graph.replay()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(20):
            engine.graph.replay()
        e.record()
        torch.cuda.synchronize()
        entry["ms_per_replay"] = s.elapsed_time(e) / 20
        result[f"forward_fused_p{prompt_len}"] = entry
        save()
        print(f"forward prompt {prompt_len}: {time.time() - t0:.0f}s, {entry['ms_per_replay']:.2f} ms per replay, |a| max {out.abs().max().item():.4g}", flush=True)
        del engine
        torch.cuda.empty_cache()


def part_episodes():
    engine = flash_vla.Pi0Inference(checkpoint(), num_views=3, chunk_size=50)
    for seed in (1, 2):
        images, state, noise = [t.cuda().to(bf16) for t in bench_inputs(seed=seed)]
        out = engine.forward(images, state, noise).float().cpu().clone()
        torch.cuda.synchronize()
        result[f"forward_fused_seed{seed}"] = {"actions": out}
        save()
        print(f"forward seed {seed}: |a| max {out.abs().max().item():.4g}", flush=True)
    del engine
    torch.cuda.empty_cache()


def part_decoder_step():
    w = checkpoint()
    cases = {}
    for tag, kv_scale in (("kv1", 1.0), ("kv01", 0.1)):
        for fused in (True,):
            K, V, st, nz = decoder_step_inputs(kv_scale)
            b, S = ref_allocate(3, 50, 0, "cuda")
            b["encoder_K"][:, :768].copy_(K)
            b["encoder_V"][:, :768].copy_(V)
            b["observation_state_normalized"].copy_(st)
            b["diffusion_noise"].copy_(nz)
            with ref_wrappers.use_pool(RefScratchPool()):
                ref_pipeline.transformer_decoder(ref_op_table(fused), w, b, S, steps=1)
            torch.cuda.synchronize()
            cases[f"{tag}_{'fused' if fused else 'unfused'}"] = {
                "kv_scale": kv_scale, "out": b["diffusion_noise"].float().cpu().clone(), "decoder_x": b["decoder_x"].float().cpu().clone()}
            print("decoder step", tag, "fused" if fused else "unfused", "|out| max", b["diffusion_noise"].float().abs().max().item(), flush=True)
    result["decoder_step"] = cases


def part_ops():
    import reference_cases as RC
    samples = {}
    for fused in (True,):
        ops = ref_op_table(fused)
        for case in RC.CASES:
            if case.fused_only and not fused:
                continue
            t0 = time.time()
            tensors = case.inputs()
            with ref_wrappers.use_pool(RefScratchPool()):
                outs = case.run(ops, {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in tensors.items()}, reference=True)
            torch.cuda.synchronize()
            key = f"{case.name}/{'fused' if fused else 'unfused'}"
            samples[key] = {name: RC.sample(t.float().cpu()) for name, t in outs.items()}
            print(f"op {key}: {time.time() - t0:.1f}s " + ", ".join(f"{n} {tuple(t.shape)}" for n, t in outs.items()), flush=True)
            result["ops"] = samples
            save()


def main():
    for part in PARTS:
        globals()["part_" + part]()
        save()
    save()
    print("wrote", OUT, {k: (list(v.keys()) if isinstance(v, dict) else v) for k, v in result.items() if k != "ops"})


if __name__ == "__main__":
    main()
