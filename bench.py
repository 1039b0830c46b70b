"""Benchmark of the Pi0 forward pass on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu]

Workload (N = 1): the full Pi0 forward at the published shape - 3 views of 224x224x3, empty
prompt, chunk 50, 10 Euler steps, 18 decoder layers, bf16, batch 1, whole pass in one CUDA
graph. A "step" is one forward. At N > 1 every GPU runs an independent replica of the same
workload on its own episode (no inter-GPU communication; weak scaling).

Reported:
  value        forwards/s over all N GPUs, inputs already resident in HBM, K graph replays timed
               with CUDA events on the launching stream, max over ranks.
  ms_per_step  milliseconds per forward (the latency figure the reference publishes).
  e2e          the same through the public API `Pi0Inference.forward` with pinned HOST inputs
               (host->device copies inside the timed region) and a device->host read of the
               action chunk every step.
  roofline     the dominant kernel class by share of the forward, the decoder's weight-streaming cluster
               GEMM (about 40 % of the step), at its largest call site: the gated FFN, 16.8 MB of weights
               per launch, HBM-bound. Timed alone inside a CUDA graph that cycles the 18 layers' distinct
               weights, so every launch reads its weights cold. roofline_encoder is the same for the
               largest single launch, the prefix encoder's gated FFN (tensor-bound).
  kernels      the same cold-in-graph timing for every GEMM of the isolated sweep configuration (decoder
               gate/up and down, encoder gate/up and down), the other two decoder GEMMs and the two
               attention kernels, each with its fraction of the measured peak.
  throughput_profile  forwards/s of the 4-episodes-per-GPU profile, measured in the same run.
  cpu_baseline the CPU fp32 oracle (a port: the reference has no CPU path) on this host's cores.
  env          GPU, driver, CUDA, torch, CPU model and core count of the run.

`--impl reference` times that CPU oracle alone, as the reference arm (and adds, as `reference_gpu`, what
`--impl reference-gpu` measures in a child process when an installed copy of the reference is present).
`--impl reference-gpu` runs the UNMODIFIED
reference itself (its TileLang kernels and engine, from an installed copy under baseline/_ref, which is not part of
this repository) on the GPU for the same metric and workload, and prints `unavailable` when that copy or TileLang
is missing; the main line carries the figure recorded when the parity fixture was made (`reference_gpu_recorded`).
`--episodes E` switches to the
throughput profile (E independent episodes per GPU inside the graph; `ms_per_step` is then the time of one
replay = E forwards); `--sweep` times the FFN GEMMs and the prefix attention alone.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

H100_PUBLISHED_MS = 15.18            # reference README.md:105-108, H100 SXM5, same shape
FORWARD_FLOPS = 4.006e12
# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) is NOT measured by this program:
# these are the figures of one ncu capture of each kernel, typed in here. The line says so
# (`traffic_source`); if a kernel changes, re-capture it.
ENC_GATE_DRAM_BYTES = 154.0e6
DEC_GATE_DRAM_BYTES = 17.03e6
TRAFFIC_SOURCE = "constant from an earlier ncu capture of this kernel (dram__bytes_read.sum + dram__bytes_write.sum, one launch); not measured by this run"


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi every 200 ms while active."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), world


def max_over_ranks(value: float, world: int) -> float:
    """Slowest rank's figure: replicas run independently, so the job is as fast as its slowest GPU."""
    if world == 1:
        return value
    import torch.distributed as dist
    device = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def job_throughput(n_replicas: int, steps: int, ms_slowest: float) -> float:
    """Forwards/s of the whole job: every replica did `steps` forwards within the slowest rank's time."""
    return n_replicas * steps / (ms_slowest / 1e3)


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


# ----------------------------------------------------------------------------- CPU oracle timing
def cpu_oracle_weights(vision_layers: int, encoder_layers: int):
    """fp32 weights for a bounded oracle run. Timing of fp32 matmuls does not depend on the
    values, so one small normal block is tiled into every tensor instead of drawing 2.7 G
    samples; only the layers the sample touches are materialised."""
    from flash_vla_b200.models.pi0.spec import weight_shapes
    base = torch.randn(1 << 20) * 0.02
    w = {}
    for name, shape in weight_shapes(0).items():
        shape = list(shape)
        if name.startswith("vision_") and len(shape) > 1 and shape[0] == 27:
            shape[0] = vision_layers
        if name.startswith("encoder_") and len(shape) > 1 and shape[0] == 18:
            shape[0] = encoder_layers
        n = 1
        for s in shape:
            n *= s
        w[name] = base.repeat((n + base.numel() - 1) // base.numel())[:n].reshape(shape).contiguous()
    return w


def env_block():
    """Where the numbers were taken: GPU, driver, CUDA, torch, host CPU (the reference stamps its runs the
    same way, benchmarks/metrics.py:122-132)."""
    env = {"torch": torch.__version__, "cuda_runtime": torch.version.cuda, "cpu_cores": os.cpu_count()}
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("model name"):
                env["cpu_model"] = line.split(":", 1)[1].strip()
                break
    except OSError:
        pass
    if torch.cuda.is_available():
        props = torch.cuda.get_device_properties(torch.cuda.current_device())
        env.update({"gpu": props.name, "sms": props.multi_processor_count, "hbm_gib": round(props.total_memory / 2 ** 30, 1),
                    "compute_capability": f"{props.major}.{props.minor}"})
        try:
            out = subprocess.run(["nvidia-smi", "--query-gpu=driver_version", "--format=csv,noheader"],
                                 capture_output=True, text=True, timeout=10).stdout.strip().splitlines()
            env["driver"] = out[0] if out else None
        except (OSError, subprocess.SubprocessError):
            pass
    try:
        out = subprocess.run(["/usr/local/cuda/bin/nvcc", "--version"], capture_output=True, text=True, timeout=10).stdout
        env["nvcc"] = next((l.split("release")[1].split(",")[0].strip() for l in out.splitlines() if "release" in l), None)
    except (OSError, subprocess.SubprocessError):
        pass
    return env


def run_oracle_sample(fraction_inv: int, weights, inputs):
    """One bounded sample: 27/f vision layers, 18/f encoder layers, ceil(10/f) decoder steps."""
    from oracle import pi0_ref as O
    images, state, noise = inputs
    vl, el = max(1, 27 // fraction_inv), max(1, 18 // fraction_inv)
    steps = max(1, -(-10 // fraction_inv))
    b, S = O.allocate_buffers(3, 50, 0)
    ops = O.op_table(True)
    b["observation_images_normalized"].copy_(images)
    b["observation_state_normalized"].copy_(state)
    b["diffusion_noise"].copy_(noise)
    t0 = time.perf_counter()
    O.vision_encoder(ops, weights, b, 3, layers=vl)
    O.transformer_encoder(ops, weights, b, S, layers=None if el == 18 else el)
    O.transformer_decoder(ops, weights, b, S, steps=steps)
    dt = time.perf_counter() - t0
    # work actually done, as a fraction of one forward (FLOPs of the three stages, 4.006 TF total)
    done = 0.657e12 * vl / 27 + 2.969e12 * el / 18 + 0.380e12 * steps / 10
    return dt, done / FORWARD_FLOPS


def time_cpu_oracle(steps: int, warmup: int, budget_s: float):
    """Forwards/s of the fp32 oracle on all host cores, from bounded samples sized to the budget."""
    from flash_vla_b200.synthetic import bench_inputs
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    inputs = bench_inputs()
    probe_w = cpu_oracle_weights(3, 2)
    t_probe, frac_probe = run_oracle_sample(9, probe_w, inputs)
    est_full = t_probe / frac_probe
    per_step_budget = budget_s / max(1, steps + warmup)
    inv = 1 if est_full <= per_step_budget else (3 if est_full / 3 <= per_step_budget else 9)
    weights = probe_w if inv == 9 else cpu_oracle_weights(max(1, 27 // inv), max(1, 18 // inv))
    for _ in range(warmup):
        run_oracle_sample(inv, weights, inputs)
    times, frac = [], None
    for _ in range(steps):
        dt, frac = run_oracle_sample(inv, weights, inputs)
        times.append(dt)
    total = sum(times)
    value = frac * steps / total
    sample = (f"{steps} x [{max(1, 27 // inv)} of 27 vision layers + {max(1, 18 // inv)} of 18 encoder layers + "
              f"{max(1, -(-10 // inv))} of 10 decoder steps] = {frac:.3f} of one forward's FLOPs per sample; "
              f"forwards/s = fraction / seconds")
    return value, total / steps, cores, sample


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    value, sec_per_sample, cores, sample = time_cpu_oracle(args.steps, args.warmup, budget_s=150.0)
    line = {
        "impl": "reference", "metric": "pi0_forwards_per_s", "value": value, "unit": "forwards/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / value,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "forwards/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "forwards/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation; this is the CPU fp32 restatement (oracle/pi0_ref.py)",
        "env": env_block(),
    }
    # Beside the CPU figure: the unmodified reference itself on this GPU, where an installed copy exists. It runs in
    # a child process with a time limit, so that whatever happens to it the line above is still printed.
    if (ROOT / "baseline" / "_ref" / "flash_vla").is_dir() and torch.cuda.is_available():
        try:
            child = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference-gpu", "--steps", str(min(args.steps, 20)),
                                    "--warmup", "3"], capture_output=True, text=True, timeout=420)
            rows = [r for r in child.stdout.splitlines() if r.startswith("{")]
            got = json.loads(rows[-1]) if rows else {"unavailable": f"no output (exit code {child.returncode})"}
        except subprocess.TimeoutExpired:
            got = {"unavailable": "the reference's GPU run did not finish within 420 s"}
        except Exception as e:
            got = {"unavailable": f"{type(e).__name__}: {e}"}
        line["reference_gpu"] = {k: got[k] for k in ("value", "unit", "ms_per_step", "e2e", "clocks", "note", "unavailable") if k in got}
    print(json.dumps(line))


def reference_gpu_recorded():
    """The reference engine's own time on a B200, recorded by tests/golden/make_reference_gpu_golden.py when the
    parity fixture was made. Not measured by this run."""
    path = ROOT / "tests" / "golden" / "reference_gpu.pt"
    if not path.exists():
        return None
    data = torch.load(path)
    if "timing" not in data:
        return None
    return {"ms_per_forward": data["timing"]["ms_per_replay"], "gpu": data["meta"]["gpu"], "tilelang": data["meta"]["tilelang"],
            "source": "recorded in tests/golden/reference_gpu.pt: one graph replay of the reference's own engine (flash_vla.Pi0Inference, "
                      "its TileLang kernels) on the same workload; not measured by this run (see --impl reference-gpu)"}


def run_reference_gpu(args):
    """The unmodified reference through its own public API, from the installed copy under baseline/_ref."""
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    ref_dir = ROOT / "baseline" / "_ref"

    def unavailable(why):
        print(json.dumps({"impl": "reference-gpu", "unavailable": why}))

    if not (ref_dir / "flash_vla").is_dir():
        return unavailable("no installed copy of the reference under baseline/_ref (pip install --no-deps --target baseline/_ref <checkout>)")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    try:
        import tilelang  # noqa: F401
    except Exception as e:      # the reference's only hard dependency besides torch
        return unavailable(f"tilelang cannot be imported: {type(e).__name__}")
    sys.path.insert(0, str(ref_dir))
    import flash_vla
    if args.sweep:
        return run_reference_gpu_sweep(args)
    from flash_vla_b200.synthetic import bench_inputs
    torch.cuda.set_device(local_rank)
    ck = flash_vla.random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cuda")
    engine = flash_vla.Pi0Inference(ck, num_views=3, chunk_size=50)
    host = [t.to(torch.bfloat16).pin_memory() for t in bench_inputs()]
    dev = [t.cuda() for t in host]
    K, W = args.steps, max(3, args.warmup)
    engine.forward(*dev)
    for _ in range(W):
        engine.graph.replay()
    with ClockSampler(local_rank) as clocks:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(K):
            engine.graph.replay()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / K
        out_host = torch.empty((50, 32), dtype=torch.bfloat16).pin_memory()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(K):
            out_host.copy_(engine.forward(*host), non_blocking=True)
            torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1000.0 / K
    line = {
        "impl": "reference-gpu", "metric": "pi0_forwards_per_s", "value": 1000.0 / ms, "unit": "forwards/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (1000.0 / ms) / (1000.0 / H100_PUBLISHED_MS), "dtype": "bf16", "data": "synthetic", "config": workload_config(1),
        "e2e": {"value": 1000.0 / e2e_ms, "unit": "forwards/s", "ms_per_forward": e2e_ms,
                "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host), "d2h_bytes_per_step": out_host.numel() * 2},
        "clocks": clocks.summary(),
        "note": "the unmodified reference (flash_vla.Pi0Inference, TileLang kernels) from baseline/_ref on this GPU; its two torch "
                "attention functions " + ("run eagerly (TORCHDYNAMO_DISABLE is set)" if os.environ.get("TORCHDYNAMO_DISABLE") else "are compiled by torch.compile, as shipped"),
        "env": env_block(),
    }
    print(json.dumps(line))


def run_reference_gpu_sweep(args):
    """The isolated-kernel sweep of `sweep_rows` through the REFERENCE's op table (and its two torch attention
    functions): the same call sites, shapes and cold-weight method, for a per-kernel comparison on this GPU."""
    names = [args.sweep_only] if args.sweep_only else list(SWEEP)
    rows = sweep_rows(names, args.sweep_layers, args.sweep_reps, reference=True)
    print(json.dumps({"impl": "reference-gpu", "metric": "isolated_kernels", "kernels": rows,
                      "note": "the reference's TileLang wrappers (fused table) and torch attention functions on this GPU, bf16 buffers throughout"}))


def workload_config(n_gpus: int, episodes: int = 1):
    return {"workload": "Pi0 full forward: 3 views 224x224x3, empty prompt (prefix 768), chunk 50, 10 Euler steps, "
                        "27 SigLIP + 18 prefix + 18 decoder layers, batch 1, one CUDA graph" +
                        ("" if episodes == 1 else f"; {episodes} independent episodes per GPU inside the graph (vision, prefix encoder "
                                                  f"and decoder batched over the episodes)"),
            "weights": "random_checkpoint N(0, 0.02) bf16, 2.709 G params",
            "replicas": n_gpus, "episodes_per_gpu": episodes, "parallelism": f"replicas x{n_gpus} (no collective)",
            "l2": "each step streams 5.4 GB of weights, far more than the 126 MB L2; no explicit flush"}


# ----------------------------------------------------------------------------- GPU arm
def time_isolated_op(fn, layers: int, reps: int):
    """Average device time (ms) of one call of `fn(layer)`, cycled over distinct layer weights so
    every call reads its weights cold; the loop is captured in a CUDA graph so that host launch
    gaps do not enter the figure (the reference's method, benchmarks/metrics.py:55-85)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for layer in range(layers):
            fn(layer)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for layer in range(layers):
            fn(layer)
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / (reps * layers)


def measure_throughput_profile(weights, rank, world, n_gpus, K, W, episodes=4):
    """Forwards/s with `episodes` independent episodes per GPU inside one captured pass (the throughput
    configuration: same shapes, one replica per GPU, no inter-GPU communication)."""
    from flash_vla_b200 import Pi0Inference
    from flash_vla_b200.synthetic import bench_inputs
    ck = dict(weights)
    engine = Pi0Inference(ck, num_views=3, chunk_size=50, episodes=episodes)
    sets = [bench_inputs(seed=rank * episodes + e) for e in range(episodes)]
    images, state, noise = [torch.stack([s[i] for s in sets]).to(torch.bfloat16).cuda() for i in range(3)]
    stream = torch.cuda.current_stream()
    engine.forward(images, state, noise)
    for _ in range(W):
        engine.graph.replay()
    barrier(world)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(K):
        engine.graph.replay()
    end.record(stream)
    torch.cuda.synchronize()
    ms = max_over_ranks(start.elapsed_time(end), world)
    barrier(world)
    del engine
    torch.cuda.empty_cache()
    return {"episodes_per_gpu": episodes, "value": job_throughput(n_gpus * episodes, K, ms), "unit": "forwards/s",
            "ms_per_replay": ms / K, "form": engine_form(episodes)}


def engine_form(episodes):
    return (f"{episodes} episodes per captured pass: SigLIP, the prefix encoder (M = {episodes} x 768) and the action-expert decoder "
            f"(M = {episodes} x 51) each run once over all episodes' rows; attention per episode; shared weights")


def run_ours(args):
    rank, local_rank, world = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from flash_vla_b200 import Pi0Inference, random_checkpoint
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib, wrappers
    from flash_vla_b200.synthetic import bench_inputs

    lib = _lib.load()
    ck = random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cuda")
    launches_before = lib.fvla_launch_count()
    E = max(1, args.episodes)
    engine = Pi0Inference(ck, num_views=3, chunk_size=50, episodes=E)
    per_forward = (lib.fvla_launch_count() - launches_before) // (4 * E)       # 3 warm-up passes + 1 captured, E episodes each
    del ck
    if E == 1:
        images, state, noise = [t.to(torch.bfloat16).pin_memory() for t in bench_inputs(seed=rank)]
    else:       # one input set per episode, seeds rank * E + e
        sets = [bench_inputs(seed=rank * E + e) for e in range(E)]
        images, state, noise = [torch.stack([s[i] for s in sets]).to(torch.bfloat16).pin_memory() for i in range(3)]
    host_out = torch.empty((50, 32) if E == 1 else (E, 50, 32), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream()

    K, W = args.steps, max(3, args.warmup)
    with ClockSampler(local_rank) as clocks:
        # resident inputs: replay only
        engine.forward(images, state, noise)
        for _ in range(W):
            engine.graph.replay()
        barrier(world)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(K):
            engine.graph.replay()
        end.record(stream)
        torch.cuda.synchronize()
        ms_total = max_over_ranks(start.elapsed_time(end), world)
        barrier(world)

        # end to end through the public API, host buffers in and out, one sync per forward
        for _ in range(W):
            host_out.copy_(engine.forward(images, state, noise), non_blocking=True)
            stream.synchronize()
        barrier(world)
        start.record(stream)
        for _ in range(K):
            host_out.copy_(engine.forward(images, state, noise), non_blocking=True)
            stream.synchronize()
        end.record(stream)
        torch.cuda.synchronize()
        ms_e2e = max_over_ranks(start.elapsed_time(end), world)
        barrier(world)
    clock_summary = clocks.summary()

    peaks = measured_peaks()
    line = {
        "metric": "pi0_forwards_per_s", "value": job_throughput(args.gpus * E, K, ms_total), "unit": "forwards/s",
        "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus, E),
        "e2e": {"value": job_throughput(args.gpus * E, K, ms_e2e), "unit": "forwards/s", "ms_per_forward": ms_e2e / K / E,
                "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in (images, state, noise)),
                "d2h_bytes_per_step": host_out.numel() * host_out.element_size()},
        "gpu_launches": int(per_forward * K * E), "gpu_launches_per_forward": int(per_forward),
        "tuned_plans": int(engine.tuned_plans),
        "clocks": clock_summary,
        "published_h100_ms_per_forward": H100_PUBLISHED_MS,
    }
    if args.gpus == 1 and E == 1:
        # the published figure is ms/forward on one H100; express it in this line's unit
        line["vs_baseline"] = line["value"] / (1000.0 / H100_PUBLISHED_MS)

    # the 4-episodes-per-GPU throughput profile, in the same run and at every N
    if E == 1 and not args.no_throughput_profile:
        line["throughput_profile"] = measure_throughput_profile(engine.weights, rank, world, args.gpus, K, W)
    del engine
    torch.cuda.empty_cache()

    if rank == 0 and args.gpus == 1 and E == 1:
        rows = sweep_rows(list(SWEEP), layers_cap=0, reps=10)
        line["kernels"] = rows
        dg, eg = rows["dec_gate"], rows["enc_gate"]
        line["roofline"] = {"kernel": "skinny_gemm_kernel (decoder cluster GEMM) at decoder_norm_gated_ffn: M=51 K=1024 N=2x4096, "
                                      "16.8 MB of weights per launch; this kernel class is about 40 % of the forward",
                            "bound": "hbm", "achieved": dg["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": dg["gbs"] / peaks["hbm_gbs"], "traffic": DEC_GATE_DRAM_BYTES,
                            "traffic_unit": "bytes per launch", "traffic_source": TRAFFIC_SOURCE,
                            "peak_source": peaks["source"], "ms_per_launch": dg["ms_per_launch"],
                            "algorithmic_bytes": dg["algorithmic_bytes"],
                            "note": "18 layers' weights cycled inside one CUDA graph, CUDA events around the replays"}
        line["roofline_encoder"] = {"kernel": "encoder_norm_gated_ffn (RMS norm kernel + two-SM tcgen05 gate/up GEMM with GeGLU epilogue, "
                                              "M=768 K=2048 N=2x16384); the largest single launch, about 13 % of the forward",
                                    "bound": "tensor", "achieved": eg["tflops"], "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                    "frac": eg["tflops"] / peaks["bf16_tflops"], "traffic": ENC_GATE_DRAM_BYTES,
                                    "traffic_unit": "bytes per launch", "traffic_source": TRAFFIC_SOURCE,
                                    "peak_source": peaks["source"] + " burst", "ms_per_launch": eg["ms_per_launch"]}
        if not args.no_cpu_baseline:
            value, _, cores, sample = time_cpu_oracle(3, 1, budget_s=30.0)
            line["cpu_baseline"] = {"value": value, "unit": "forwards/s", "cores": cores, "kind": "port", "sample": sample}
    line["env"] = env_block()
    recorded = reference_gpu_recorded()
    if recorded is not None and E == 1:
        line["reference_gpu_recorded"] = recorded
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


SWEEP = {   # name: (M, K, N, gated, residual, layers cycled)
    "dec_qkv": (51, 1024, 2560, False, False, 18),
    "dec_o": (51, 2048, 1024, False, True, 18),
    "dec_gate": (51, 1024, 4096, True, False, 18),
    "dec_down": (51, 4096, 1024, False, True, 18),
    "enc_gate": (768, 2048, 16384, True, False, 6),
    "enc_down": (768, 16384, 2048, False, True, 6),
    "enc_attn": (768 * 8, 256, 768, False, False, 6),     # prefix attention: flat queries, head dim, keys
    "dec_attn": (51 * 8, 256, 819, False, False, 18),     # decoder attention: flat queries, head dim, keys (768 prefix + 51)
    # the remaining call sites of the M = 768 stages (row norm kernel included where the op has one)
    "enc_qkv": (768, 2048, 2560, False, False, 9),
    "enc_o": (768, 2048, 2048, False, True, 9),
    "vis_qkv": (768, 1152, 3456, False, False, 9),
    "vis_attn": (3 * 16 * 256, 72, 256, False, False, 9), # SigLIP attention: views x heads x queries, head dim, keys
    "vis_o": (768, 1152, 1152, False, True, 9),
    "vis_up": (768, 1152, 4304, False, False, 9),
    "vis_down": (768, 4304, 1152, False, True, 9),
}


def sweep_rows(names, layers_cap: int, reps: int, fused: bool = True, reference: bool = False):
    """Isolated kernel timings: bf16 weights ~ N(0, 0.02), activations ~ N(0, 1), fp32 accumulate, distinct
    weight copies cycled inside one CUDA graph so every launch streams its weights cold. Returns
    {name: {ms_per_launch, tflops, gbs, algorithmic_bytes, flops, frac_of_hbm, frac_of_bf16, ...}}."""
    if reference:       # the reference's own table (bf16 buffers only; attention for SigLIP and the prefix is plain torch there)
        from types import SimpleNamespace
        from flash_vla.hardware.nvidia.h100.pi0.backends.tilelang import wrappers
        from flash_vla.hardware.nvidia.h100.pi0.backends.tilelang.kernels import attention as ref_attention
        from flash_vla.hardware.nvidia.h100.pi0.buffers import rope_table
        from flash_vla.hardware.nvidia.h100.pi0.ops import op_table
        from flash_vla.runtime.cuda import ScratchPool
        table = op_table(True)
        ops = SimpleNamespace(**vars(table))
        ops.encoder_attention = lambda Q, K, V, scale, out: out.view(-1, 2048).copy_(ref_attention.encoder_attention(Q, K, V, scale))
        ops.vision_attention = lambda QKV, out: out.copy_(ref_attention.vision_attention(QKV))
    else:
        from flash_vla_b200 import op_table
        from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import wrappers
        from flash_vla_b200.hardware.nvidia.b200.pi0.buffers import rope_table
        from flash_vla_b200.runtime.cuda import ScratchPool
        ops = op_table(fused)
    peaks, bf16 = measured_peaks(), torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(0)
    rows = {}

    def row(ms, flops, nbytes, **shape):
        return {**shape, "ms_per_launch": ms, "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6,
                "algorithmic_bytes": nbytes, "flops": flops, "frac_of_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                "frac_of_bf16": flops / ms / 1e9 / peaks["bf16_tflops"]}

    with wrappers.use_pool(ScratchPool()):
        for name in names:
            M, K, N, gated, residual, layers = SWEEP[name]
            layers = min(layers, layers_cap) if layers_cap else layers
            if name in ("enc_attn", "dec_attn"):
                scale = 1.0 if name == "enc_attn" else 0.1
                q = [torch.randn(M, K, device="cuda", generator=g).to(bf16) for _ in range(layers)]
                kv = [(torch.randn(2, N, K, device="cuda", generator=g) * scale).to(bf16) for _ in range(layers)]
                o = torch.zeros(M, K, device="cuda", dtype=bf16)
                if name == "enc_attn":
                    fn = lambda i: ops.encoder_attention(q[i], kv[i][0], kv[i][1], K ** -0.5, o)
                else:
                    scores = torch.zeros(M, N, device="cuda", dtype=bf16)
                    fn = lambda i: ops.decoder_attention(q[i], kv[i][0], kv[i][1], scores, o, N - 51)
                ms = time_isolated_op(fn, layers, reps)
                rows[name] = row(ms, 4.0 * M * N * K, 2 * (2 * M * K + 2 * N * K), queries=M, keys=N, head_dim=K)
                continue
            if name == "vis_attn":
                qkv = [torch.randn(3, 256, 3 * 1152, device="cuda", generator=g).to(bf16) for _ in range(layers)]
                o = torch.zeros(3, 256, 1152, device="cuda", dtype=bf16)
                ms = time_isolated_op(lambda i: ops.vision_attention(qkv[i], o), layers, reps)
                rows[name] = row(ms, 4.0 * M * N * K, 2 * 4 * 768 * 1152, queries=M, keys=N, head_dim=K)
                continue
            w = [(torch.randn(K, N, device="cuda", generator=g) * 0.02).to(bf16) for _ in range(layers * (2 if gated else 1))]
            if name.startswith(("vis_", "enc_qkv", "enc_o")):
                x = torch.randn(M, K, device="cuda", generator=g).to(bf16)
                bias = (torch.randn(N, device="cuda", generator=g) * 0.02).to(bf16)
                nw = torch.ones(K, device="cuda", dtype=bf16)
                nb = torch.zeros(K, device="cuda", dtype=bf16)
                xn = torch.zeros(M, K, device="cuda", dtype=bf16)
                out = torch.zeros(M, N, device="cuda", dtype=bf16)
                if name == "enc_qkv":
                    rope = rope_table(M, 0, 256, "cuda")
                    Q = torch.zeros(M * 8, 256, device="cuda", dtype=bf16)
                    Kc, Vc = torch.zeros(M, 256, device="cuda", dtype=bf16), torch.zeros(M, 256, device="cuda", dtype=bf16)
                    fn = lambda i: ops.encoder_norm_qkv_rope(x, w[i], rope, Q, Kc, Vc, xn)
                elif name == "enc_o":
                    fn = lambda i: ops.encoder_out_proj_residual(x, w[i], out)
                elif name == "vis_qkv":
                    fn = lambda i: ops.vision_norm_qkv(x.view(3, 256, K), nw, nb, w[i], bias, out.view(3, 256, N), xn.view(3, 256, K))
                elif name == "vis_up":
                    fn = lambda i: ops.vision_norm_ffn_up(x.view(3, 256, K), nw, nb, w[i], bias, out.view(3, 256, N), xn.view(3, 256, K))
                elif name == "vis_o":     # out = x @ W + b + out, in place
                    fn = lambda i: ops.vision_out_proj_residual(x.view(3, 256, K), w[i], bias, out.view(3, 256, N), out.view(3, 256, N))
                else:
                    fn = lambda i: ops.vision_ffn_down_residual(x.view(3, 256, K), w[i], bias, out.view(3, 256, N), out.view(3, 256, N))
                ms = time_isolated_op(fn, layers, reps)
                nbytes = K * N * 2 + M * K * 2 + M * N * 2 * (2 if residual else 1)
                rows[name] = row(ms, 2.0 * M * K * N, nbytes, M=M, K=K, N=N)
                del w
                torch.cuda.empty_cache()
                continue
            x32 = torch.randn(M, K, device="cuda", generator=g)
            f32_in = name in ("dec_gate", "dec_qkv") and not reference   # the decoder's residual stream is fp32 ...
            f32_out = name in ("dec_down", "dec_o") and not reference
            x = x32 if f32_in else x32.to(bf16)
            if f32_in:                                                 # ... with a bf16 shadow its GEMMs read, as in the engine
                shadow = torch.zeros(M, K, device="cuda", dtype=bf16)
                wrappers.register_bf16_shadow(x, shadow)
            out = torch.zeros(M, N, device="cuda", dtype=torch.float32 if f32_out else bf16)
            if f32_out:
                wrappers.register_bf16_shadow(out, torch.zeros(M, N, device="cuda", dtype=bf16))
            xn = torch.zeros(M, K, device="cuda", dtype=bf16)
            if name == "dec_gate":
                nfg = torch.zeros(M, device="cuda", dtype=bf16) if reference else None
                fn = lambda i: ops.decoder_norm_gated_ffn(x, w[2 * i], w[2 * i + 1], out, nfg)
            elif name == "enc_gate":
                fn = lambda i: ops.encoder_norm_gated_ffn(x, w[2 * i], w[2 * i + 1], out, xn)
            elif name in ("dec_down", "dec_o"):
                fn = lambda i: ops.decoder_ffn_down_residual(x, w[i], out)
            elif name == "dec_qkv":
                rope = rope_table(M, 768, 256, "cuda")
                Q = torch.zeros(M * 8, 256, device="cuda", dtype=bf16)
                Kc, Vc = torch.zeros(M, 256, device="cuda", dtype=bf16), torch.zeros(M, 256, device="cuda", dtype=bf16)
                nf = torch.zeros(M, device="cuda", dtype=bf16)
                fn = lambda i: ops.decoder_norm_qkv_rope(x, w[i], rope, Q, Kc, Vc, nf)
            else:
                fn = lambda i: ops.encoder_ffn_down_residual(x, w[i], out)
            ms = time_isolated_op(fn, layers, reps)
            flops = 2.0 * M * K * N * (2 if gated else 1)
            # weights once + the activation operand as the kernel reads it (bf16) + the output (read and written for a residual)
            nbytes = K * N * 2 * (2 if gated else 1) + M * K * 2 + M * N * out.element_size() * (2 if residual else 1)
            rows[name] = row(ms, flops, nbytes, M=M, K=K, N=N)
            del w
            torch.cuda.empty_cache()
    return rows


def run_sweep(args):
    """Isolated kernel roofline sweep: one JSON line with HBM GB/s and TFLOP/s against the measured peaks."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --sweep needs a CUDA device")
    names = [args.sweep_only] if args.sweep_only else list(SWEEP)
    rows = sweep_rows(names, args.sweep_layers, args.sweep_reps, fused=not args.sweep_unfused)
    print(json.dumps({"metric": "isolated_gemm_roofline", "peaks": measured_peaks(), "kernels": rows,
                      "note": "fractions are of the measured copy bandwidth and measured cuBLAS bf16 burst rate"}))


def run_profile_pass():
    """Two eager (uncaptured) forwards and nothing else: the command to put under a profiler, e.g.
    `ncu --metrics gpu__time_duration.sum --clock-control none -s <launches of pass 1> -c <same> ...`."""
    from flash_vla_b200 import Pi0Inference, random_checkpoint
    from flash_vla_b200.synthetic import bench_inputs
    engine = Pi0Inference(random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cuda"), 3, 50, capture=False)
    images, state, noise = [t.cuda() for t in bench_inputs()]
    for _ in range(2):
        out = engine.forward(images, state, noise)
    torch.cuda.synchronize()
    print(json.dumps({"profile_pass": "ok", "max_abs_action": float(out.float().abs().max())}))


def main():
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=30)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", choices=["ours", "reference", "reference-gpu"], default="ours")
    p.add_argument("--episodes", type=int, default=1,
                   help="independent episodes per GPU inside the graph (throughput profile; the default 1 is the headline workload)")
    p.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle leg (faster iteration)")
    p.add_argument("--no-throughput-profile", action="store_true", help="skip the 4-episodes-per-GPU measurement")
    p.add_argument("--sweep", action="store_true", help="isolated GEMM roofline sweep instead of the forward pass")
    p.add_argument("--sweep-only", choices=list(SWEEP), default=None)
    p.add_argument("--sweep-layers", type=int, default=0, help="cap on distinct weight copies (small profiler runs)")
    p.add_argument("--sweep-reps", type=int, default=20)
    p.add_argument("--sweep-unfused", action="store_true",
                   help="sweep the unfused op table (row norm as a kernel of its own in front of the prefix GEMMs)")
    p.add_argument("--profile-pass", action="store_true", help="two eager forwards only (for ncu launch lists)")
    p.add_argument("--autotune", action="store_true",
                   help="sweep the launch plans of every GEMM call site and write the winners to the tuned-plan file")
    p.add_argument("--autotune-sites", default="", help="comma-separated call sites (default: all)")
    args = p.parse_args()
    if args.autotune:
        from flash_vla_b200.hardware.nvidia.b200.pi0 import autotune
        table = autotune.tune([x for x in args.autotune_sites.split(",") if x] or None, reps=args.sweep_reps)
        autotune.save_plans(table)
        print(json.dumps({"metric": "autotune", "plans": table["plans"], "report": table["report"]}))
    elif args.profile_pass:
        run_profile_pass()
    elif args.sweep and args.impl == "reference-gpu":
        run_reference_gpu(args)
    elif args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
