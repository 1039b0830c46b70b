"""Per-call-site launch-plan sweep for the CUDA backend, at the real shapes.

Counterpart of the reference's sweeper (`benchmarks/autotune.py:34-100`: every tiling x
warp-specialisation variant of one TileLang kernel is compiled, checked and timed cold inside a CUDA
graph, fastest first) and of its timer (`benchmarks/metrics.py:55-85`, `graph_time_cold`). The B200
kernels are compiled once; what varies per GEMM call site is the launch plan: kernel family (one-SM
tcgen05 kernel, two-SM kernel, decoder cluster GEMM), tile width, K split and where the split is reduced
(global scratch or a thread-block cluster). The library picks these from cost models; this module measures
them instead:

    sweep(site)        time every candidate plan of one call site, fastest first, dropping candidates the
                       library refuses or whose result differs from the default plan's
    tune(sites)        sweep several sites, keep the winners that beat the default by a margin
    save_plans / load_plans / apply_plans
                       winners as a JSON table, pinned at run time through fvla_gemm_plan_set

    python -m flash_vla_b200.hardware.nvidia.b200.pi0.autotune [--out plans.json] [--sites a,b] [--reps N]

`Pi0Inference` applies `tuned_plans_b200.json` (next to this file) at construction when it exists.
Timing cycles distinct weight copies inside one CUDA graph so that every launch reads its weights cold
and no host launch gap enters the figure.
"""
from __future__ import annotations

import argparse
import itertools
import json
import statistics
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

import torch

KIND = {"plain": 0, "rope": 1, "dual": 2, "skinny": 3, "skinny_dual": 4}
ENGINE = {"auto": 0, "tc5_scratch": 1, "tc5_cluster": 2, "pair": 3, "skinny": 4}
ENGINE_NAME = {v: k for k, v in ENGINE.items()}
DEFAULT_PLAN_FILE = Path(__file__).with_name("tuned_plans_b200.json")
bf16 = torch.bfloat16


def grid(**axes) -> list[dict]:
    """Cartesian product of named axes: grid(bn=[128, 256], splits=[1, 2])."""
    keys = list(axes)
    return [dict(zip(keys, values)) for values in itertools.product(*[axes[k] for k in keys])]


def graph_time_cold(invoke: Callable[[int], object], n_inner: int, reps: int = 20, warmup: int = 2) -> float:
    """Median microseconds per call of `invoke(i)`, i cycling over `n_inner` distinct input sets inside one
    captured graph (cold weight reads, no host launch overhead)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(min(warmup, n_inner)):
            invoke(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(n_inner):
            invoke(i)
    torch.cuda.synchronize()
    samples = []
    for _ in range(reps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        samples.append(start.elapsed_time(end) / n_inner * 1000.0)
    return statistics.median(samples)


@dataclass
class CallSite:
    """One GEMM call site of the forward pass: its plan key and how to launch it on synthetic operands."""
    name: str
    M: int
    N: int
    K: int
    kind: str
    layers: int                      # distinct weight copies to cycle (enough to exceed L2 where it matters)

    def key(self) -> tuple[int, int, int, int]:
        return self.M, self.N, self.K, KIND[self.kind]


# The GEMM call sites of the benchmark configuration (3 views, empty prompt: M = 768 and M = 51 / 50).
SITES = {s.name: s for s in (
    CallSite("vis_qkv", 768, 3456, 1152, "plain", 9), CallSite("vis_o", 768, 1152, 1152, "plain", 9),
    CallSite("vis_up", 768, 4304, 1152, "plain", 9), CallSite("vis_down", 768, 1152, 4304, "plain", 9),
    CallSite("enc_projector", 768, 2048, 1152, "plain", 9), CallSite("enc_o", 768, 2048, 2048, "plain", 9),
    CallSite("enc_down", 768, 2048, 16384, "plain", 6), CallSite("enc_gate", 768, 16384, 2048, "dual", 6),
    CallSite("dec_qkv", 51, 2560, 1024, "skinny", 18), CallSite("dec_o", 51, 1024, 2048, "skinny", 18),
    CallSite("dec_gate", 51, 4096, 1024, "skinny_dual", 18), CallSite("dec_down", 51, 1024, 4096, "skinny", 18),
    CallSite("dec_action_mlp", 50, 1024, 1024, "skinny", 18),
    # the same M = 768 sites in the 4-episode throughput plan (M = 3072)
    CallSite("vis_qkv_x4", 3072, 3456, 1152, "plain", 6), CallSite("vis_o_x4", 3072, 1152, 1152, "plain", 6),
    CallSite("vis_up_x4", 3072, 4304, 1152, "plain", 6), CallSite("vis_down_x4", 3072, 1152, 4304, "plain", 6),
    CallSite("enc_o_x4", 3072, 2048, 2048, "plain", 6), CallSite("enc_down_x4", 3072, 2048, 16384, "plain", 4),
    CallSite("enc_gate_x4", 3072, 16384, 2048, "dual", 4),
    # the residual projections of a decoder batched over 4 episodes (M = 204, fp32 residual stream, no shadow)
    CallSite("dec_o_x4", 204, 1024, 2048, "plain", 18), CallSite("dec_down_x4", 204, 1024, 4096, "plain", 18),
)}


def candidates(site: CallSite) -> list[dict]:
    """Every plan worth timing for a call site (the library rejects the ones a shape cannot take)."""
    if site.kind == "plain":
        return ([{"engine": "tc5_scratch", **c} for c in grid(bn=[64, 128, 192, 256], splits=[1, 2, 3, 4])] +
                [{"engine": "tc5_cluster", "bn": 128, "splits": s} for s in (2, 3, 4)] +
                [{"engine": "pair", "bn": 256, "splits": s} for s in (1, 2, 3, 4, 6)])
    if site.kind == "dual":
        return [{"engine": "pair", "bn": 256, "splits": 1}, {"engine": "tc5_scratch", "bn": 128, "splits": 1}]
    if site.kind in ("skinny", "skinny_dual"):
        return [{"engine": "skinny", "bn": 128, "splits": s} for s in (1, 2, 4, 8)]
    return []


def build_site(site: CallSite, ops, generator):
    """Synthetic operands for a call site (weights ~ N(0, 0.02), activations ~ N(0, 1), as the isolated
    sweep configuration says) and `invoke(i)`, one launch against the i-th weight copy. Returns
    (invoke, result tensor)."""
    from .backends.cuda import wrappers
    from .buffers import rope_table
    M, N, K, L = site.M, site.N, site.K, site.layers
    dual = site.kind in ("dual", "skinny_dual")

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=generator) * scale).to(bf16)

    w = [rnd(K, N, scale=0.02) for _ in range(L * (2 if dual else 1))]
    name = site.name[:-3] if site.name.endswith("_x4") else site.name      # batched sites run the same ops on more rows
    views = M // 256
    if name in ("vis_qkv", "vis_up", "enc_projector"):
        x, bias = rnd(views, 256, K), rnd(N, scale=0.02)
        nw, nb = torch.ones(K, device="cuda", dtype=bf16), torch.zeros(K, device="cuda", dtype=bf16)
        xn = torch.zeros(views, 256, K, device="cuda", dtype=bf16)
        out = torch.zeros(M, N, device="cuda", dtype=bf16)
        op = {"vis_qkv": ops.vision_norm_qkv, "vis_up": ops.vision_norm_ffn_up, "enc_projector": ops.encoder_projector}[name]
        target = out if name == "enc_projector" else out.view(views, 256, N)
        return (lambda i: op(x, nw, nb, w[i], bias, target, xn)), out
    if name in ("vis_o", "vis_down"):
        x, bias, res = rnd(M, K), rnd(N, scale=0.02), rnd(M, N)
        out = torch.zeros(M, N, device="cuda", dtype=bf16)
        return (lambda i: ops.vision_ffn_down_residual(x, w[i], bias, res, out)), out
    if name in ("enc_o", "enc_down"):
        x = rnd(M, K)
        out = torch.zeros(M, N, device="cuda", dtype=bf16)      # accumulates in place; checks start it from zero
        return (lambda i: ops.encoder_ffn_down_residual(x, w[i], out)), out
    if name == "enc_gate":
        x, xn = rnd(M, K), torch.zeros(M, K, device="cuda", dtype=bf16)
        out = torch.zeros(M, N, device="cuda", dtype=bf16)
        return (lambda i: ops.encoder_norm_gated_ffn(x, w[2 * i], w[2 * i + 1], out, xn)), out
    # decoder sites: the residual stream is fp32 with a bf16 shadow, as in the engine
    if name in ("dec_qkv", "dec_gate"):
        x = torch.randn(M, K, device="cuda", generator=generator)
        wrappers.register_bf16_shadow(x, torch.zeros(M, K, device="cuda", dtype=bf16))
        nf = torch.zeros(M, device="cuda", dtype=bf16)
        if name == "dec_gate":
            out = torch.zeros(M, N, device="cuda", dtype=bf16)
            return (lambda i: ops.decoder_norm_gated_ffn(x, w[2 * i], w[2 * i + 1], out, nf)), out
        rope = rope_table(M, 768, 256, "cuda")
        Q = torch.zeros(M * 8, 256, device="cuda", dtype=bf16)
        Kc, Vc = torch.zeros(M, 256, device="cuda", dtype=bf16), torch.zeros(M, 256, device="cuda", dtype=bf16)
        return (lambda i: ops.decoder_norm_qkv_rope(x, w[i], rope, Q, Kc, Vc, nf)), Q
    if name in ("dec_o", "dec_down"):
        x = rnd(M, K)
        out = torch.zeros(M, N, device="cuda")
        if M <= 64:
            wrappers.register_bf16_shadow(out, torch.zeros(M, N, device="cuda", dtype=bf16))
        return (lambda i: ops.decoder_ffn_down_residual(x, w[i], out)), out
    if name == "dec_action_mlp":
        x, bias = rnd(M, K), rnd(N, scale=0.02)
        out = torch.zeros(M, N, device="cuda")
        return (lambda i: ops.decoder_action_mlp(x, w[i], bias, out)), out
    raise KeyError(name)


def _close(got: torch.Tensor, ref: torch.Tensor) -> bool:
    """Same result up to summation order: |diff| <= 1e-2 rms(ref) + 1e-2 |ref| on all but a 1e-4 fraction."""
    got, ref = got.float(), ref.float()
    bound = 1e-2 * ref.pow(2).mean().sqrt() + 1e-2 * ref.abs()
    return bool(torch.isfinite(got).all()) and ((got - ref).abs() > bound).float().mean().item() <= 1e-4


def sweep(site: CallSite, reps: int = 20, verbose: bool = True, seed: int = 0) -> list[dict]:
    """Time the default plan and every candidate of one call site; results fastest first. Each entry:
    {"us", "engine", "bn", "splits"} (the default plan has engine "auto"). Candidates the library refuses,
    and candidates whose result differs from the default plan's, are dropped and counted."""
    from flash_vla_b200 import op_table
    from flash_vla_b200.runtime.cuda import ScratchPool
    from .backends.cuda import _lib, wrappers
    lib = _lib.load()
    # The unfused table: a pinned plan addresses the plain GEMM of an op. (The fused table's three prefix ops that
    # fold their row norm into the GEMM pick their tile from the shape alone and consult no plan.)
    ops = op_table(False)
    saved = _pinned_snapshot()
    results, refused, wrong = [], 0, 0
    try:
        invoke, out = build_site(site, ops, torch.Generator(device="cuda").manual_seed(seed))
        # Every plan gets a scratch pool of its own: split-K scratch holds self-resetting tile counters whose
        # layout depends on the plan, so a buffer must never serve two plans.
        lib.fvla_gemm_plan_clear()
        with wrappers.use_pool(ScratchPool()):
            out.zero_()
            invoke(0)
            torch.cuda.synchronize()
            ref = out.clone()
            results.append({"us": round(graph_time_cold(invoke, site.layers, reps), 3), "engine": "auto", "bn": 0, "splits": 0})
        for cand in candidates(site):
            lib.fvla_gemm_plan_clear()
            if lib.fvla_gemm_plan_set(*site.key(), ENGINE[cand["engine"]], cand["bn"], cand["splits"]) != 0:
                refused += 1
                continue
            with wrappers.use_pool(ScratchPool()):
                try:
                    out.zero_()
                    invoke(0)
                    torch.cuda.synchronize()
                except _lib.FvlaError:
                    refused += 1
                    continue
                if lib.fvla_device_status(None) != 0 or not _close(out, ref):
                    wrong += 1
                    continue
                results.append({"us": round(graph_time_cold(invoke, site.layers, reps), 3), **cand})
    finally:
        _pinned_restore(saved)
    results.sort(key=lambda r: r["us"])
    if verbose:
        print(f"[{site.name}] M={site.M} N={site.N} K={site.K} {site.kind}: {len(results)} plans timed "
              f"({refused} refused, {wrong} incorrect)")
        for r in results[:6]:
            print(f"    us={r['us']:8.3f}  {r['engine']:12s} bn={r['bn']:3d} splits={r['splits']}")
    return results


# The plans this process has pinned through `apply_plans` (the library has no read-back call).
_PINNED: list[dict] = []


def _pinned_snapshot() -> list[dict]:
    return list(_PINNED)


def _pinned_restore(plans: list[dict]) -> None:
    apply_plans({"plans": plans})


def tune(names=None, reps: int = 20, margin: float = 0.03, verbose: bool = True) -> dict:
    """Sweep the named call sites (default: all). A winner is kept only if it beats the default plan by more
    than `margin` (run-to-run noise is a few per cent); the table also records every site's default time."""
    plans, report = [], {}
    for name in (names or [n for n in SITES if not n.endswith("_x4")]):
        site = SITES[name]
        res = sweep(site, reps=reps, verbose=verbose)
        auto = next(r for r in res if r["engine"] == "auto")
        best = res[0]
        report[name] = {"auto_us": auto["us"], "best": best, "timed": len(res)}
        if best["engine"] != "auto" and best["us"] < auto["us"] * (1.0 - margin):
            plans.append({"site": name, "M": site.M, "N": site.N, "K": site.K, "kind": site.kind,
                          "engine": best["engine"], "bn": best["bn"], "splits": best["splits"],
                          "us": best["us"], "auto_us": auto["us"]})
    return {"device": torch.cuda.get_device_name(0), "plans": plans, "report": report}


def save_plans(table: dict, path=DEFAULT_PLAN_FILE) -> None:
    Path(path).write_text(json.dumps(table, indent=1) + "\n")


def load_plans(path=DEFAULT_PLAN_FILE) -> dict | None:
    path = Path(path)
    return json.loads(path.read_text()) if path.exists() else None


def apply_plans(table: dict | None) -> int:
    """Pin the table's plans (clearing any pinned before). Returns how many are in force."""
    from .backends.cuda import _lib
    lib = _lib.load()
    lib.fvla_gemm_plan_clear()
    _PINNED.clear()
    for p in (table or {}).get("plans", []):
        _lib.call("fvla_gemm_plan_set", p["M"], p["N"], p["K"], KIND[p["kind"]], ENGINE[p["engine"]], p["bn"], p["splits"])
        _PINNED.append(p)
    return lib.fvla_gemm_plan_count()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", default=str(DEFAULT_PLAN_FILE))
    ap.add_argument("--sites", default="", help="comma-separated call sites (default: all)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--margin", type=float, default=0.03)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a CUDA device")
    table = tune([s for s in args.sites.split(",") if s] or None, reps=args.reps, margin=args.margin)
    save_plans(table, args.out)
    print(json.dumps({"plans": table["plans"]}))


if __name__ == "__main__":
    main()
