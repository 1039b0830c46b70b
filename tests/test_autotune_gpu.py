"""The launch-plan sweep on the GPU: pinned plans give the default plan's result, plans a launch cannot
honour are refused loudly, and the sweep itself ranks real timings."""
from __future__ import annotations

import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


@pytest.fixture()
def clean_plans():
    from flash_vla_b200.hardware.nvidia.b200.pi0 import autotune
    autotune.apply_plans(None)
    yield autotune
    autotune.apply_plans(None)


def test_pinned_plans_reproduce_the_default_result(clean_plans):
    from flash_vla_b200 import op_table
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib, wrappers
    from flash_vla_b200.runtime.cuda import ScratchPool
    autotune, ops = clean_plans, op_table()
    g = torch.Generator().manual_seed(3)
    M, K, N = 768, 4304, 1152                                          # SigLIP down projection: ragged K
    x, w = torch.randn(M, K, generator=g).to(bf16).cuda(), (torch.randn(K, N, generator=g) * 0.02).to(bf16).cuda()
    b, res = (torch.randn(N, generator=g) * 0.02).to(bf16).cuda(), torch.randn(M, N, generator=g).to(bf16).cuda()
    want = res.float().cpu() + x.float().cpu() @ w.float().cpu() + b.float().cpu()
    for plan in (None, ("tc5_scratch", 192, 2), ("tc5_scratch", 256, 1), ("tc5_cluster", 128, 2), ("tc5_scratch", 128, 4),
                 ("pair", 256, 1), ("pair", 256, 3)):
        table = None if plan is None else {"plans": [{"M": M, "N": N, "K": K, "kind": "plain", "engine": plan[0],
                                                       "bn": plan[1], "splits": plan[2]}]}
        assert autotune.apply_plans(table) == (0 if plan is None else 1)
        out = torch.zeros(M, N, dtype=bf16, device="cuda")
        with wrappers.use_pool(ScratchPool()):                         # one scratch buffer must not serve two plans
            ops.vision_ffn_down_residual(x, w, b, res, out)
        torch.cuda.synchronize()
        assert_close(out, want, what=f"vision_ffn_down_residual under plan {plan}")
    # a 4-way cluster split of this shape needs 216 CTAs at once: pinned, the launch must fail, not fall back
    autotune.apply_plans({"plans": [{"M": M, "N": N, "K": K, "kind": "plain", "engine": "tc5_cluster", "bn": 128, "splits": 4}]})
    with wrappers.use_pool(ScratchPool()), pytest.raises(_lib.FvlaError, match="pinned plan"):
        ops.vision_ffn_down_residual(x, w, b, res, torch.zeros(M, N, dtype=bf16, device="cuda"))
    torch.cuda.synchronize()


def test_sweep_ranks_the_plans_of_a_call_site(clean_plans):
    autotune = clean_plans
    results = autotune.sweep(autotune.SITES["dec_o"], reps=5, verbose=False)
    assert [r["us"] for r in results] == sorted(r["us"] for r in results)
    assert any(r["engine"] == "auto" for r in results) and len(results) >= 3
    assert all(1.0 < r["us"] < 500.0 for r in results)
    table = autotune.tune(["dec_o"], reps=5, verbose=False)
    assert set(table) == {"device", "plans", "report"} and "dec_o" in table["report"]
    for p in table["plans"]:                                           # a kept winner beats the default by the margin
        assert p["us"] < 0.97 * p["auto_us"]
