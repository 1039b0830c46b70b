"""Shared test plumbing: path setup, the `gpu` marker, tolerance helper, cached checkpoints."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def assert_close(got: torch.Tensor, ref: torch.Tensor, rtol: float = 1e-2, atol_rms: float = 1e-2,
                 what: str = ""):
    """|got - ref| <= atol_rms * rms(ref) + rtol * |ref| elementwise, both taken as fp32 on CPU.

    bf16 storage alone costs 2^-9 relative per rounding; the defaults allow a few roundings
    plus fp32 accumulation-order differences.
    """
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values in the result"
    rms = ref.pow(2).mean().sqrt().item()
    bound = atol_rms * rms + rtol * ref.abs()
    err = (got - ref).abs()
    worst = (err - bound).max().item()
    assert worst <= 0, (f"{what}: max abs err {err.max().item():.4g} (rms(ref)={rms:.4g}), "
                        f"exceeds bound by {worst:.4g}")


@pytest.fixture(scope="session")
def full_checkpoint():
    """The synthetic checkpoint named by the benchmark configs: seed 0, scale 0.02, no prompt,
    generated on the CPU (CPU and CUDA generators differ for one seed)."""
    from flash_vla_b200.models.pi0 import random_checkpoint
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    return random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cpu")


@pytest.fixture(scope="session")
def decoder_checkpoint():
    """The decoder tensors of the same checkpoint, drawn once per session (a draw walks the whole
    2.7 G-parameter stream on one CPU thread, about a minute, whatever is kept)."""
    from flash_vla_b200.models.pi0 import random_checkpoint
    return random_checkpoint(prompt_len=0, wscale=0.02, seed=0, device="cpu", only=("decoder_",))
