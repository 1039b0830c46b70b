"""A bounded device-side wait that really runs out.

Every wait in the kernels (on an mbarrier that TMA, a tensor-core commit or a peer CTA completes) polls
a limited number of times; past the limit the kernel raises an abort flag in shared memory, every role
leaves its loops, tensor memory is released and a code lands in the device status word. This test makes
one such wait expire without faulting anything: `fvla_selftest_wait_timeout` runs the decoder's cluster
GEMM with its finishing CTAs told (by the host) to expect 16 bytes more than their peers will ever send,
and with the poll limit lowered to a few thousand, so the whole thing takes microseconds.
"""
from __future__ import annotations

import time

import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def test_a_wait_that_runs_out_is_reported_and_leaves_the_gpu_usable():
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib
    from flash_vla_b200 import op_table
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(21)
    M, K, N = 51, 2048, 1024
    x = torch.randn(M, K, generator=g).to(bf16).cuda()
    w = (torch.randn(K, N, generator=g) * 0.02).to(bf16).cuda()
    out = torch.zeros(M, N, dtype=bf16, device="cuda")
    assert lib.fvla_device_status(None) == 0

    t0 = time.perf_counter()
    _lib.call("fvla_selftest_wait_timeout", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, 4096, stream)
    torch.cuda.synchronize()                                   # returns: the kernel did not hang
    elapsed = time.perf_counter() - t0
    assert elapsed < 2.0, f"the expired wait took {elapsed:.3f} s"
    assert lib.fvla_device_status(None) == 2                   # code of the cluster GEMM; reading clears it
    assert lib.fvla_device_status(None) == 0

    # tensor memory was released and the context is healthy: the same kernel, launched normally right
    # after, gives the right answer, several times over (a leaked TMEM allocation would stall these)
    for _ in range(4):
        res = torch.ones(M, N, dtype=bf16, device="cuda")
        op_table().decoder_out_proj_residual(x, w, res)
        torch.cuda.synchronize()
        assert_close(res, 1.0 + x.float().cpu() @ w.float().cpu(), what="cluster GEMM after an expired wait")
    assert lib.fvla_device_status(None) == 0

    # argument errors of the self-test itself come back as codes, with nothing launched
    assert lib.fvla_selftest_wait_timeout(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, 0, stream) == -1
    assert lib.fvla_selftest_wait_timeout(x.data_ptr(), w.data_ptr(), out.data_ptr(), 300, N, K, 4096, stream) == -4
