"""The scratch-free patch embedding entry point, called straight through the C ABI.

`fvla_vision_patch_embed_noalloc` exists for callers that cannot hand the library any scratch
memory: a robot's control loop that must not call cudaMalloc (the call stalls the device and may
take arbitrarily long), a plain C host with no allocator, or Python code whose ScratchPool has been
frozen after graph capture. It keeps the patchified images in a fixed array inside the library, so
it must give exactly what the scratch-taking entry point gives, call after call, although every
call reuses the same array with the previous call's data still in it.

This file sorts last on purpose: with `pytest -x` everything else has already run when it does.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _inputs(views: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    img = (torch.rand(views, 224, 224, 3, generator=g) * 2 - 1).to(bf16).cuda()
    pw = (torch.randn(14, 14, 3, 1152, generator=g) * 0.02).to(bf16).cuda()
    pb = (torch.randn(1152, generator=g) * 0.02).to(bf16).cuda()
    pos = (torch.randn(256, 1152, generator=g) * 0.02).to(bf16).cuda()
    return img, pw, pb, pos


def test_noalloc_patch_embed_matches_the_scratch_taking_entry_point():
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different sizes and data: the second one finds the first one's
    # patches still in the shared array and must not be affected by them
    for views, seed in ((3, 1), (1, 2), (3, 3), (4, 5)):          # 4 views fill the array exactly
        img, pw, pb, pos = _inputs(views, seed)
        want = torch.zeros(views, 256, 1152, dtype=bf16, device="cuda")
        nbytes = lib.fvla_patch_embed_workspace_bytes(views)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        _lib.call("fvla_vision_patch_embed", img.data_ptr(), pw.data_ptr(), pb.data_ptr(), pos.data_ptr(),
                  want.data_ptr(), views, ws.data_ptr(), nbytes, stream)
        got = torch.full_like(want, 7.0)
        before = torch.cuda.memory_allocated()
        _lib.call("fvla_vision_patch_embed_noalloc", img.data_ptr(), pw.data_ptr(), pb.data_ptr(),
                  pos.data_ptr(), got.data_ptr(), views, stream)
        assert torch.cuda.memory_allocated() == before          # nothing was taken from torch's allocator
        torch.cuda.synchronize()
        # same kernels on the same patch matrix: the tolerance of the other op tests would do, but the
        # two results are in fact bit-identical
        assert torch.equal(got, want)
        assert lib.fvla_device_status(None) == 0


def test_noalloc_patch_embed_rejects_more_views_than_its_array_holds():
    from flash_vla_b200.hardware.nvidia.b200.pi0.backends.cuda import _lib
    lib = _lib.load()
    img, pw, pb, pos = _inputs(1, 4)
    out = torch.zeros(5, 256, 1152, dtype=bf16, device="cuda")
    status = lib.fvla_vision_patch_embed_noalloc(img.data_ptr(), pw.data_ptr(), pb.data_ptr(), pos.data_ptr(),
                                                 out.data_ptr(), 5, torch.cuda.current_stream().cuda_stream)
    assert status == -2                                         # FVLA_ERR_WORKSPACE
    message = lib.fvla_last_error().decode()
    assert "at most 4 views" in message
    torch.cuda.synchronize()
    assert (out == 0).all()                                     # nothing was launched

