"""The diagnostic environment switches select other kernels for the same ops; those kernels must stay
parity-clean too. Each switch is read once per process, so every case runs in a child interpreter.

  FVLA_ATTN=mma   prefix attention on the warp-level kernels (key-split form with the merge kernel)
  FVLA_GEMM=mma   every GEMM on the warp-level kernel (no tcgen05)
  FVLA_PDL=0      no programmatic dependent launch
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

CHILD = r"""
import sys, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from conftest import assert_close
from oracle import pi0_ref as O
from flash_vla_b200 import op_table
bf16 = torch.bfloat16
ops, ref = op_table(fused=True), O.op_table(fused=True)
g = torch.Generator().manual_seed(11)
rnd = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale).to(bf16)
for S in (768, 817):                                   # prefix attention, aligned and ragged
    Q, K, V = rnd(S * 8, 256), rnd(S, 256), rnd(S, 256)
    want = torch.zeros(S, 2048)
    ref.encoder_attention(Q.float(), K.float(), V.float(), 256 ** -0.5, want)
    got = torch.zeros(S, 2048, dtype=bf16, device="cuda")
    ops.encoder_attention(Q.cuda(), K.cuda(), V.cuda(), 256 ** -0.5, got)
    assert_close(got, want, what=f"encoder_attention S={S}")
x, w = rnd(768, 2048), rnd(2048, 2048, scale=0.02)     # a residual GEMM of the prefix encoder
out = rnd(768, 2048)
want = out.float().clone()
ref.encoder_out_proj_residual(x.float(), w.float(), want)
got = out.cuda()
ops.encoder_out_proj_residual(x.cuda(), w.cuda(), got)
assert_close(got, want, what="encoder_out_proj_residual")
x32, wd = torch.randn(51, 1024, generator=g), rnd(4096, 1024, scale=0.02)   # a decoder GEMM into the fp32 stream
h = rnd(51, 4096)
want = x32.clone()
ref.decoder_ffn_down_residual(h.float(), wd.float(), want)
got = x32.cuda()
ops.decoder_ffn_down_residual(h.cuda(), wd.cuda(), got)
assert_close(got, want, what="decoder_ffn_down_residual")
torch.cuda.synchronize()
print("SWITCH-OK")
"""


@pytest.mark.parametrize("env", [{"FVLA_ATTN": "mma"}, {"FVLA_GEMM": "mma"}, {"FVLA_PDL": "0"}],
                         ids=["attn-mma", "gemm-mma", "no-pdl"])
def test_switch_keeps_parity(env):
    child_env = dict(os.environ, **env)
    res = subprocess.run([sys.executable, "-c", CHILD, str(ROOT)], env=child_env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "SWITCH-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
