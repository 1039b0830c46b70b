"""ctypes binding of libfvla_b200.so, the C ABI declared in include/flash_vla_b200.h.

The library is the only implementation behind the CUDA backend: when it is missing or an
entry point returns an error, the caller gets an exception; nothing falls back to PyTorch.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parents[6] / "libfvla_b200.so"

_P, _I, _Z, _F = c_void_p, c_int, c_size_t, c_float

# name -> argument ctypes (every function returns int except the three queries below)
SIGNATURES: dict[str, list] = {
    "fvla_vision_patch_embed": [_P, _P, _P, _P, _P, _I, _P, _Z, _P],
    "fvla_vision_patch_embed_noalloc": [_P, _P, _P, _P, _P, _I, _P],
    "fvla_vision_norm_qkv": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "fvla_vision_attention": [_P, _P, _I, _I, _I, _I, _P],
    "fvla_vision_linear_bias_residual": [_P, _P, _P, _P, _P, _I, _I, _I, _P, _Z, _P],
    "fvla_vision_norm_ffn_up": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "fvla_fold_layernorm": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _P],
    "fvla_vision_folded_norm_linear": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "fvla_encoder_qkv_rope_fused_norm": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "fvla_encoder_projector": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "fvla_encoder_norm_qkv_rope": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "fvla_encoder_attention": [_P, _P, _P, _P, _I, _I, _I, _F, _P, _Z, _P],
    "fvla_linear_residual": [_P, _P, _P, _I, _P, _I, _I, _I, _I, _P, _Z, _P],
    "fvla_encoder_norm_gated_ffn": [_P, _P, _P, _P, _P, _I, _I, _I, _P],
    "fvla_decoder_small_proj": [_P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P, _Z, _P],
    "fvla_decoder_norm_qkv_rope": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _Z, _P],
    "fvla_decoder_attention": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, ctypes.c_longlong, ctypes.c_longlong, _P, _Z, _P],
    "fvla_decoder_norm_gated_ffn": [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _P, _Z, _P],
    "fvla_decoder_action_out_proj": [_P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _P],
    "fvla_embed_rows": [_P, _P, _P, _I, _I, ctypes.c_longlong, _P],
    "fvla_convert_copy": [_P, _I, _P, _I, _P, _Z, _P],
    "fvla_selftest_wait_timeout": [_P, _P, _P, _I, _I, _I, ctypes.c_uint, _P],
    "fvla_gemm_plan_set": [_I, _I, _I, _I, _I, _I, _I],
    "fvla_gemm_plan_clear": [],
}
QUERIES: dict[str, tuple] = {
    "fvla_last_error": ([], c_char_p),
    "fvla_abi_version": ([], c_int),
    "fvla_fused_norm_supported": ([_I, _I, _I, _I], c_int),
    "fvla_gemm_plan_count": ([], c_int),
    "fvla_launch_count": ([], ctypes.c_ulonglong),
    "fvla_device_status": ([_P], c_int),
    "fvla_gemm_workspace_bytes": ([_I, _I, _I, _I], c_size_t),
    "fvla_decoder_attention_workspace_bytes": ([_I, _I], c_size_t),
    "fvla_encoder_attention_workspace_bytes": ([_I, _I], c_size_t),
    "fvla_patch_embed_workspace_bytes": ([_I], c_size_t),
}

_lib = None


class FvlaError(RuntimeError):
    """An entry point of libfvla_b200 returned a non-zero status."""


def load() -> ctypes.CDLL:
    """Load the library once and attach argument/return types to every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise FvlaError(
            f"{LIB_PATH} is missing: build it with `python -m flash_vla_b200.build`. "
            "The CUDA backend has no other implementation to fall back to.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = argtypes, c_int
    for name, (argtypes, restype) in QUERIES.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = argtypes, restype
    _lib = lib
    return lib


def call(name: str, *args) -> None:
    """Invoke an entry point; raise FvlaError with the library's message on failure."""
    lib = load()
    status = getattr(lib, name)(*args)
    if status != 0:
        raise FvlaError(f"{name} failed with status {status}: {lib.fvla_last_error().decode()}")
