"""Loads the CUDA libraries and declares their C entry points.

There is no other implementation behind these calls: when the GPU, nvcc or a library is
missing, the first kernel call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

from ..csrc import build as _build


class KernelError(RuntimeError):
    pass


_P, _I, _L, _F = c_void_p, c_int, c_longlong, c_float

# name -> argument types (all return int: 0 ok, else fmx_last_error() tells why)
_SIGNATURES = {
    "common": {
        "fmx_gather_rows": [_P, _P, _P, _I, _I, _L, _I, _P, _I, _P],
        "fmx_gather_rows_f32_to_bf16": [_P, _P, _P, _I, _I, _L, _P, _I, _P],
        "fmx_add_rmsnorm": [_P, _P, _P, _P, _I, _I, _F, _I, _I, _I, _P],
        "fmx_silu_mul": [_P, _P, _I, _I, _I, _I, _P],
        "fmx_gemm_simple": [_P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _I, _I, _P],
        "fmx_rope_kv_write": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _L, _L, _I, _P, _P],
        "fmx_paged_attention_simple": [_P, _L, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _L, _F, _I, _I, _I, _P, _P],
        "fmx_sample": [_P, _L, _I, _I, _P, _P, _P, _L, _P, _I, _P, _I, _P, _I, _P],
        "fmx_filter_mask": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _L, _P],
        "fmx_filter_sample": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P],
        "fmx_penalties": [_P, _L, _I, _I, _P, _I, _P, _P, _P, _P, _P],
        "fmx_logit_bias": [_P, _L, _I, _P, _P, _P, _I, _P],
    },
    "bf16": {
        "fmx_gemv": [_P, _L, _P, _L, _P, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _I, _P],
        "fmx_gemv_argmax": [_P, _L, _P, _L, _P, _P, _P, _I, _I, _I, _P],
    },
    "tc": {
        "fmx_gemm_tcgen05": [_P, _L, _P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _P, _P],
    },
    "attn": {
        "fmx_attn_prefill_tc": [_P, _L, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _L, _F, _I, _P, _I, _P, _L, _P],
        "fmx_attn_prefill": [_P, _L, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _L, _F, _I, _P, _P],
        "fmx_attn_decode": [_P, _L, _P, _P, _I, _P, _P, _P, _P, _L, _P, _I, _I, _I, _I, _I, _L, _F, _I, _P, _P, _I, _I, _I, _P],
    },
}

_libs: dict[str, ctypes.CDLL] = {}
launches = 0          # entry-point calls so far; each launches at least one kernel of this package


def load(group: str) -> ctypes.CDLL:
    lib = _libs.get(group)
    if lib is not None:
        return lib
    try:
        path = _build.build(group)
        lib = ctypes.CDLL(path)
    except (OSError, _build.BuildError) as e:
        raise KernelError(f"the CUDA library of group {group!r} is not available: {e}") from None
    if group.startswith("attn_hd"):
        lib.fmx_attn_decode_scratch_floats.argtypes = [_I, _I, _I]
        lib.fmx_attn_decode_scratch_floats.restype = c_longlong
        lib.fmx_attn_decode_plan.argtypes = [_I, _I, _L, _I]
        lib.fmx_attn_decode_plan.restype = c_int
        lib.fmx_attn_prefill_tc_plan_splits.argtypes = [_I, _I, _I, _I, _I, _I]
        lib.fmx_attn_prefill_tc_scratch_floats.argtypes = [_I, _I, _I]
        lib.fmx_attn_prefill_tc_scratch_floats.restype = c_longlong
    if group == "bf16":
        lib.fmx_gemv_plan_width.argtypes = [_I, _I, _I]
        lib.fmx_gemv_plan_warps.argtypes = [_I, _I, _I, _I]
    if group in ("tc", "tc_expiry"):
        lib.fmx_gemm_tcgen05_plan_width.argtypes = [_I, _I, _I]
        lib.fmx_gemm_tcgen05_plan_fills.argtypes = [_I, _I, _I]
    lib.fmx_last_error.restype = ctypes.c_char_p
    family = "attn" if group.startswith("attn_hd") else "tc" if group == "tc_expiry" else group
    for name, args in _SIGNATURES.get(family, {}).items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
    _libs[group] = lib
    return lib


def call(group: str, name: str, *args) -> None:
    global launches
    launches += 1
    lib = load(group)
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(lib.fmx_last_error().decode(errors="replace"))


def loaded_libraries() -> dict[str, str]:
    return {g: lib._name for g, lib in _libs.items()}
