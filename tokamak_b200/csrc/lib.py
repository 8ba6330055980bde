"""Loads the CUDA library and declares its C interface for ``ctypes``.

The engine has no path without this library: :func:`library` raises if it can
neither be found nor built.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p
from functools import lru_cache

from .build import BuildError, ensure_built

_P = c_void_p

# name -> argument types (every function returns a cudaError_t as int unless noted)
_SIGNATURES: dict[str, list] = {
    "tk_embed_gather": [_P, c_int, _P, _P, c_int, c_int, c_int, _P, _P],
    "tk_step_begin": [_P, c_int, c_int, _P, c_int, _P, c_longlong, _P, _P, _P, _P, _P, c_int, c_int, _P, _P],
    "tk_decode_begin": [_P, c_int, c_int, _P, c_int, _P, c_longlong, _P, c_int, c_int, _P, _P, _P, _P, _P],
    "tk_sample_slots": [_P, c_longlong, _P, _P, c_int, _P, c_int, c_int, _P, _P],
    "tk_wait_probe": [c_uint, _P, _P],
    "tk_probe_mma_issue": [c_int, c_int, c_int, _P, _P, _P],
    "tk_probe_softmax_tile": [c_int, c_int, c_int, c_int, _P, _P],
    "tk_gemm_chain": [_P, c_int, c_int, _P, _P, _P, c_int, _P],
    "tk_gemm_chain_blocks": [],
    "tk_gemm_chain_max_phases": [],
    "tk_slot_words": [],
    "tk_add_rmsnorm": [_P, _P, _P, c_int, c_longlong, _P, _P, _P, c_int, c_int, c_float, c_int, _P],
    "tk_swiglu": [_P, _P, c_int, c_longlong, _P, c_int, c_int, c_int, c_int, _P],
    "tk_rope_kv": [_P, _P, c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                   c_float, c_int, _P],
    "tk_rope_table": [_P, _P, _P, c_int, c_int, _P],
    "tk_attention_plain": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_float, c_int, _P],
    "tk_attention_decode": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_float, _P],
    "tk_attention_decode_balanced": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                     c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_float, _P],
    "tk_attention_prefill": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_float, _P],
    "tk_attention_prefill_tc": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_float, _P],
    "tk_attention_prefill_tc_takes": [c_int, c_int, c_int, c_int],
    "tk_attention_prefill_tc_rows": [],
    "tk_attention_prefill_tc_keys": [],
    "tk_attention_prefill_tc_record_ints": [],
    "tk_attention_prefill_tc_max_parts": [],
    "tk_gemm_bf16_tcgen05": [_P, _P, _P, _P, c_int, c_int, c_int, c_longlong, c_longlong,
                             c_int, c_int, c_int, c_int, c_int,
                             _P, c_int, c_float, c_float, _P, _P, _P, _P, _P],
    "tk_gemm_qkv_rope": [_P, _P, _P, c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_int,
                         _P, c_int, c_float, c_float,
                         _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                         c_int, c_int, c_int, c_int, c_int, c_int, c_float, _P],
    "tk_gemm_bf16_pair": [_P, _P, _P, _P, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, _P],
    "tk_gemm_f32": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "tk_sample": [_P, c_longlong, _P, _P, _P, _P, _P, _P, c_int, c_int, _P],
}


@lru_cache(maxsize=1)
def library() -> ctypes.CDLL:
    """The loaded library, compiled on first use if it is stale or absent."""
    try:
        path = ensure_built()
    except BuildError as exc:
        raise RuntimeError(
            f"tokamak_b200 needs its CUDA extension and could not build it: {exc}") from exc
    lib = ctypes.CDLL(str(path))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    for name, args in (("tk_gemm_chain_scratch_floats", [c_int]), ("tk_gemm_chain_counter_ints", [c_int]),
                       ("tk_attention_decode_balanced_scratch_floats", [c_int, c_int])):
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_longlong
    lib.tk_philox_u32.argtypes = [c_ulonglong, c_uint, ctypes.POINTER(c_uint)]
    lib.tk_philox_u32.restype = None
    return lib
