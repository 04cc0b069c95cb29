"""ctypes binding of include/hqq_moe.h.

The library is the only compute path: if it is missing or a call fails, this
module raises — there is no eager / CPU substitute behind it.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhqq_moe_b200.so")

HQM_ERR_ARG, HQM_ERR_CUDA, HQM_ERR_SCRATCH, HQM_ERR_STATE = -1, -2, -3, -4


class HqmWeight(C.Structure):
    """struct hqm_weight."""
    _fields_ = [
        ("N", C.c_int32), ("K", C.c_int32), ("nbits", C.c_int32), ("group_size", C.c_int32),
        ("meta_group", C.c_int32), ("meta_group_zero", C.c_int32),
        ("W_q", C.c_void_p), ("scale_q", C.c_void_p), ("zero_q", C.c_void_p),
        ("ms_scale", C.c_void_p), ("mz_scale", C.c_void_p), ("ms_zero", C.c_void_p), ("mz_zero", C.c_void_p),
    ]


class HqmAttnLayer(C.Structure):
    """struct hqm_attn_layer."""
    _fields_ = [
        ("q", HqmWeight), ("k", HqmWeight), ("v", HqmWeight), ("o", HqmWeight),
        ("ln_in", C.c_void_p), ("ln_post", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("max_len", C.c_int32),
        ("rope_theta", C.c_float), ("rms_eps", C.c_float),
    ]


class HqmDecoderLayer(C.Structure):
    """struct hqm_decoder_layer."""
    _fields_ = [
        ("attn", HqmAttnLayer), ("gate_w", C.c_void_p), ("table", C.c_void_p),
        ("w1", HqmWeight), ("w2", HqmWeight), ("w3", HqmWeight), ("next_ln", C.c_void_p),
        ("n_experts", C.c_int32), ("reserved", C.c_int32),
    ]


class HqmEpComm(C.Structure):
    """struct hqm_ep_comm."""
    _fields_ = [
        ("rank", C.c_int32), ("world", C.c_int32), ("hidden", C.c_int32), ("reserved", C.c_int32),
        ("shares", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("seq", C.c_void_p),
    ]


_P = C.c_void_p
_I64 = C.c_int64
_I32 = C.c_int32
_WP = C.POINTER(HqmWeight)

# name -> (restype, argtypes); mirrors include/hqq_moe.h line for line
SIGNATURES = {
    "hqm_last_error": (C.c_char_p, []),
    "hqm_version": (C.c_int, []),
    "hqm_launch_count": (C.c_int64, []),
    "hqm_device_error": (C.c_int, []),
    "hqm_set_overlap": (C.c_int, [C.c_int]),
    "hqm_set_tma_mode": (C.c_int, [C.c_int]),
    "hqm_pack_4bit_u8": (C.c_int, [_P, _P, _I64, _I64, _P]),
    "hqm_unpack_4bit_u8": (C.c_int, [_P, _P, _I64, _I64, _P]),
    "hqm_pack_2bit_u8": (C.c_int, [_P, _P, _I64, _I64, _P]),
    "hqm_unpack_2bit_u8": (C.c_int, [_P, _P, _I64, _I64, _P]),
    "hqm_pack_3bit_i32": (C.c_int, [_P, _P, _I64, _I64, _P]),
    "hqm_unpack_3bit_i32": (C.c_int, [_P, _P, _I64, _I64, _P]),
    "hqm_dequantize": (C.c_int, [_P, C.c_int, _WP, _P]),
    "hqm_scratch_header_bytes": (C.c_size_t, []),
    "hqm_scratch_init": (C.c_int, [_P, _P]),
    "hqm_linear_scratch_bytes": (C.c_size_t, [_I64, _WP]),
    "hqm_linear": (C.c_int, [_P, _P, _I64, _WP, _P, _P, C.c_size_t, _P]),
    "hqm_static_scratch_capacity": (C.c_size_t, []),
    "hqm_linear_static_scratch": (C.c_int, [_P, _P, _I64, _WP, _P, _P]),
    "hqm_expert_ffn_scratch_bytes": (C.c_size_t, [_I64, _WP, _WP, _WP]),
    "hqm_expert_ffn": (C.c_int, [_P, _P, _I64, _P, _P, C.c_int, _WP, _WP, _WP, _P, C.c_size_t, _P]),
    "hqm_expert_table_bytes": (C.c_size_t, [_I32]),
    "hqm_expert_table_build": (C.c_int, [_P, _WP, _I32]),
    "hqm_moe_decode_scratch_bytes": (C.c_size_t, [_I32, _WP, _WP, _WP]),
    "hqm_moe_decode": (C.c_int, [_P, _P, _P, _P, _I32, _P, _WP, _WP, _WP, _P, C.c_size_t, _P]),
    "hqm_attn_decode_scratch_bytes": (C.c_size_t, [C.POINTER(HqmAttnLayer)]),
    "hqm_attn_decode": (C.c_int, [_P, _P, _P, C.POINTER(HqmAttnLayer), _P, _P, C.c_size_t, _P]),
    "hqm_decode_layer_scratch_bytes": (C.c_size_t, [C.POINTER(HqmDecoderLayer)]),
    "hqm_decode_layer": (C.c_int, [_P, _P, _P, C.POINTER(HqmDecoderLayer), _P, _P, C.c_size_t, _P]),
    "hqm_decode_layer_ep_scratch_bytes": (C.c_size_t, [C.POINTER(HqmDecoderLayer), _I32]),
    "hqm_ep_exchange_bytes": (C.c_size_t, [_I32, _I32]),
    "hqm_ep_exchange_flags_offset": (C.c_size_t, [_I32, _I32]),
    "hqm_decode_layer_ep": (C.c_int, [_P, _P, _P, _P, C.POINTER(HqmEpComm), C.POINTER(HqmDecoderLayer), _I32, _I32, _P, _P,
                                      C.c_size_t, _P]),
    "hqm_ep_combine_add_rmsnorm": (C.c_int, [_P, C.POINTER(HqmEpComm), _P, _P, _I32, C.c_float, _P]),
    "hqm_add_f32_rmsnorm": (C.c_int, [_P, _P, _P, _P, _I32, C.c_float, _P]),
    "hqm_add_rmsnorm": (C.c_int, [_P, _P, _P, _P, _I32, C.c_float, _P]),
    "hqm_add_rmsnorm_rows": (C.c_int, [_P, _P, _P, _P, C.c_int64, _I32, C.c_float, _P]),
    "hqm_rope_append_rows": (C.c_int, [_P, _P, _P, _P, _P, C.c_int64, _I32, _I32, _I32, _I32, C.c_int64, _P, _I32, _I32,
                                       C.c_float, _P]),
    "hqm_router_top2": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I32, _P]),
    "hqm_cache_create": (C.c_int, [C.POINTER(_P), _I32, _I32, _I32, C.c_size_t, C.POINTER(_P), _I32]),
    "hqm_cache_destroy": (None, [_P]),
    "hqm_cache_add": (C.c_int, [_P, _I64, _I32, _I32, _P, C.POINTER(_I32), _P]),
    "hqm_cache_begin": (C.c_int, [_P, C.POINTER(_I64), _I32, _I32, C.POINTER(_I64), _P]),
    "hqm_cache_next": (C.c_int, [_P, C.POINTER(_I64), C.POINTER(_P), C.POINTER(_I32), _P]),
    "hqm_cache_end": (C.c_int, [_P, _P]),
    "hqm_cache_prefetch": (C.c_int, [_P, C.POINTER(_I64), _I32, C.POINTER(_I32)]),
    "hqm_cache_prefetch_stats": (C.c_int, [_P, C.POINTER(_I64), C.POINTER(_I64), C.POINTER(_I64)]),
    "hqm_cache_stats": (C.c_int, [_P, _I32, C.POINTER(_I64), C.POINTER(_I64), C.POINTER(_I64), C.POINTER(_I64)]),
    "hqm_cache_resident": (C.c_int, [_P, _I32, C.POINTER(_I64), _I32]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(python -m mixtral_offloading_b200.build); there is no fallback path")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def last_error() -> str:
    return (lib().hqm_last_error() or b"").decode()


def check(rc: int) -> None:
    """Turn a status into the exception type the reference raises for that failure."""
    if rc >= 0:
        return
    msg = last_error()
    if rc == HQM_ERR_STATE:
        if msg in ("Cache is full", "No evictable experts"):
            raise ValueError(msg)                          # expert_cache.py:36,118
        if msg.startswith("internal error"):
            raise RuntimeError(msg)                        # expert_cache.py:177
        raise AssertionError(msg)                          # expert_cache.py:98,134-140 are asserts
    if rc == HQM_ERR_ARG:
        raise ValueError(msg)
    raise RuntimeError(msg)


def ptr(t):
    """Device (or host) address of a tensor, None passes NULL."""
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("this operation runs only on a CUDA device (no CPU path exists)")
