"""Bit packing with the names and layouts of the reference's src/packing.py, run by
the CUDA kernels of csrc/packing.cu through the C ABI.

There is ONE layout here (the reference's "common" one: K contiguous, packing along
the output rows), so the reference's PackedTensor tag and the *_universal
dispatchers (packing.py:5-7,29-33,55-59,99-113) have nothing to distinguish and are
not reproduced.
"""
from __future__ import annotations

import torch

from . import _cabi


def _prep(t: torch.Tensor, dtype):
    _cabi.require_cuda(t)
    if t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _flat_k(t: torch.Tensor) -> int:
    k = 1
    for d in t.shape[1:]:
        k *= d
    return k


def pack_4bit_u8_common(W_q: torch.Tensor) -> torch.Tensor:
    """packing.py:10-17: rows 2R / 2R+1 -> high / low nibble of row R."""
    assert W_q.size(0) % 2 == 0
    W_q = _prep(W_q, torch.uint8)
    out = torch.empty((W_q.size(0) // 2,) + W_q.shape[1:], dtype=torch.uint8, device=W_q.device)
    _cabi.check(_cabi.lib().hqm_pack_4bit_u8(_cabi.ptr(out), _cabi.ptr(W_q), W_q.size(0), _flat_k(W_q),
                                            _cabi.stream_ptr(W_q.device)))
    return out


def unpack_4bit_u8_common(W_q: torch.Tensor) -> torch.Tensor:
    """packing.py:19-27."""
    W_q = _prep(W_q, torch.uint8)
    out = torch.empty((2 * W_q.size(0),) + W_q.shape[1:], dtype=torch.uint8, device=W_q.device)
    _cabi.check(_cabi.lib().hqm_unpack_4bit_u8(_cabi.ptr(out), _cabi.ptr(W_q), W_q.size(0), _flat_k(W_q),
                                              _cabi.stream_ptr(W_q.device)))
    return out


def pack_2bit_u8_common(W_q: torch.Tensor) -> torch.Tensor:
    """packing.py:36-41: rows 4R..4R+3 -> bits 7-6, 5-4, 3-2, 1-0 of row R."""
    assert W_q.size(0) % 4 == 0
    W_q = _prep(W_q, torch.uint8)
    out = torch.empty((W_q.size(0) // 4,) + W_q.shape[1:], dtype=torch.uint8, device=W_q.device)
    _cabi.check(_cabi.lib().hqm_pack_2bit_u8(_cabi.ptr(out), _cabi.ptr(W_q), W_q.size(0), _flat_k(W_q),
                                            _cabi.stream_ptr(W_q.device)))
    return out


def unpack_2bit_u8_common(W_q: torch.Tensor) -> torch.Tensor:
    """packing.py:43-53."""
    W_q = _prep(W_q, torch.uint8)
    out = torch.empty((4 * W_q.size(0),) + W_q.shape[1:], dtype=torch.uint8, device=W_q.device)
    _cabi.check(_cabi.lib().hqm_unpack_2bit_u8(_cabi.ptr(out), _cabi.ptr(W_q), W_q.size(0), _flat_k(W_q),
                                              _cabi.stream_ptr(W_q.device)))
    return out


def pack_3bit_i32_common(W_q: torch.Tensor) -> torch.Tensor:
    """packing.py:62-81: ten codes per int32, row 10R+i at bits 3*(9-i); the tail of the last word is zero."""
    W_q = _prep(W_q, torch.uint8)
    rows = (W_q.size(0) + 9) // 10
    out = torch.empty((rows,) + W_q.shape[1:], dtype=torch.int32, device=W_q.device)
    _cabi.check(_cabi.lib().hqm_pack_3bit_i32(_cabi.ptr(out), _cabi.ptr(W_q), W_q.size(0), _flat_k(W_q),
                                             _cabi.stream_ptr(W_q.device)))
    return out


def unpack_3bit_i32_common(W_q: torch.Tensor) -> torch.Tensor:
    """packing.py:83-97: returns 10 * rows rows; callers slice [:N]."""
    assert W_q.dtype == torch.int32
    W_q = _prep(W_q, torch.int32)
    out = torch.empty((10 * W_q.size(0),) + W_q.shape[1:], dtype=torch.uint8, device=W_q.device)
    _cabi.check(_cabi.lib().hqm_unpack_3bit_i32(_cabi.ptr(out), _cabi.ptr(W_q), W_q.size(0), _flat_k(W_q),
                                               _cabi.stream_ptr(W_q.device)))
    return out


PACK = {"4bit_u8": pack_4bit_u8_common, "2bit_u8": pack_2bit_u8_common, "3bit_32": pack_3bit_i32_common}
UNPACK = {"4bit_u8": unpack_4bit_u8_common, "2bit_u8": unpack_2bit_u8_common, "3bit_32": unpack_3bit_i32_common}
BIT_TO_PACKING = {4: "4bit_u8", 3: "3bit_32", 2: "2bit_u8"}
