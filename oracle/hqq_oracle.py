"""CPU oracle for the quantized-expert hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the arithmetic of the reference's quantized
linear / expert FFN / MoE block so that the CUDA path can be checked against
it.  Nothing in the product package may import it; only the tests, the smoke
check and the benchmark's CPU-baseline legs do.

Parity status: the reference ships no tests and no golden vectors, and the
HQQ quantiser (hqq @ 37502bea31f2969c6680c0c4a88ca74b3bb234a5, the pinned
third-party dependency) is not available.  The restatement is therefore pinned
against outputs of the reference's own files (packing.py, custom_layers.py,
expert_cache.py, expert_wrapper.py) imported on the CPU under a small stand-in
for the hqq import surface; the generated vectors live in tests/golden/ next
to the script that made them.  The *quantiser* (how codes / scale / zero are
produced from a float weight) is defined here, not by hqq: parity with hqq's
solver is unpinned and not claimed.

Layout recap (all follow the reference, file:line in each function):
  W        : (N, K) = (out_features, in_features)
  codes    : uint8 (N, K), values in [0, 2**nbits)
  W_q      : codes packed along N, K contiguous:
             4-bit uint8 (N/2, K), 2-bit uint8 (N/4, K), 3-bit int32 (ceil(N/10), K)
  scale/zero: one value per (n % G, k), G = N / group_size; i.e. a quantisation
             group is the `group_size` rows {j*G + r} at one input column k
  scale_q/zero_q: uint8, the flat (G*K,) scale (zero) vector quantised to 8 bit
             in groups of `meta_group` along axis 0 of its (meta_group, G*K/meta_group)
             view, with one fp16 (scale, zero) pair per column of that view
"""
from __future__ import annotations

import numpy as np
import torch

CODES_PER_WORD = {2: 4, 3: 10, 4: 2}


# --------------------------------------------------------------------------- #
# bit packing (bit-exact)                                                      #
# --------------------------------------------------------------------------- #
def pack_4bit_u8(codes: np.ndarray) -> np.ndarray:
    """packing.py:10-17 — even rows go to the high nibble, odd rows to the low."""
    codes = np.asarray(codes, dtype=np.uint8)
    assert codes.shape[0] % 2 == 0
    return ((codes[0::2] << 4) | codes[1::2]).astype(np.uint8)


def unpack_4bit_u8(packed: np.ndarray) -> np.ndarray:
    """packing.py:19-27."""
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty((2 * packed.shape[0],) + packed.shape[1:], dtype=np.uint8)
    out[0::2] = packed >> 4
    out[1::2] = packed & 0xF
    return out


def pack_2bit_u8(codes: np.ndarray) -> np.ndarray:
    """packing.py:36-41 — row n%4==0 in bits 7-6 ... n%4==3 in bits 1-0."""
    codes = np.asarray(codes, dtype=np.uint8)
    assert codes.shape[0] % 4 == 0
    return ((codes[0::4] << 6) | (codes[1::4] << 4) | (codes[2::4] << 2) | codes[3::4]).astype(np.uint8)


def unpack_2bit_u8(packed: np.ndarray) -> np.ndarray:
    """packing.py:43-53."""
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty((4 * packed.shape[0],) + packed.shape[1:], dtype=np.uint8)
    out[0::4] = (packed >> 6) & 3
    out[1::4] = (packed >> 4) & 3
    out[2::4] = (packed >> 2) & 3
    out[3::4] = packed & 3
    return out


def pack_3bit_i32(codes: np.ndarray) -> np.ndarray:
    """packing.py:62-81 — ten codes per int32, row n%10==i at bits 3*(9-i)+2..3*(9-i);
    bits 31-30 stay zero; rows past the end of the last word are zero."""
    codes = np.asarray(codes, dtype=np.uint8)
    n = codes.shape[0]
    rows = (n + 9) // 10
    padded = np.zeros((rows * 10,) + codes.shape[1:], dtype=np.int32)
    padded[:n] = codes
    out = np.zeros((rows,) + codes.shape[1:], dtype=np.int32)
    for i in range(10):
        out |= padded[i::10] << (3 * (9 - i))
    return out


def unpack_3bit_i32(packed: np.ndarray) -> np.ndarray:
    """packing.py:83-97 — returns 10*rows rows; callers slice [:N] (custom_layers.py:46,106)."""
    packed = np.asarray(packed)
    assert packed.dtype == np.int32
    out = np.empty((10 * packed.shape[0],) + packed.shape[1:], dtype=np.uint8)
    for i in range(10):
        out[i::10] = (packed >> (3 * (9 - i))) & 7
    return out


PACK = {2: pack_2bit_u8, 3: pack_3bit_i32, 4: pack_4bit_u8}
UNPACK = {2: unpack_2bit_u8, 3: unpack_3bit_i32, 4: unpack_4bit_u8}


# --------------------------------------------------------------------------- #
# quantiser (defined by this build, see module docstring)                      #
# --------------------------------------------------------------------------- #
def _affine_quantize(t: torch.Tensor, nbits: int, group: int):
    """Min/max affine round-to-nearest over axis 0 of the (group, -1) view.

    Takes the place of hqq's Quantizer.quantize as called from
    custom_layers.py:35-39 (weights) and for the 8-bit scale/zero.  Returns
    integer codes of that view, and the *dequantisation* scale and zero so that
    value ~= (code - zero) * scale.
    """
    v = t.detach().to(torch.float32).reshape(group, -1)
    vmin = v.min(dim=0, keepdim=True).values
    vmax = v.max(dim=0, keepdim=True).values
    qmax = float(2 ** nbits - 1)
    q_scale = (qmax / (vmax - vmin)).clamp(max=2e4)
    zero = -vmin * q_scale
    codes = torch.round(v * q_scale + zero).clamp(0, qmax).to(torch.uint8)
    return codes, (1.0 / q_scale), zero


def quantize(W: torch.Tensor, nbits: int, group_size: int, meta_group: int = 256, meta_group_zero=None) -> dict:
    """Quantise a float (N, K) weight into the layer dictionary used everywhere here.

    Keys: N, K, nbits, group_size, meta_group, codes (uint8 (N,K)), W_q (packed),
    scale_q / zero_q (uint8 (G*K,)), ms_scale, mz_scale, ms_zero, mz_zero
    (fp16 (G*K/meta_group,)).  The tensor names follow custom_layers.py:139-162
    (scale_q, meta_scale.{scale,zero}, zero_q, meta_zero.{scale,zero}).  meta_group_zero gives the zero vector its
    own 8-bit group size (the reference's notebook overrides the scale's group size only, so the two can differ).
    """
    N, K = W.shape
    assert N % group_size == 0
    G = N // group_size
    L = G * K
    assert L % meta_group == 0
    codes, scale, zero = _affine_quantize(W, nbits, group_size)          # (g, G*K), (1, L), (1, L)
    codes = codes.reshape(N, K).contiguous()                             # custom_layers.py:44-45
    sq, ms_s, mz_s = _affine_quantize(scale, 8, meta_group)              # (meta_group, L/meta_group)
    zq, ms_z, mz_z = _affine_quantize(zero, 8, meta_group_zero or meta_group)
    return dict(
        N=N, K=K, nbits=nbits, group_size=group_size, meta_group=meta_group,
        **({"meta_group_zero": meta_group_zero} if meta_group_zero and meta_group_zero != meta_group else {}),
        codes=codes.numpy(),
        W_q=PACK[nbits](codes.numpy()),
        scale_q=sq.reshape(-1).contiguous().numpy(), zero_q=zq.reshape(-1).contiguous().numpy(),
        ms_scale=ms_s.reshape(-1).to(torch.float16).numpy(), mz_scale=mz_s.reshape(-1).to(torch.float16).numpy(),
        ms_zero=ms_z.reshape(-1).to(torch.float16).numpy(), mz_zero=mz_z.reshape(-1).to(torch.float16).numpy(),
    )


# --------------------------------------------------------------------------- #
# decode                                                                       #
# --------------------------------------------------------------------------- #
def meta_dequant(q: np.ndarray, ms: np.ndarray, mz: np.ndarray, meta_group: int) -> torch.Tensor:
    """8-bit scale/zero -> fp32 flat (G*K,) vector.

    custom_layers.py:64,66 call hqq's Quantizer.dequantize(scale_q, meta_scale)
    on every forward; its arithmetic is (code - zero) * scale over the
    (meta_group, -1) view.  The reference does it in fp16; the oracle keeps the
    fp16-stored (ms, mz) but multiplies in fp32.
    """
    qv = torch.from_numpy(np.asarray(q)).to(torch.float32).reshape(meta_group, -1)
    ms_t = torch.from_numpy(np.asarray(ms)).to(torch.float32).reshape(1, -1)
    mz_t = torch.from_numpy(np.asarray(mz)).to(torch.float32).reshape(1, -1)
    return ((qv - mz_t) * ms_t).reshape(-1)


def scale_zero(layer: dict):
    """fp32 (G, K) scale and zero of a layer (custom_layers.py:83-84 views them (-1, K))."""
    K = layer["K"]
    s = meta_dequant(layer["scale_q"], layer["ms_scale"], layer["mz_scale"], layer["meta_group"]).reshape(-1, K)
    z = meta_dequant(layer["zero_q"], layer["ms_zero"], layer["mz_zero"],
                     layer.get("meta_group_zero") or layer["meta_group"]).reshape(-1, K)
    return s, z


def dequantize(layer: dict) -> torch.Tensor:
    """fp32 W_est (N, K), following HQQLinearTritonSavable.dequantize, custom_layers.py:95-116:
    unpack, slice [:N], view (group_size, -1), (code - zero) * scale, view (N, K)."""
    N, K, g = layer["N"], layer["K"], layer["group_size"]
    codes = UNPACK[layer["nbits"]](layer["W_q"])[:N]
    q = torch.from_numpy(codes.astype(np.float32)).reshape(g, -1)
    s, z = scale_zero(layer)
    return ((q - z.reshape(1, -1)) * s.reshape(1, -1)).reshape(N, K)


def dequantize_kernel_indexing(layer: dict) -> torch.Tensor:
    """The same weights, indexed the way the Triton kernels do (triton_kernels.py:84-118,
    279,469): storage row n // per, shift by the slot n % per, scale[n % G, k], zero[n % G, k]."""
    N, K, g, nbits = layer["N"], layer["K"], layer["group_size"], layer["nbits"]
    per = CODES_PER_WORD[nbits]
    G = N // g
    Wq = np.asarray(layer["W_q"]).astype(np.int64)
    n = np.arange(N)
    shift = (per - 1 - (n % per)) * nbits
    q = (Wq[n // per, :] >> shift[:, None]) & (2 ** nbits - 1)
    s, z = scale_zero(layer)
    r = torch.from_numpy(n % G)
    return (torch.from_numpy(q.astype(np.float32)) - z[r]) * s[r]


def linear(x: torch.Tensor, layer: dict) -> torch.Tensor:
    """y = x . W_est^T in fp32 (HQQLinearTritonSavable.forward, custom_layers.py:49-92)."""
    return x.to(torch.float32) @ dequantize(layer).T


def expert_ffn(x: torch.Tensor, w1: dict, w2: dict, w3: dict, round_to=torch.bfloat16) -> torch.Tensor:
    """MixtralBLockSparseTop2MLP_HQQ.forward, custom_layers.py:253-256:
    w2(silu(w1 x) * w3 x).  Each linear's output is rounded to the activation
    dtype as the reference's fp16 layers do (bf16 here)."""
    def rnd(t):
        return t.to(round_to).to(torch.float32) if round_to is not None else t
    a = rnd(linear(x, w1))
    b = rnd(linear(x, w3))
    h = rnd(torch.nn.functional.silu(a) * b)
    return rnd(linear(h, w2))


def router_top2(x: torch.Tensor, gate_w: torch.Tensor, top_k: int = 2, round_to=None):
    """SparseMoeWrapper.forward, custom_layers.py:276-282: gate linear (whose output the
    reference holds in the activation dtype, hence round_to), fp32 softmax, top-k,
    renormalise.  Returns (router_logits, weights, expert indices)."""
    logits = x.to(torch.float32) @ gate_w.to(torch.float32).T
    if round_to is not None:
        logits = logits.to(round_to).to(torch.float32)
    probs = torch.softmax(logits, dim=1, dtype=torch.float32)
    w, idx = torch.topk(probs, top_k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return logits, w, idx


def moe_forward(x: torch.Tensor, gate_w: torch.Tensor, experts: list, round_to=torch.bfloat16, routing=None):
    """SparseMoeWrapper.forward, custom_layers.py:272-314, with every expert resident.
    `experts` is a list of (w1, w2, w3) layer dictionaries.  `routing` = (weights, indices)
    replaces the router's decision (used to take near-ties of rounded logits out of a comparison)."""
    logits, w, idx = router_top2(x, gate_w, round_to=round_to)
    if routing is not None:
        w, idx = routing[0].to(torch.float32), routing[1].to(torch.int64)
    if round_to is not None:
        w = w.to(round_to).to(torch.float32)                              # custom_layers.py:282
    out = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32)
    for e in sorted(set(idx.flatten().tolist())):
        tok, slot = torch.where(idx == e)
        y = expert_ffn(x[tok], *experts[e], round_to=round_to) * w[tok, slot, None]
        out.index_add_(0, tok, y)
    return out, logits


# --------------------------------------------------------------------------- #
# the reference's CPU-runnable path, used as the timed CPU baseline            #
# --------------------------------------------------------------------------- #
def reference_cpu_linear(x: torch.Tensor, layer: dict, dtype=torch.float32) -> torch.Tensor:
    """dequantize() followed by torch.matmul, the CPU path BASELINE names
    (custom_layers.py:95-116 then x @ W_est.T), with torch's own threading."""
    return x.to(dtype) @ dequantize(layer).to(dtype).T


def reference_cpu_expert(x: torch.Tensor, w1: dict, w2: dict, w3: dict) -> torch.Tensor:
    a = reference_cpu_linear(x, w1)
    b = reference_cpu_linear(x, w3)
    return reference_cpu_linear(torch.nn.functional.silu(a) * b, w2)


def rel_err(y: torch.Tensor, y_ref: torch.Tensor) -> float:
    """The parity figure: max|y - y_ref| / max|y_ref|."""
    y = y.to(torch.float32)
    y_ref = y_ref.to(torch.float32)
    return float((y - y_ref).abs().max() / y_ref.abs().max().clamp_min(1e-30))
