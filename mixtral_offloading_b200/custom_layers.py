"""Drop-in counterparts of the reference's src/custom_layers.py classes, computing
through the C-ABI CUDA library (no Triton, no eager-torch compute path).

  HQQLinearTritonSavable          custom_layers.py:16-240
  MixtralBLockSparseTop2MLP_HQQ   custom_layers.py:243-256
  SparseMoeWrapper                custom_layers.py:259-314

Activations are bf16 (the reference is fp16 end to end); fp16 / fp32 inputs are
converted on the way in and the result is cast back.
"""
from __future__ import annotations

import copy
import ctypes as C
from typing import Any, Dict, Optional

import torch
from torch import nn

from . import _cabi, packing
from .quantize import affine_quantize, meta_template

_SCRATCH: Dict[Any, torch.Tensor] = {}
_SCRATCH_RETIRED: list = []


def _scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """Grow-only per-device workspace handed to the library (which never allocates).

    A buffer that has been outgrown is kept alive, not freed: a captured CUDA graph may still hold its address
    (a decode step captured before a larger request, e.g. a long prompt, arrives).  Growth is geometric, so the
    retired buffers together stay below the size of the current one.  The first hqm_scratch_header_bytes() bytes
    of every buffer are library state that has to start at zero (hqm_scratch_init)."""
    key = (device.type, device.index)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(nbytes, 1 << 20, 0 if buf is None else 2 * buf.numel())
        if buf is not None:
            _SCRATCH_RETIRED.append(buf)
        with torch.inference_mode(False):
            buf = torch.empty(size, dtype=torch.uint8, device=device)
        _cabi.check(_cabi.lib().hqm_scratch_init(_cabi.ptr(buf), _cabi.stream_ptr(device)))
        _SCRATCH[key] = buf
    return buf


def _as_bf16_2d(x: torch.Tensor, K: int) -> torch.Tensor:
    _cabi.require_cuda(x)
    assert x.shape[-1] == K, f"last dimension {x.shape[-1]} != in_features {K}"
    x2 = x.reshape(-1, K)
    if x2.dtype != torch.bfloat16:
        x2 = x2.to(torch.bfloat16)
    return x2.contiguous()


class HQQLinearTritonSavable(nn.Module):
    """Quantized linear layer holding W_q and meta exactly as the reference does after repack().

    meta keys: shape (N, K), nbits, group_size, axis (0), packing, quant_scale, quant_zero,
    scale_q, zero_q (uint8, (256, G*K/256)), meta_scale / meta_zero = {scale, zero (fp16,
    (1, G*K/256)), nbits, group_size, shape, axis, packing}.
    """

    def __init__(self, layer, quant_config, meta=None, **kwargs):
        super().__init__()
        assert quant_config["weight_quant_params"]["nbits"] in [2, 3, 4]       # custom_layers.py:24
        self.quant_config = copy.deepcopy(quant_config)
        self.ready = False
        self.bias = None
        self.W_q = None
        self._desc = None
        if layer is not None:
            self.bias = None if layer.bias is None else layer.bias.detach().to(torch.bfloat16)
            self.quantize(layer.weight.data, **self.quant_config)
        else:
            assert meta is not None                                            # custom_layers.py:28-30
            self.meta = copy.deepcopy(meta)
        self._register_state_dict_hook(self._add_to_state_dict_hook)
        self._register_load_state_dict_pre_hook(self._load_from_state_dict_hook)

    # ------------------------------------------------------------------ build
    def quantize(self, W, weight_quant_params, scale_quant_params, zero_quant_params):
        """custom_layers.py:35-39 (hqq's quantize followed by repack); the packed tensor comes
        out in its final (N/per, K) layout directly."""
        if scale_quant_params is None or zero_quant_params is None:
            raise NotImplementedError("the CUDA kernels decode 8-bit scale and zero; quant_scale and "
                                      "quant_zero must both be set (as every reference config does)")
        _cabi.require_cuda(W)
        N, K = W.shape
        meta = meta_template((N, K), {"weight_quant_params": weight_quant_params,
                                      "scale_quant_params": scale_quant_params,
                                      "zero_quant_params": zero_quant_params})
        codes, scale, zero = affine_quantize(W, meta["nbits"], meta["group_size"])
        self.W_q = packing.PACK[meta["packing"]](codes.reshape(N, K))
        for name, vec in (("scale", scale), ("zero", zero)):
            mm = meta["meta_" + name]
            q, ms, mz = affine_quantize(vec, 8, mm["group_size"])
            meta[name + "_q"] = q.contiguous()
            mm["scale"], mm["zero"] = ms.to(torch.float16).contiguous(), mz.to(torch.float16).contiguous()
        self.meta = meta
        self.ready = True
        self._desc = None

    def repack(self):
        """custom_layers.py:41-47: bring a tensor packed over the (group_size, G*K) code matrix
        into the (N/per, K) layout.  A tensor already in that layout is left alone."""
        N, K = self.meta["shape"]
        per = {2: 4, 3: 10, 4: 2}[self.meta["nbits"]]
        if tuple(self.W_q.shape) == ((N + per - 1) // per, K):
            return
        codes = packing.UNPACK[self.meta["packing"]](self.W_q)
        codes = codes.reshape((-1, K))[:N]
        self.W_q = packing.PACK[self.meta["packing"]](codes)
        self._desc = None

    @classmethod
    def get_hqq_meta(cls, linear_shape, quant_config):
        """custom_layers.py:118-134.  linear_shape is (in_features, out_features) as passed to
        nn.Linear; the reference quantises a throw-away layer to harvest this dictionary."""
        return meta_template((linear_shape[1], linear_shape[0]), quant_config)

    # ---------------------------------------------------------------- compute
    def descriptor(self) -> _cabi.HqmWeight:
        """The struct hqm_weight for the tensors this layer currently points at."""
        m = self.meta
        ms, mz = m["meta_scale"], m["meta_zero"]
        key = (self.W_q.data_ptr(), m["scale_q"].data_ptr(), m["zero_q"].data_ptr(), ms["scale"].data_ptr(),
               ms["zero"].data_ptr(), mz["scale"].data_ptr(), mz["zero"].data_ptr())
        if self._desc is None or self._desc[0] != key:
            _cabi.require_cuda(self.W_q, m["scale_q"], m["zero_q"], ms["scale"], ms["zero"], mz["scale"], mz["zero"])
            if not (m.get("quant_scale") and m.get("quant_zero")):
                raise NotImplementedError("layer without 8-bit scale/zero")
            N, K = m["shape"]
            L = (N // m["group_size"]) * K
            # the meta group sizes are what the TENSORS say (a loaded checkpoint may differ from the template, and
            # scale and zero may differ from each other): one fp16 (scale, zero) pair per column of the (group, L/group) view
            groups = []
            for name, q, mm in (("scale", m["scale_q"], ms), ("zero", m["zero_q"], mz)):
                if q.numel() != L or q.dtype != torch.uint8 or not q.is_contiguous():
                    raise ValueError(f"{name}_q holds {q.numel()} values of {q.dtype}, expected {L} contiguous uint8")
                cols = mm["scale"].numel()
                if cols == 0 or L % cols != 0 or mm["zero"].numel() != cols:
                    raise ValueError(f"meta_{name}: {cols} scale and {mm['zero'].numel()} zero values do not divide "
                                     f"the {L} {name} values into groups")
                for t in (mm["scale"], mm["zero"]):
                    if t.dtype != torch.float16 or not t.is_contiguous():
                        raise ValueError(f"meta_{name} tensors must be contiguous float16")
                groups.append(L // cols)
                mm["group_size"] = L // cols
            d = _cabi.HqmWeight(
                N=N, K=K, nbits=m["nbits"], group_size=m["group_size"],
                meta_group=groups[0], meta_group_zero=0 if groups[1] == groups[0] else groups[1],
                W_q=self.W_q.data_ptr(), scale_q=m["scale_q"].data_ptr(), zero_q=m["zero_q"].data_ptr(),
                ms_scale=ms["scale"].data_ptr(), mz_scale=ms["zero"].data_ptr(),
                ms_zero=mz["scale"].data_ptr(), mz_zero=mz["zero"].data_ptr())
            self._desc = (key, d)
        return self._desc[1]

    def forward(self, x):
        return self.forward_triton(x)

    def set_backend(self, backend):
        pass                                                                   # custom_layers.py:52-53

    @torch.inference_mode()
    def forward_triton(self, x):
        """custom_layers.py:55-92, one fused launch (the name is kept for callers; nothing here is Triton)."""
        assert self.ready, "model was not quantized"
        assert self.meta["axis"] == 0
        N, K = self.meta["shape"]
        x2 = _as_bf16_2d(x, K)
        M = x2.shape[0]
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x2.device)
        d = self.descriptor()
        lib = _cabi.lib()
        need = lib.hqm_linear_scratch_bytes(M, C.byref(d))
        ws = _scratch(x2.device, need) if need else None
        _cabi.check(lib.hqm_linear(_cabi.ptr(y), _cabi.ptr(x2), M, C.byref(d), _cabi.ptr(self.bias),
                                   _cabi.ptr(ws), need, _cabi.stream_ptr(x2.device)))
        y = y.view(x.shape[:-1] + (N,))
        return y if x.dtype == torch.bfloat16 else y.to(x.dtype)

    @torch.inference_mode()
    def dequantize(self, dtype=torch.bfloat16):
        """custom_layers.py:95-116: the full (N, K) weight."""
        assert self.ready, "model was not quantized"
        code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[dtype]
        N, K = self.meta["shape"]
        out = torch.empty((N, K), dtype=dtype, device=self.W_q.device)
        _cabi.check(_cabi.lib().hqm_dequantize(_cabi.ptr(out), code, C.byref(self.descriptor()),
                                               _cabi.stream_ptr(out.device)))
        return out

    # ------------------------------------------------------------- state dict
    _TENSOR_PATHS = (("meta.scale_q", ("scale_q",)), ("meta.meta_scale.scale", ("meta_scale", "scale")),
                     ("meta.meta_scale.zero", ("meta_scale", "zero")), ("meta.zero_q", ("zero_q",)),
                     ("meta.meta_zero.scale", ("meta_zero", "scale")), ("meta.meta_zero.zero", ("meta_zero", "zero")))

    @staticmethod
    def _add_to_state_dict_hook(self, state_dict, prefix, local_metadata):
        """Same keys as custom_layers.py:136-166."""
        if not self.ready:
            return state_dict
        state_dict[prefix + "W_q"] = self.W_q
        if self.bias is not None:
            state_dict[prefix + "bias"] = self.bias
        for key, path in self._TENSOR_PATHS:
            node = self.meta
            for p in path:
                node = node[p]
            state_dict[prefix + key] = node
        return state_dict

    def _load_from_state_dict_hook(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                   error_msgs):
        """custom_layers.py:168-222; tensors must already be in the (N/per, K) layout or in the
        (group_size, G*K)-packed form repack() understands."""
        if prefix + "W_q" not in state_dict:
            return
        self.W_q = state_dict.pop(prefix + "W_q")
        self.bias = state_dict.pop(prefix + "bias") if (prefix + "bias") in state_dict else None
        if self.bias is not None and self.bias.dtype != torch.bfloat16:
            self.bias = self.bias.to(torch.bfloat16)          # the kernels read the bias as bf16 (the reference's is fp16)
        for key, path in self._TENSOR_PATHS:
            node = self.meta
            for p in path[:-1]:
                node = node.setdefault(p, {})
            node[path[-1]] = state_dict.pop(prefix + key)
        self.meta["quant_scale"] = self.meta["quant_zero"] = True
        self.ready = True
        self._desc = None
        if self.W_q.is_cuda:
            self.repack()


class MixtralBLockSparseTop2MLP_HQQ(nn.Module):
    """custom_layers.py:243-256: w2(act(w1 x) * w3 x) — one fused call into the library."""

    def __init__(self, config, quant_config: Dict[str, Any], meta1, meta2):
        super().__init__()
        self.w1 = HQQLinearTritonSavable(None, quant_config, meta1)
        self.w2 = HQQLinearTritonSavable(None, quant_config, meta2)
        self.w3 = HQQLinearTritonSavable(None, quant_config, meta1)
        act = getattr(config, "hidden_act", "silu")
        if act != "silu":
            raise NotImplementedError(f"the fused expert kernel implements SiLU gating, not {act!r}")
        self.act_fn = torch.nn.functional.silu

    @torch.inference_mode()
    def forward_routed(self, x2d, token_idx, route_w, out, accumulate=True):
        """Rows token_idx of x2d through the expert, scaled by route_w, added into the same rows of out."""
        M = x2d.shape[0] if token_idx is None else token_idx.shape[0]
        d1, d2, d3 = self.w1.descriptor(), self.w2.descriptor(), self.w3.descriptor()
        lib = _cabi.lib()
        need = lib.hqm_expert_ffn_scratch_bytes(M, C.byref(d1), C.byref(d2), C.byref(d3))
        ws = _scratch(x2d.device, need)
        _cabi.check(lib.hqm_expert_ffn(_cabi.ptr(out), _cabi.ptr(x2d), M, _cabi.ptr(token_idx), _cabi.ptr(route_w),
                                       1 if accumulate else 0, C.byref(d1), C.byref(d2), C.byref(d3),
                                       _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(x2d.device)))
        return out

    @torch.inference_mode()
    def forward(self, hidden_states):
        K = self.w1.meta["shape"][1]
        x2 = _as_bf16_2d(hidden_states, K)
        out = torch.empty((x2.shape[0], self.w2.meta["shape"][0]), dtype=torch.bfloat16, device=x2.device)
        self.forward_routed(x2, None, None, out, accumulate=False)
        out = out.view(hidden_states.shape[:-1] + (out.shape[-1],))
        return out if hidden_states.dtype == torch.bfloat16 else out.to(hidden_states.dtype)


class SparseMoeWrapper(nn.Module):
    """custom_layers.py:259-314.  Router, token lists and expert FFNs all run on the device; the
    host reads back only the per-expert row counts (it has to know which experts to ask the
    cache for), once per call."""

    def __init__(self, config, layer_id, gate, expert_cache):
        super().__init__()
        self.hidden_dim = config.hidden_size
        self.ffn_dim = config.intermediate_size
        self.num_experts = config.num_local_experts
        self.top_k = config.num_experts_per_tok
        assert self.top_k == 2, "the router kernel implements top-2 routing"
        self.layer_id = layer_id
        self.gate = gate
        self.experts = expert_cache
        self._host_counts = None
        # Speculative loading (README.md:24-27 of the reference lists it as upcoming): when set to the next
        # layer's SparseMoeWrapper, this block also runs that block's router on its own input, reads the guess
        # back with its own counts, and after its experts have been requested asks the cache to start loading the
        # guessed experts of the next layer.  At most SPECULATE_MAX_TOKENS rows (with more, every expert is active).
        self.speculate_next: Optional["SparseMoeWrapper"] = None
        self.speculate_width = 2          # guessed experts per token that are prefetched: 2, or 1 (the likelier only)

    SPECULATE_MAX_TOKENS = 8

    @torch.inference_mode()
    def route(self, x2d):
        """Launch the router; returns device tensors (logits, topk_w, topk_idx, meta, token_idx, token_w)
        where meta = [counts (E), offsets (E+1)] int32."""
        M, K = x2d.shape
        E = self.num_experts
        dev = x2d.device
        gate_w = self.gate.weight
        if gate_w.dtype != torch.bfloat16:
            gate_w = gate_w.to(torch.bfloat16)
        logits = torch.empty((M, E), dtype=torch.bfloat16, device=dev)
        topk_w = torch.empty((M, 2), dtype=torch.float32, device=dev)
        topk_idx = torch.empty((M, 2), dtype=torch.int32, device=dev)
        meta = torch.empty((2 * E + 1,), dtype=torch.int32, device=dev)
        token_idx = torch.empty((2 * M,), dtype=torch.int32, device=dev)
        token_w = torch.empty((2 * M,), dtype=torch.float32, device=dev)
        _cabi.check(_cabi.lib().hqm_router_top2(
            _cabi.ptr(logits), _cabi.ptr(topk_w), _cabi.ptr(topk_idx), _cabi.ptr(meta[:E]), _cabi.ptr(meta[E:]),
            _cabi.ptr(token_idx), _cabi.ptr(token_w), _cabi.ptr(x2d), _cabi.ptr(gate_w.contiguous()), M, K, E,
            _cabi.stream_ptr(dev)))
        return logits, topk_w, topk_idx, meta, token_idx, token_w

    @torch.inference_mode()
    def forward(self, hidden_states: torch.Tensor):
        batch_size, sequence_length, hidden_dim = hidden_states.shape
        x2 = _as_bf16_2d(hidden_states, hidden_dim)
        E = self.num_experts
        logits, _, _, meta, token_idx, token_w = self.route(x2)
        nxt = self.speculate_next if x2.shape[0] <= self.SPECULATE_MAX_TOKENS else None
        if self._host_counts is None:
            with torch.inference_mode(False):     # a normal tensor: it is written from any mode later
                self._host_counts = torch.empty((2 * E + 1 + 2 * self.SPECULATE_MAX_TOKENS,), dtype=torch.int32).pin_memory()
        self._host_counts[:2 * E + 1].copy_(meta, non_blocking=True)
        n_guess = 0
        if nxt is not None:
            guess = nxt.route(x2)[2][:, :self.speculate_width].reshape(-1)
            n_guess = guess.numel()
            self._host_counts[2 * E + 1:2 * E + 1 + n_guess].copy_(guess, non_blocking=True)
        torch.cuda.current_stream(x2.device).synchronize()
        host = self._host_counts.tolist()
        counts, offsets = host[:E], host[E:2 * E + 1]
        final = torch.zeros((x2.shape[0], hidden_dim), dtype=torch.bfloat16, device=x2.device)
        active = [e for e in range(E) if counts[e] > 0]
        for (_layer, e), expert in self.experts.load_experts(*((self.layer_id, e) for e in active), unordered=True):
            lo, hi = offsets[e], offsets[e + 1]
            expert.forward_routed(x2, token_idx[lo:hi], token_w[lo:hi], final, accumulate=True)
        if n_guess:     # after this layer's own copies, so that they are first in line on the copy stream
            self.experts.prefetch(*((nxt.layer_id, e) for e in sorted(set(host[2 * E + 1:2 * E + 1 + n_guess]))))
        final = final.reshape(batch_size, sequence_length, hidden_dim)
        if hidden_states.dtype != torch.bfloat16:
            final, logits = final.to(hidden_states.dtype), logits.to(hidden_states.dtype)
        return final, logits


class ResidentMoe(nn.Module):
    """SparseMoeWrapper.forward for a layer whose experts ALL live on the device (no ExpertCache).

    With nothing to swap, the host does not need to know the routing: for a single token the whole block —
    router, the two chosen experts, weighted sum — runs as one chain of launches that pick the experts on
    the device (hqm_moe_decode), so it can be captured in a CUDA graph.  More tokens take the same
    per-expert loop as SparseMoeWrapper (one read-back of the row counts).
    `experts` is a list of MixtralBLockSparseTop2MLP_HQQ / MixtralExpertWrapper, index = expert id.
    """

    def __init__(self, config, layer_id, gate, experts):
        super().__init__()
        self.hidden_dim = config.hidden_size
        self.num_experts = config.num_local_experts
        assert config.num_experts_per_tok == 2 and len(experts) == self.num_experts
        self.layer_id = layer_id
        self.gate = gate
        self._experts = list(experts)              # kept out of the module registry like the wrapper does
        self._router = SparseMoeWrapper(config, layer_id, gate, expert_cache=None)
        self._table = None
        self._host_counts = None

    @staticmethod
    def _ffn(expert):
        return expert._expert if hasattr(expert, "_expert") else expert

    def invalidate(self):
        """Forget the device-side descriptor table (call after the experts' tensors were replaced or moved)."""
        self._table = None

    @staticmethod
    def _build_table(experts, device):
        """The device-side expert table (hqm_expert_table_build): (w1, w2, w3) of experts[0], experts[1], ..."""
        lib = _cabi.lib()
        n = 3 * len(experts)
        descs = (_cabi.HqmWeight * n)()
        for e, ex in enumerate(experts):
            f = ResidentMoe._ffn(ex)
            for i, lyr in enumerate((f.w1, f.w2, f.w3)):
                descs[3 * e + i] = lyr.descriptor()
        nbytes = lib.hqm_expert_table_bytes(n)
        with torch.inference_mode(False):
            host = torch.empty(nbytes + 64, dtype=torch.uint8)
            off = (-host.data_ptr()) % 64
            _cabi.check(lib.hqm_expert_table_build(C.c_void_p(host.data_ptr() + off), descs, n))
            return host[off:off + nbytes].to(device)

    def _descriptor_table(self, device):
        if self._table is None:
            self._table = self._build_table(self._experts, device)
        return self._table

    @torch.inference_mode()
    def forward(self, hidden_states: torch.Tensor):
        batch, seq, hidden = hidden_states.shape
        x2 = _as_bf16_2d(hidden_states, hidden)
        T, E = x2.shape[0], self.num_experts
        dev = x2.device
        if T == 1:
            f0 = self._ffn(self._experts[0])
            d1, d2, d3 = f0.w1.descriptor(), f0.w2.descriptor(), f0.w3.descriptor()
            lib = _cabi.lib()
            need = lib.hqm_moe_decode_scratch_bytes(E, C.byref(d1), C.byref(d2), C.byref(d3))
            if need:
                gate_w = self.gate.weight if self.gate.weight.dtype == torch.bfloat16 else self.gate.weight.to(torch.bfloat16)
                out = torch.empty((1, hidden), dtype=torch.bfloat16, device=dev)
                logits = torch.empty((1, E), dtype=torch.bfloat16, device=dev)
                ws = _scratch(dev, need)
                _cabi.check(lib.hqm_moe_decode(_cabi.ptr(out), _cabi.ptr(logits), _cabi.ptr(x2), _cabi.ptr(gate_w), E,
                                               _cabi.ptr(self._descriptor_table(dev)), C.byref(d1), C.byref(d2),
                                               C.byref(d3), _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(dev)))
                out = out.reshape(batch, seq, hidden)
                if hidden_states.dtype != torch.bfloat16:
                    out, logits = out.to(hidden_states.dtype), logits.to(hidden_states.dtype)
                return out, logits
        logits, _, _, meta, token_idx, token_w = self._router.route(x2)
        if self._host_counts is None:
            with torch.inference_mode(False):
                self._host_counts = torch.empty((2 * E + 1,), dtype=torch.int32).pin_memory()
        self._host_counts.copy_(meta, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        host = self._host_counts.tolist()
        counts, offsets = host[:E], host[E:]
        final = torch.zeros((T, hidden), dtype=torch.bfloat16, device=dev)
        for e in range(E):
            if counts[e] > 0:
                lo, hi = offsets[e], offsets[e + 1]
                self._experts[e].forward_routed(x2, token_idx[lo:hi], token_w[lo:hi], final, accumulate=True)
        final = final.reshape(batch, seq, hidden)
        if hidden_states.dtype != torch.bfloat16:
            final, logits = final.to(hidden_states.dtype), logits.to(hidden_states.dtype)
        return final, logits
