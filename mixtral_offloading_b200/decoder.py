"""The steps either side of the MoE block for single-token decode, as device-side launch sequences.

In the reference these steps are the Hugging Face Mixtral decoder layer (src/build_model.py:166-241
assembles the model; its q/k/v/o projections are HQQLinearTritonSavable modules,
src/custom_layers.py:49-92).  AttentionDecode runs them for ONE new token without returning to the
host: RMSNorm, the three projections in one streaming launch, rotate-half RoPE, the KV-cache append, the
attention over the cache, the output projection, the residual add and the post-attention RMSNorm
(hqm_attn_decode).  Together with ResidentMoe a whole decode step is a fixed sequence of launches that a
CUDA graph can replay.
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import nn

from . import _cabi
from .custom_layers import HQQLinearTritonSavable, ResidentMoe, _scratch


def _bf16_vec(t: torch.Tensor, n: int) -> torch.Tensor:
    assert t.is_cuda and t.dtype == torch.bfloat16 and t.numel() == n and t.is_contiguous()
    return t


def add_rmsnorm(h: torch.Tensor, delta, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """h += delta (in place, when delta is given); returns rmsnorm(h) * weight.  h: (1, hidden) bf16."""
    hidden = h.shape[-1]
    _bf16_vec(h, hidden), _bf16_vec(weight, hidden)
    if delta is not None:
        _bf16_vec(delta, hidden)
    x = torch.empty_like(h)
    _cabi.check(_cabi.lib().hqm_add_rmsnorm(_cabi.ptr(h), _cabi.ptr(delta) if delta is not None else None,
                                            _cabi.ptr(weight), _cabi.ptr(x), hidden, eps, _cabi.stream_ptr(h.device)))
    return x


def rms_norm_rows(h: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm of every row of h (rows, hidden) bf16 as the decode kernels compute it: fp32 normalisation, one
    rounding to bf16, times the bf16 weight (the Hugging Face form).  One launch (hqm_add_rmsnorm_rows)."""
    rows, hidden = h.shape
    _cabi.require_cuda(h, w)
    if h.dtype != torch.bfloat16 or not h.is_contiguous():
        h = h.to(torch.bfloat16).contiguous()
    _bf16_vec(w, hidden)
    x = torch.empty_like(h)
    _cabi.check(_cabi.lib().hqm_add_rmsnorm_rows(_cabi.ptr(h), None, _cabi.ptr(w), _cabi.ptr(x), rows, hidden, eps,
                                                 _cabi.stream_ptr(h.device)))
    return x


def rope_append_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     n_heads: int, n_kv_heads: int, head_dim: int, theta: float, pos, pos_step: int) -> None:
    """Rotary embedding and cache append of T tokens in one launch (hqm_rope_append_rows): q (T, n_heads * head_dim)
    bf16 is rotated in place; k is rotated and, with v, written into the caches.  A prompt: caches
    (n_kv_heads, max_len, head_dim), pos = position of the first token (int), pos_step = 1.  A batch of sequences
    at one position: caches (T, n_kv_heads, max_len, head_dim), pos = int64 device tensor of one element,
    pos_step = 0."""
    T = q.shape[0]
    for t, n in ((q, n_heads), (k, n_kv_heads), (v, n_kv_heads)):
        assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and t.shape == (T, n * head_dim)
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    max_len = k_cache.shape[-2]
    batch_stride = 0 if k_cache.dim() == 3 else n_kv_heads * max_len * head_dim
    assert k_cache.dim() == 3 or k_cache.shape[0] == T
    on_device = isinstance(pos, torch.Tensor)
    if on_device:
        assert pos.is_cuda and pos.dtype == torch.int64 and pos.numel() == 1
    _cabi.check(_cabi.lib().hqm_rope_append_rows(
        _cabi.ptr(q), _cabi.ptr(k), _cabi.ptr(v), _cabi.ptr(k_cache), _cabi.ptr(v_cache), T, n_heads, n_kv_heads, head_dim,
        max_len, batch_stride, _cabi.ptr(pos) if on_device else None, 0 if on_device else int(pos), pos_step, theta,
        _cabi.stream_ptr(q.device)))


class AttentionDecode(nn.Module):
    """Attention half of a decoder layer for one token at a time, with its own KV cache.

    q, k, v, o: HQQLinearTritonSavable.  ln_in / ln_post: the RMSNorm weights in front of the attention and
    in front of the MoE block (bf16, hidden).  The cache holds `max_len` positions."""

    def __init__(self, q: HQQLinearTritonSavable, k: HQQLinearTritonSavable, v: HQQLinearTritonSavable,
                 o: HQQLinearTritonSavable, ln_in: torch.Tensor, ln_post: torch.Tensor, n_heads: int, n_kv_heads: int,
                 head_dim: int, max_len: int, rope_theta: float = 1e6, rms_eps: float = 1e-5):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = q, k, v, o
        self.ln_in, self.ln_post = ln_in, ln_post
        self.n_heads, self.n_kv_heads, self.head_dim, self.max_len = n_heads, n_kv_heads, head_dim, max_len
        self.rope_theta, self.rms_eps = rope_theta, rms_eps
        dev = ln_in.device
        self.k_cache = torch.zeros((n_kv_heads, max_len, head_dim), dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros((n_kv_heads, max_len, head_dim), dtype=torch.bfloat16, device=dev)
        self._layer, self._layer_key = None, None

    def _descriptor(self) -> _cabi.HqmAttnLayer:
        """struct hqm_attn_layer for the tensors the block currently points at (rebuilt when one of them moved)."""
        projs = [p.descriptor() for p in (self.q_proj, self.k_proj, self.v_proj, self.o_proj)]
        key = tuple(d.W_q for d in projs) + (self.ln_in.data_ptr(), self.ln_post.data_ptr(), self.k_cache.data_ptr(),
                                             self.v_cache.data_ptr())
        if self._layer is None or self._layer_key != key:
            self._layer_key = key
            hidden = self.n_heads * self.head_dim
            self._layer = _cabi.HqmAttnLayer(
                q=self.q_proj.descriptor(), k=self.k_proj.descriptor(), v=self.v_proj.descriptor(),
                o=self.o_proj.descriptor(), ln_in=_bf16_vec(self.ln_in, hidden).data_ptr(),
                ln_post=_bf16_vec(self.ln_post, hidden).data_ptr(), k_cache=self.k_cache.data_ptr(),
                v_cache=self.v_cache.data_ptr(), n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                head_dim=self.head_dim, max_len=self.max_len, rope_theta=self.rope_theta, rms_eps=self.rms_eps)
        return self._layer

    @torch.inference_mode()
    def forward(self, h: torch.Tensor, pos: torch.Tensor, delta=None) -> torch.Tensor:
        """h: (1, hidden) bf16 residual stream, updated in place (h += delta first when delta is given).
        pos: int32 tensor of one element on the device, the position of this token.  Returns the
        post-attention RMSNorm of the updated h: the MoE block's input."""
        hidden = h.shape[-1]
        _bf16_vec(h, hidden)
        assert pos.is_cuda and pos.dtype == torch.int32 and pos.numel() == 1
        if delta is not None:
            _bf16_vec(delta, hidden)
        lib = _cabi.lib()
        layer = self._descriptor()
        need = lib.hqm_attn_decode_scratch_bytes(C.byref(layer))
        if need == 0:
            raise ValueError(lib.hqm_last_error().decode() or "attention decode: unsupported layer")
        ws = _scratch(h.device, need)
        x_out = torch.empty_like(h)
        _cabi.check(lib.hqm_attn_decode(_cabi.ptr(h), _cabi.ptr(x_out), _cabi.ptr(delta) if delta is not None else None,
                                        C.byref(layer), _cabi.ptr(pos), _cabi.ptr(ws), ws.numel(),
                                        _cabi.stream_ptr(h.device)))
        return x_out


class DecoderLayerDecode(nn.Module):
    """One decoder layer for one token: AttentionDecode followed by a ResidentMoe block, with the residual adds
    and norms between and after them, as one launch sequence (hqm_decode_layer).

    attention: an AttentionDecode (its ln_in is the norm the CALLER applies to produce x for the first layer);
    moe: a ResidentMoe; next_ln: the RMSNorm weight applied to the layer's output: the next layer's
    input_layernorm weight, or the model's final norm weight after the last layer."""

    def __init__(self, attention: AttentionDecode, moe: ResidentMoe, next_ln: torch.Tensor):
        super().__init__()
        self.attention, self.moe, self.next_ln = attention, moe, next_ln
        self._layer, self._layer_key = None, None
        self._gate_w = None

    def _descriptor(self, device) -> _cabi.HqmDecoderLayer:
        """struct hqm_decoder_layer; rebuilt when the attention block's tensors, the gate or the norm weight moved.
        (The expert table is built once by ResidentMoe; call moe.invalidate() after replacing expert tensors.)"""
        attn_desc = self.attention._descriptor()
        key = (self.attention._layer_key, self.moe.gate.weight.data_ptr(), self.next_ln.data_ptr(),
               self.moe._descriptor_table(device).data_ptr())
        if self._layer is None or self._layer_key != key:
            self._layer_key = key
            hidden = self.attention.n_heads * self.attention.head_dim
            gate = self.moe.gate.weight
            self._gate_w = gate if gate.dtype == torch.bfloat16 else gate.to(torch.bfloat16)
            f0 = self.moe._ffn(self.moe._experts[0])
            self._layer = _cabi.HqmDecoderLayer(
                attn=attn_desc, gate_w=self._gate_w.data_ptr(),
                table=self.moe._descriptor_table(device).data_ptr(), w1=f0.w1.descriptor(), w2=f0.w2.descriptor(),
                w3=f0.w3.descriptor(), next_ln=_bf16_vec(self.next_ln, hidden).data_ptr(),
                n_experts=self.moe.num_experts, reserved=0)
        return self._layer

    @staticmethod
    def tokens_shared(T: int, pos0: int, device):
        """The attention mask of T tokens at positions pos0 .. pos0 + T - 1: token i sees positions 0 .. pos0 + i."""
        positions = torch.arange(pos0, pos0 + T, device=device)
        return torch.arange(pos0 + T, device=device)[None, :] <= positions[:, None]

    @torch.inference_mode()
    def forward_tokens(self, h: torch.Tensor, pos0: int, ln_in=None, shared=None):
        """T new tokens at once (a prompt, or a chunk of 32 / 256 tokens behind a cache that already holds pos0
        positions): h (T, hidden) bf16 is the residual stream of the tokens at positions pos0 .. pos0 + T - 1.
        The quantized projections and the experts take their many-row (tensor-core) kernels; norms, RoPE and the
        attention over the cache are torch ops; the MoE block groups the tokens per expert.  Appends the tokens'
        keys and values to the cache; returns (updated h, router logits (T, n_experts)).  ln_in: the layer's input
        norm weight when it is not attention.ln_in (a model hands every layer the weight its predecessor was built
        with as next_ln, which is what the one-token path applies).  shared: what tokens_shared() returned for the
        same (T, pos0), when several layers process the same tokens (the mask is the same for all of them)."""
        a = self.attention
        ln_in = a.ln_in if ln_in is None else ln_in
        T, hidden = h.shape
        if pos0 < 0 or pos0 + T > a.max_len:
            raise ValueError(f"{T} tokens at position {pos0} do not fit a cache of {a.max_len}")
        mask = shared if shared is not None else self.tokens_shared(T, pos0, h.device)
        x = rms_norm_rows(h, ln_in, a.rms_eps)
        q = a.q_proj(x)
        rope_append_rows(q, a.k_proj(x), a.v_proj(x), a.k_cache, a.v_cache, a.n_heads, a.n_kv_heads, a.head_dim,
                         a.rope_theta, pos0, 1)
        q = q.view(T, a.n_heads, a.head_dim)
        keys, vals = a.k_cache[:, :pos0 + T].unsqueeze(0), a.v_cache[:, :pos0 + T].unsqueeze(0)
        ctx = torch.nn.functional.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), keys, vals, attn_mask=mask,
                                                               enable_gqa=True)          # (1, heads, T, head_dim)
        h = h + a.o_proj(ctx[0].transpose(0, 1).reshape(T, hidden))
        y, logits = self.moe(rms_norm_rows(h, a.ln_post, a.rms_eps).view(1, T, hidden))
        return h + y.view(T, hidden), logits

    @torch.inference_mode()
    def forward(self, h: torch.Tensor, x: torch.Tensor, pos: torch.Tensor):
        """h: (1, hidden) bf16 residual stream, updated in place.  x: (1, hidden) bf16, on entry the normalised
        input of this layer, on return the normalised input of the next one (updated in place).
        pos: int32 tensor of one element on the device.  Returns the router logits (1, n_experts)."""
        hidden = h.shape[-1]
        _bf16_vec(h, hidden), _bf16_vec(x, hidden)
        assert pos.is_cuda and pos.dtype == torch.int32 and pos.numel() == 1
        lib = _cabi.lib()
        layer = self._descriptor(h.device)
        need = lib.hqm_decode_layer_scratch_bytes(C.byref(layer))
        if need == 0:
            raise ValueError(lib.hqm_last_error().decode() or "decoder layer: unsupported shapes")
        ws = _scratch(h.device, need)
        logits = torch.empty((1, self.moe.num_experts), dtype=torch.bfloat16, device=h.device)
        _cabi.check(lib.hqm_decode_layer(_cabi.ptr(h), _cabi.ptr(x), _cabi.ptr(logits), C.byref(layer), _cabi.ptr(pos),
                                         _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(h.device)))
        return logits


class PeerExchange:
    """The buffers of the expert-parallel exchange over peer memory (struct hqm_ep_comm): every rank allocates
    hqm_ep_exchange_bytes() of symmetric memory (torch.distributed._symmetric_memory: device memory that the other
    ranks of the node map into their address space), zeroes it, and learns its peers' addresses at the rendezvous.
    One object serves all layers of a model (they exchange one after the other)."""

    def __init__(self, group, hidden: int, device: torch.device):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        lib = _cabi.lib()
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        nbytes = lib.hqm_ep_exchange_bytes(self.world, hidden)
        if nbytes == 0:
            raise ValueError(f"expert-parallel exchange: {self.world} ranks / hidden {hidden} not supported")
        with torch.inference_mode(False):
            self.buffer = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=device)
            self.buffer.zero_()
            self.seq = torch.zeros(1, dtype=torch.int32, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, group)
        ptrs = list(self.handle.buffer_ptrs)
        off = lib.hqm_ep_exchange_flags_offset(self.world, hidden)
        comm = _cabi.HqmEpComm(rank=self.rank, world=self.world, hidden=hidden, reserved=0, seq=self.seq.data_ptr())
        for r in range(self.world):
            comm.shares[r] = ptrs[r]
            comm.flags[r] = ptrs[r] + off
        self.comm = comm
        torch.cuda.synchronize(device)
        dist.barrier(group)                      # everybody's buffer is zero before anybody publishes


class ExpertParallelDecoderLayer(nn.Module):
    """DecoderLayerDecode for one rank of an expert-parallel group (torch.distributed): attention, norms and router
    are replicated, the rank holds `experts` = the layer's experts [expert_lo, expert_lo + len(experts)) and runs
    those of the routed pair that are its own, without the host learning the routing (hqm_decode_layer_ep).  The
    ranks' fp32 shares of the block output are added by ONE all-reduce on the compute stream, then the residual
    add and the next layer's norm follow (hqm_add_f32_rmsnorm).  The sequence is fixed, so a decode step with it
    can be captured in a CUDA graph.  The reference has no distributed code; the block that is sharded is
    src/custom_layers.py:272-314.

    attention: AttentionDecode (same weights on every rank); gate: nn.Linear over ALL n_experts (same on every
    rank); next_ln as for DecoderLayerDecode; group: the process group (None: no reduction, a single rank).
    exchange: a PeerExchange; with it the ranks' shares travel by peer stores from inside the library's kernels
    (no collective call, two launches between the experts and the next layer) instead of the NCCL all-reduce."""

    def __init__(self, attention: AttentionDecode, gate, experts, expert_lo: int, n_experts: int, next_ln: torch.Tensor,
                 group=None, exchange=None):
        super().__init__()
        assert 0 <= expert_lo and expert_lo + len(experts) <= n_experts and len(experts) >= 1
        self.attention, self.gate, self.next_ln, self.group = attention, gate, next_ln, group
        self.exchange = exchange
        self.expert_lo, self.n_experts = expert_lo, n_experts
        self._experts = list(experts)
        self._table = None
        self._layer, self._layer_key, self._gate_w = None, None, None
        hidden = attention.n_heads * attention.head_dim
        self.y_partial = torch.zeros((1, hidden), dtype=torch.float32, device=next_ln.device)

    def _descriptor(self, device) -> _cabi.HqmDecoderLayer:
        attn_desc = self.attention._descriptor()
        if self._table is None:
            self._table = ResidentMoe._build_table(self._experts, device)
        key = (self.attention._layer_key, self.gate.weight.data_ptr(), self.next_ln.data_ptr(), self._table.data_ptr())
        if self._layer is None or self._layer_key != key:
            self._layer_key = key
            hidden = self.attention.n_heads * self.attention.head_dim
            gate = self.gate.weight
            self._gate_w = gate if gate.dtype == torch.bfloat16 else gate.to(torch.bfloat16)
            f0 = ResidentMoe._ffn(self._experts[0])
            self._layer = _cabi.HqmDecoderLayer(
                attn=attn_desc, gate_w=self._gate_w.data_ptr(), table=self._table.data_ptr(), w1=f0.w1.descriptor(),
                w2=f0.w2.descriptor(), w3=f0.w3.descriptor(), next_ln=_bf16_vec(self.next_ln, hidden).data_ptr(),
                n_experts=self.n_experts, reserved=0)
        return self._layer

    @torch.inference_mode()
    def forward(self, h: torch.Tensor, x: torch.Tensor, pos: torch.Tensor):
        """Same contract as DecoderLayerDecode.forward."""
        hidden = h.shape[-1]
        _bf16_vec(h, hidden), _bf16_vec(x, hidden)
        assert pos.is_cuda and pos.dtype == torch.int32 and pos.numel() == 1
        lib = _cabi.lib()
        layer = self._descriptor(h.device)
        n_local = len(self._experts)
        need = lib.hqm_decode_layer_ep_scratch_bytes(C.byref(layer), n_local)
        if need == 0:
            raise ValueError(lib.hqm_last_error().decode() or "decoder layer: unsupported shapes")
        ws = _scratch(h.device, need)
        logits = torch.empty((1, self.n_experts), dtype=torch.bfloat16, device=h.device)
        if self.exchange is not None:
            comm = C.byref(self.exchange.comm)
            _cabi.check(lib.hqm_decode_layer_ep(_cabi.ptr(h), _cabi.ptr(x), _cabi.ptr(logits), None, comm, C.byref(layer),
                                                self.expert_lo, n_local, _cabi.ptr(pos), _cabi.ptr(ws), ws.numel(),
                                                _cabi.stream_ptr(h.device)))
            _cabi.check(lib.hqm_ep_combine_add_rmsnorm(_cabi.ptr(h), comm, _cabi.ptr(self.next_ln), _cabi.ptr(x), hidden,
                                                       self.attention.rms_eps, _cabi.stream_ptr(h.device)))
            return logits
        _cabi.check(lib.hqm_decode_layer_ep(_cabi.ptr(h), _cabi.ptr(x), _cabi.ptr(logits), _cabi.ptr(self.y_partial), None,
                                            C.byref(layer), self.expert_lo, n_local, _cabi.ptr(pos), _cabi.ptr(ws),
                                            ws.numel(), _cabi.stream_ptr(h.device)))
        if self.group is not None:
            import torch.distributed as dist
            dist.all_reduce(self.y_partial, group=self.group)
        _cabi.check(lib.hqm_add_f32_rmsnorm(_cabi.ptr(h), _cabi.ptr(self.y_partial), _cabi.ptr(self.next_ln), _cabi.ptr(x),
                                            hidden, self.attention.rms_eps, _cabi.stream_ptr(h.device)))
        return logits
