"""CPU oracle for the steps either side of the MoE block in a decoder layer.  TEST INFRASTRUCTURE ONLY.

The reference takes these steps from the Hugging Face Mixtral decoder layer that src/build_model.py:166-241
assembles (its q/k/v/o projections are the reference's HQQLinearTritonSavable, custom_layers.py:49-92).  This
file restates that layer's arithmetic for ONE new token against a key/value cache, in plain torch on the CPU:

  rms_norm        transformers/models/mixtral/modeling_mixtral.py:139-156  (MixtralRMSNorm.forward)
  rope_cos_sin    modeling_mixtral.py:207-226  (MixtralRotaryEmbedding.forward, default rope, cat(freqs, freqs))
  apply_rope      modeling_mixtral.py:229-262  (rotate_half, apply_rotary_pos_emb)
  attention_step  modeling_mixtral.py:265-352  (repeat_kv, eager_attention_forward, MixtralAttention.forward)
  decoder_layer_step  modeling_mixtral.py MixtralDecoderLayer.forward: residual + attention, residual + MoE block,
                  the MoE block being SparseMoeWrapper.forward of the reference (oracle/hqq_oracle.py:moe_forward)

Parity status: pinned against the installed transformers (5.5.0) run in fp32 on the CPU
(tests/golden/attention_hf.npz, written by tests/golden/make_attention_golden.py;
tests/test_oracle_golden.py checks this file against it).  The reference pins transformers 4.36.1, which is
not installed; the arithmetic of these functions is the same in both.

`round_to` = a torch dtype makes every tensor the Hugging Face layer would hold in the model dtype take that
dtype's rounding (projection outputs, cos / sin, the two products and the sum of the rotation, the context,
the residual stream, the norm's two casts).  Attention scores and probabilities stay in fp32, as fused attention
kernels keep them (the Hugging Face eager path rounds them to the model dtype as well).  With round_to=None
everything is fp32.
"""
from __future__ import annotations

import math

import torch

from . import hqq_oracle as O


def _rnd(t: torch.Tensor, round_to):
    return t if round_to is None else t.to(round_to).to(torch.float32)


def rms_norm(h: torch.Tensor, weight: torch.Tensor, eps: float, round_to=None) -> torch.Tensor:
    """weight * cast(h * rsqrt(mean(h^2) + eps)): the normalisation in fp32, one rounding of the normalised
    value and one of the product (modeling_mixtral.py:149-154)."""
    v = h.to(torch.float32)
    v = _rnd(v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps), round_to)
    return _rnd(weight.to(torch.float32) * v, round_to)


def rope_cos_sin(pos, head_dim: int, theta: float, round_to=None):
    """cos / sin rows of position(s) `pos` (int or 1-D tensor): inv_freq = theta^(-2i/d), emb = cat(freqs, freqs)
    (modeling_mixtral.py:198-226)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).to(torch.float32) / head_dim))
    p = torch.as_tensor(pos, dtype=torch.float32).reshape(-1, 1)
    freqs = p * inv[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return _rnd(emb.cos(), round_to), _rnd(emb.sin(), round_to)


def apply_rope(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, round_to=None) -> torch.Tensor:
    """(t * cos) + (rotate_half(t) * sin) over the last dimension (modeling_mixtral.py:229-262).
    t: (..., heads, head_dim); cos / sin broadcast over heads."""
    half = t.shape[-1] // 2
    rot = torch.cat((-t[..., half:], t[..., :half]), dim=-1)
    return _rnd(_rnd(t * cos, round_to) + _rnd(rot * sin, round_to), round_to)


class AttentionOracle:
    """One attention block with its own key/value cache, fed one token at a time.

    Wq, Wk, Wv, Wo: float (N, K) weights (for a quantized layer: oracle.hqq_oracle.dequantize)."""

    def __init__(self, Wq, Wk, Wv, Wo, n_heads: int, n_kv: int, head_dim: int, max_len: int, theta: float = 1e6,
                 round_to=torch.bfloat16):
        self.W = [w.to(torch.float32) for w in (Wq, Wk, Wv, Wo)]
        self.nh, self.nkv, self.hd, self.theta, self.round_to = n_heads, n_kv, head_dim, theta, round_to
        self.kc = torch.zeros(n_kv, max_len, head_dim)
        self.vc = torch.zeros(n_kv, max_len, head_dim)

    def step(self, x: torch.Tensor, pos: int) -> torch.Tensor:
        """x: (1, hidden) the normalised input of the token at position pos.  Appends its key / value to the
        cache and returns o_proj(attention) (1, hidden) (modeling_mixtral.py:306-352, eager path :265-288)."""
        r = self.round_to
        x = x.to(torch.float32)
        q = _rnd(x @ self.W[0].t(), r).view(self.nh, self.hd)
        k = _rnd(x @ self.W[1].t(), r).view(self.nkv, self.hd)
        v = _rnd(x @ self.W[2].t(), r).view(self.nkv, self.hd)
        cos, sin = rope_cos_sin(pos, self.hd, self.theta, r)
        q, k = apply_rope(q, cos, sin, r), apply_rope(k, cos, sin, r)
        self.kc[:, pos], self.vc[:, pos] = k, v
        grp = self.nh // self.nkv
        K = self.kc[:, :pos + 1].repeat_interleave(grp, 0)                  # repeat_kv: (heads, len, head_dim)
        V = self.vc[:, :pos + 1].repeat_interleave(grp, 0)
        scores = torch.einsum("hd,hld->hl", q, K) * (1.0 / math.sqrt(self.hd))
        p = torch.softmax(scores, dim=-1, dtype=torch.float32)
        ctx = _rnd(torch.einsum("hl,hld->hd", p, V), r).reshape(1, -1)
        return _rnd(ctx @ self.W[3].t(), r)


class DecoderLayerOracle:
    """MixtralDecoderLayer.forward for one token: h += attention(norm(h)); h += moe(norm(h)), with the MoE block
    of the reference (custom_layers.py:272-314 through oracle.hqq_oracle.moe_forward).

    attn_ods: the four quantized projections (q, k, v, o) as oracle layer dictionaries; experts: list of
    (w1, w2, w3) dictionaries; gate_w (E, hidden); ln_in / ln_post: norm weights."""

    def __init__(self, attn_ods, ln_in, ln_post, gate_w, experts, n_heads, n_kv, head_dim, max_len, theta=1e6,
                 eps=1e-5, round_to=torch.bfloat16):
        self.attn = AttentionOracle(*[O.dequantize(od) for od in attn_ods], n_heads, n_kv, head_dim, max_len, theta,
                                    round_to)
        self.ln_in, self.ln_post, self.gate_w, self.experts = ln_in, ln_post, gate_w, experts
        self.eps, self.round_to = eps, round_to

    def step(self, h: torch.Tensor, pos: int, routing=None, x_in=None):
        """h: (1, hidden) residual stream.  Returns (h_out, parts) where parts holds the intermediate tensors
        (x_in, attn_out, h_mid, x_moe, router_logits, moe_out).  `routing` = (weights, indices) replaces the
        router's own decision; `x_in` replaces rms_norm(h) * ln_in (when the caller normalised already)."""
        r = self.round_to
        h = h.to(torch.float32)
        x = rms_norm(h, self.ln_in, self.eps, r) if x_in is None else x_in.to(torch.float32)
        attn_out = self.attn.step(x, pos)
        h_mid = _rnd(h + attn_out, r)
        x_moe = rms_norm(h_mid, self.ln_post, self.eps, r)
        moe_out, logits = O.moe_forward(x_moe, self.gate_w, self.experts, round_to=r, routing=routing)
        moe_out = _rnd(moe_out, r)
        h_out = _rnd(h_mid + moe_out, r)
        return h_out, dict(x_in=x, attn_out=attn_out, h_mid=h_mid, x_moe=x_moe, router_logits=logits, moe_out=moe_out)
