"""Generate attention_hf.npz: outputs of the installed transformers' Mixtral decoder-layer pieces, in fp32
on the CPU, for the attention oracle to be pinned against.

    python tests/golden/make_attention_golden.py

It builds MixtralRMSNorm, MixtralRotaryEmbedding and MixtralAttention (eager path) from
transformers.models.mixtral.modeling_mixtral with seeded random weights on a small configuration
(hidden 128, 4 query heads, 2 key/value heads, head_dim 32, theta 1e6, eps 1e-5), runs a sequence of 6 tokens
through norm -> attention (causal mask) -> residual add -> post-attention norm in one pass, and records the
weights, the input and every intermediate tensor.  Feeding the same tokens one at a time against a cache must
give the same rows; that is what tests/test_oracle_golden.py checks on oracle/attention_oracle.py.
"""
import os

import numpy as np
import torch
import transformers
from transformers.models.mixtral import modeling_mixtral as mm
from transformers.models.mixtral.configuration_mixtral import MixtralConfig

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    torch.manual_seed(0)
    hidden, nh, nkv, hd, T, theta, eps = 128, 4, 2, 32, 6, 1e6, 1e-5
    cfg = MixtralConfig(hidden_size=hidden, intermediate_size=512, num_hidden_layers=1, num_attention_heads=nh,
                        num_key_value_heads=nkv, head_dim=hd, num_local_experts=4, num_experts_per_tok=2,
                        rms_norm_eps=eps, rope_theta=theta, max_position_embeddings=64, sliding_window=None,
                        attn_implementation="eager")
    ln_in, ln_post = mm.MixtralRMSNorm(hidden, eps), mm.MixtralRMSNorm(hidden, eps)
    ln_in.weight.data = 1 + 0.1 * torch.randn(hidden)
    ln_post.weight.data = 1 + 0.1 * torch.randn(hidden)
    attn = mm.MixtralAttention(cfg, 0).eval()
    for p in attn.parameters():
        p.data.normal_(0, 0.05)
    rope = mm.MixtralRotaryEmbedding(cfg)
    h = torch.randn(1, T, hidden)
    pos = torch.arange(T)[None]
    with torch.no_grad():
        x = ln_in(h)
        cos, sin = rope(x, pos)
        mask = torch.full((T, T), float("-inf")).triu(1)[None, None]
        o, _ = attn(x, (cos, sin), mask)
        h_mid = h + o
        x_post = ln_post(h_mid)
        q = attn.q_proj(x).view(1, T, nh, hd).transpose(1, 2)
        k = attn.k_proj(x).view(1, T, nkv, hd).transpose(1, 2)
        q_rot, k_rot = mm.apply_rotary_pos_emb(q, k, cos, sin)
    f = lambda t: t.detach().to(torch.float32).numpy()
    np.savez_compressed(
        os.path.join(HERE, "attention_hf.npz"),
        transformers_version=np.array(transformers.__version__),
        hidden=hidden, n_heads=nh, n_kv=nkv, head_dim=hd, tokens=T, theta=theta, eps=eps,
        ln_in=f(ln_in.weight), ln_post=f(ln_post.weight),
        Wq=f(attn.q_proj.weight), Wk=f(attn.k_proj.weight), Wv=f(attn.v_proj.weight), Wo=f(attn.o_proj.weight),
        h=f(h[0]), x=f(x[0]), cos=f(cos[0]), sin=f(sin[0]), q_rot=f(q_rot[0]), k_rot=f(k_rot[0]),
        attn_out=f(o[0]), h_mid=f(h_mid[0]), x_post=f(x_post[0]))
    print("attention_hf.npz written with transformers", transformers.__version__)


if __name__ == "__main__":
    main()
