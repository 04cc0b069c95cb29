"""Checkpoint directories in the reference's layout (src/build_model.py:137-163, 194-202): index file, one trunk
file, one file per expert, Hugging Face Mixtral names; written and read back without the hub."""
import json
import os

import numpy as np
import pytest
import torch

from mixtral_offloading_b200 import HQQLinearTritonSavable, MixtralExpertWrapper
from mixtral_offloading_b200 import checkpoint as ckpt
from tests.helpers import fill_layer, quant_config, random_layer

HD = 128


def _cfg(hidden, ffn, n_heads, n_kv, layers, experts, vocab):
    return dict(hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers, vocab_size=vocab,
                num_attention_heads=n_heads, num_key_value_heads=n_kv, head_dim=HD, num_local_experts=experts,
                num_experts_per_tok=2, rope_theta=1e6, rms_norm_eps=1e-5, hidden_act="silu",
                attn_quant={"nbits": 4, "group_size": 64}, ffn_quant={"nbits": 2, "group_size": 16})


def _linear(od, device):
    cfg = quant_config(od["nbits"], od["group_size"])
    return fill_layer(HQQLinearTritonSavable(None, cfg, HQQLinearTritonSavable.get_hqq_meta((od["K"], od["N"]), cfg)), od, device)


def _model_parts(device, hidden, ffn, n_heads, n_kv, L, E, vocab, seed=0):
    from tests.test_gpu_parity import Cfg
    from mixtral_offloading_b200 import MixtralBLockSparseTop2MLP_HQQ
    g = torch.Generator().manual_seed(seed)
    layers, ods = [], []
    qc = quant_config(2, 16)
    m1 = HQQLinearTritonSavable.get_hqq_meta((hidden, ffn), qc)
    m2 = HQQLinearTritonSavable.get_hqq_meta((ffn, hidden), qc)
    for l in range(L):
        attn_ods = [random_layer(n, k, 4, 64, seed=seed + 10 * l + i, std=0.05) for i, (n, k) in
                    enumerate(((n_heads * HD, hidden), (n_kv * HD, hidden), (n_kv * HD, hidden), (hidden, n_heads * HD)))]
        experts, e_ods = [], []
        for e in range(E):
            trio = (random_layer(ffn, hidden, 2, 16, seed + 1000 * l + 3 * e), random_layer(hidden, ffn, 2, 16, seed + 1000 * l + 3 * e + 1),
                    random_layer(ffn, hidden, 2, 16, seed + 1000 * l + 3 * e + 2))
            ex = MixtralBLockSparseTop2MLP_HQQ(Cfg(hidden, ffn, E), qc, m1, m2)
            for name, od in zip(("w1", "w2", "w3"), trio):
                fill_layer(getattr(ex, name), od, device)
            experts.append(ex)
            e_ods.append(trio)
        layers.append(dict(q=_linear(attn_ods[0], device), k=_linear(attn_ods[1], device), v=_linear(attn_ods[2], device),
                           o=_linear(attn_ods[3], device),
                           ln_in=(1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16),
                           ln_post=(1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16),
                           gate=(0.5 * torch.randn(E, hidden, generator=g)).to(torch.bfloat16), experts=experts))
        ods.append(e_ods)
    embed = torch.randn(vocab, hidden, generator=g).to(torch.bfloat16)
    lm_head = (0.05 * torch.randn(vocab, hidden, generator=g)).to(torch.bfloat16)
    final_norm = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    return layers, ods, embed, lm_head, final_norm


def test_directory_layout_and_expert_round_trip(tmp_path):
    hidden, ffn, n_heads, n_kv, L, E, vocab = 256, 512, 2, 1, 2, 3, 50
    layers, ods, embed, lm_head, final_norm = _model_parts("cpu", hidden, ffn, n_heads, n_kv, L, E, vocab)
    d = str(tmp_path)
    ckpt.save_checkpoint(d, _cfg(hidden, ffn, n_heads, n_kv, L, E, vocab), embed, lm_head, final_norm, layers)
    wm = json.load(open(os.path.join(d, ckpt.INDEX)))["weight_map"]
    # the entries build_model.py looks up: the trunk through the embedding, an expert through its w1.W_q
    trunk_file = wm["model.embed_tokens.weight"]
    assert wm["model.layers.1.self_attn.k_proj.meta.zero_q"] == trunk_file and wm["lm_head.weight"] == trunk_file
    files = {wm[f"{ckpt.expert_prefix(l, e)}.w1.W_q"] for l in range(L) for e in range(E)}
    assert len(files) == L * E and trunk_file not in files
    for l in range(L):
        for e in range(E):
            for w in ("w1", "w2", "w3"):
                for k in ("W_q", "meta.scale_q", "meta.meta_scale.scale", "meta.meta_zero.zero"):
                    assert wm[f"{ckpt.expert_prefix(l, e)}.{w}.{k}"] == wm[f"{ckpt.expert_prefix(l, e)}.w1.W_q"]
    cfg = ckpt.load_config(d)
    wrapped = ckpt.load_expert(d, cfg, cfg.quant_config(), (1, 2), torch.device("cpu"))
    assert isinstance(wrapped, MixtralExpertWrapper)
    for name, od in zip(("w1", "w2", "w3"), ods[1][2]):
        lay = getattr(wrapped._expert, name)
        assert np.array_equal(lay.W_q.numpy(), od["W_q"])
        assert np.array_equal(lay.meta["scale_q"].numpy().reshape(-1), od["scale_q"])
        assert np.array_equal(lay.meta["meta_zero"]["zero"].numpy().reshape(-1), od["mz_zero"])


@pytest.mark.gpu
def test_saved_model_decodes_like_the_one_it_was_saved_from(tmp_path):
    from mixtral_offloading_b200 import AttentionDecode, DecoderLayerDecode, MixtralDecodeModel, ResidentMoe
    from tests.test_gpu_parity import Cfg
    dev = torch.device("cuda:0")
    hidden, ffn, n_heads, n_kv, L, E, vocab, max_len = 512, 1792, 4, 2, 2, 8, 300, 48
    layers, _, embed, lm_head, final_norm = _model_parts(dev, hidden, ffn, n_heads, n_kv, L, E, vocab, seed=5)
    d = str(tmp_path)
    ckpt.save_checkpoint(d, _cfg(hidden, ffn, n_heads, n_kv, L, E, vocab), embed, lm_head, final_norm, layers)
    # the live model
    built = []
    for l, ly in enumerate(layers):
        attn = AttentionDecode(ly["q"], ly["k"], ly["v"], ly["o"], ly["ln_in"].to(dev), ly["ln_post"].to(dev), n_heads, n_kv, HD, max_len)
        gate = torch.nn.Linear(hidden, E, bias=False, dtype=torch.bfloat16, device=dev)
        gate.weight.data = ly["gate"].to(dev)
        nxt = layers[l + 1]["ln_in"] if l + 1 < L else final_norm
        built.append(DecoderLayerDecode(attn, ResidentMoe(Cfg(hidden, ffn, E), l, gate, ly["experts"]), nxt.to(dev)))
    live = MixtralDecodeModel(embed.to(dev), built, layers[0]["ln_in"].to(dev), lm_head.to(dev))
    loaded = ckpt.load_decode_model(d, dev, max_len)
    prompt = [3, 17, 250, 9]
    assert loaded.generate(prompt, 10, use_graph=False) == live.generate(prompt, 10, use_graph=False)
    assert loaded.generate(prompt, 10, use_graph=True) == live.generate(prompt, 10, use_graph=False)


@pytest.mark.gpu
def test_build_model_offloaded_decodes_like_resident_with_and_without_speculation(tmp_path):
    """build_model (build_model.py:166-241): 3 of 8 experts per layer in host memory, LRU swaps; the logits follow
    the resident decoder's on the same fed tokens, and speculative loading changes traffic, not results."""
    from mixtral_offloading_b200 import OffloadConfig
    from oracle import hqq_oracle as O
    dev = torch.device("cuda:0")
    hidden, ffn, n_heads, n_kv, L, E, vocab, max_len = 512, 1792, 4, 2, 3, 8, 300, 48
    layers, _, embed, lm_head, final_norm = _model_parts(dev, hidden, ffn, n_heads, n_kv, L, E, vocab, seed=9)
    d = str(tmp_path)
    ckpt.save_checkpoint(d, _cfg(hidden, ffn, n_heads, n_kv, L, E, vocab), embed, lm_head, final_norm, layers)
    resident = ckpt.load_decode_model(d, dev, max_len)
    off = 3
    oc = OffloadConfig(main_size=L * (E - off), offload_size=L * off, buffer_size=4, offload_per_layer=off)
    fed = [3, 17, 250, 9, 44, 120, 7, 299, 51, 8, 200, 13]

    def run(model):
        out = []
        model.position.zero_()
        for t in fed:
            model.token.fill_(t)
            out.append(model.step().float().cpu())
        return torch.cat(out)
    want = run(resident)
    results = {}
    for speculate in (False, True):
        model = ckpt.build_model(dev, None, oc, d, max_len=max_len, speculate=speculate)
        got = run(model)
        cache = model.expert_cache
        hits = sum(cache.group_infos[l].hits for l in range(L))
        misses = sum(cache.group_infos[l].misses for l in range(L))
        assert hits + misses == 2 * L * len(fed)
        assert all(len(cache.group_infos[l].resident) == E - off for l in range(L))
        results[speculate] = (got, hits, misses, cache.prefetch_stats(), cache.stats())
        assert O.rel_err(got, want) < 2e-2, O.rel_err(got, want)
        assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.9
        del model
    assert torch.equal(results[False][0], results[True][0])
    assert results[False][3] == (0, 0, 0)
    issued, used, wasted = results[True][3]
    assert issued > 0 and used + wasted <= issued
    print("misses without / with speculation:", results[False][2], results[True][2], "prefetch:", results[True][3])
    assert _hqm_device_error() == 0


def _hqm_device_error():
    from mixtral_offloading_b200 import _cabi
    return _cabi.lib().hqm_device_error()
