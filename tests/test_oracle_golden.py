"""The CPU oracle against the fixtures recorded from the reference's own code."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import hqq_oracle as O
from oracle.lru_oracle import LruOracle


def _bf16(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def _layer(z, prefix=""):
    keys = ("W_q", "scale_q", "zero_q", "ms_scale", "mz_scale", "ms_zero", "mz_zero")
    return {k: z[prefix + k] for k in keys}


@pytest.mark.parametrize("nbits,rows", [(4, 64), (2, 64), (3, 64), (3, 60), (3, 7)])
def test_pack_unpack_bit_exact(golden_dir, nbits, rows):
    z = np.load(os.path.join(golden_dir, "packing.npz"))
    codes, packed, unpacked = z[f"codes_{nbits}_{rows}"], z[f"packed_{nbits}_{rows}"], z[f"unpacked_{nbits}_{rows}"]
    mine = O.PACK[nbits](codes)
    assert mine.dtype == packed.dtype and np.array_equal(mine, packed)
    back = O.UNPACK[nbits](packed)
    assert back.dtype == np.uint8 and np.array_equal(back, unpacked)
    assert np.array_equal(back[:rows], codes)


def test_3bit_known_answers(golden_dir):
    z = np.load(os.path.join(golden_dir, "packing.npz"))
    assert int(z["ka_3bit_ten_sevens"][0, 0]) == 0x3FFFFFFF
    assert int(z["ka_3bit_first_seven"][0, 0]) == 0x38000000
    assert int(O.pack_3bit_i32(np.full((10, 1), 7, np.uint8))[0, 0]) == 0x3FFFFFFF
    first = np.zeros((10, 1), np.uint8)
    first[0] = 7
    assert int(O.pack_3bit_i32(first)[0, 0]) == 0x38000000


@pytest.mark.parametrize("nbits", [2, 3, 4])
def test_layer_against_reference(golden_dir, nbits):
    z = np.load(os.path.join(golden_dir, f"layer_{nbits}bit.npz"))
    N, K, g = int(z["N"]), int(z["K"]), int(z["group_size"])
    W = _bf16(z["W_bf16"]).reshape(N, K)
    # the quantiser restated in the oracle produces the reference layer's tensors bit for bit
    mine = O.quantize(W, nbits, g, 256)
    for k in ("W_q", "scale_q", "zero_q", "ms_scale", "mz_scale", "ms_zero", "mz_zero"):
        assert mine[k].dtype == z[k].dtype, k
        assert np.array_equal(mine[k], z[k]), k
    layer = dict(N=N, K=K, nbits=nbits, group_size=g, meta_group=256, **_layer(z))
    # decode: the reference works in fp16, the oracle in fp32
    W_ref = torch.from_numpy(z["W_est_f16"]).float()
    W_est = O.dequantize(layer)
    assert O.rel_err(W_est, W_ref) < 3e-3
    # the Triton kernels' indexing describes the same matrix as dequantize()
    assert torch.equal(O.dequantize_kernel_indexing(layer), W_est)
    # quantisation error itself stays within half a step
    x = _bf16(z["x_bf16"]).reshape(-1, K)
    assert O.rel_err(O.linear(x, layer), torch.from_numpy(z["y_f32"])) < 3e-3


def _experts(z):
    out = []
    hidden, ffn = int(z["hidden"]), int(z["ffn"])
    for e in range(int(z["n_exp"])):
        ws = []
        for name, (N, K) in (("w1", (ffn, hidden)), ("w2", (hidden, ffn)), ("w3", (ffn, hidden))):
            ws.append(dict(N=N, K=K, nbits=2, group_size=16, meta_group=256, **_layer(z, f"e{e}_{name}_")))
        out.append(tuple(ws))
    return out


def test_expert_ffn_and_moe_against_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "expert_moe.npz"))
    hidden = int(z["hidden"])
    experts = _experts(z)
    x = _bf16(z["x_bf16"]).reshape(-1, hidden)
    gate = _bf16(z["gate_bf16"]).reshape(-1, hidden)
    y = O.expert_ffn(x, *experts[0], round_to=torch.float16)
    assert O.rel_err(y, torch.from_numpy(z["ffn0_y_f16"])) < 1e-2
    out, logits = O.moe_forward(x, gate, experts, round_to=torch.float16)
    assert O.rel_err(logits, torch.from_numpy(z["moe_logits_f16"])) < 1e-2
    assert O.rel_err(out, torch.from_numpy(z["moe_y_f16"])) < 1e-2


def test_lru_oracle_against_reference_traces(golden_dir):
    traces = json.load(open(os.path.join(golden_dir, "lru_traces.json")))
    assert len(traces) >= 3
    for tr in traces:
        lru = LruOracle(tr["main_size"], tr["offload_size"], tr["buffer_size"])
        for uid, group, offload in tr["placement"]:
            lru.add(tuple(uid), group, offload)
        for step in tr["steps"]:
            uids = [tuple(u) for u in step["request"]]
            order, swaps, issued = lru.load(uids, unordered=step["unordered"])
            group = uids[0][0]
            assert [list(u) for u in order] == step["order"]
            assert [list(u) for u in lru.resident(group)] == step["resident"]
            assert (lru.hits[group], lru.misses[group]) == (step["hits"], step["misses"])


def test_lru_known_answer_table(golden_dir):
    """One layer, experts 0-3 offloaded / 4-7 resident, 4 buffers, unordered requests."""
    tr = json.load(open(os.path.join(golden_dir, "lru_traces.json")))[0]
    want = [([4, 5], [4, 5], [6, 7, 4, 5], 2, 0), ([0, 5], [5, 0], [7, 4, 5, 0], 3, 1),
            ([1, 2], [1, 2], [5, 0, 1, 2], 3, 3), ([0, 1], [0, 1], [5, 2, 0, 1], 5, 3),
            ([6, 7], [6, 7], [0, 1, 6, 7], 5, 5),
            (list(range(8)), [0, 1, 6, 7, 2, 3, 4, 5], [2, 3, 4, 5], 9, 9), ([3, 4], [3, 4], [2, 5, 3, 4], 11, 9)]
    for step, (req, order, resident, hits, misses) in zip(tr["steps"], want):
        assert [u[1] for u in step["request"]] == req
        assert [u[1] for u in step["order"]] == order
        assert [u[1] for u in step["resident"]] == resident
        assert (step["hits"], step["misses"]) == (hits, misses)


# ---- the attention oracle against the installed transformers' Mixtral layer pieces (fp32, CPU) -------------
def test_attention_oracle_matches_transformers(golden_dir):
    from oracle import attention_oracle as A
    z = np.load(os.path.join(golden_dir, "attention_hf.npz"))
    t = lambda k: torch.from_numpy(z[k])
    nh, nkv, hd, T = int(z["n_heads"]), int(z["n_kv"]), int(z["head_dim"]), int(z["tokens"])
    theta, eps = float(z["theta"]), float(z["eps"])
    h = t("h")
    # RMSNorm and the rotation tables
    x = A.rms_norm(h, t("ln_in"), eps)
    assert torch.allclose(x, t("x"), atol=1e-6, rtol=1e-5)
    cos, sin = A.rope_cos_sin(torch.arange(T), hd, theta)
    assert torch.allclose(cos, t("cos"), atol=1e-6) and torch.allclose(sin, t("sin"), atol=1e-6)
    q = (x @ t("Wq").t()).view(T, nh, hd)
    q_rot = A.apply_rope(q, cos[:, None, :], sin[:, None, :]).transpose(0, 1)
    assert torch.allclose(q_rot, t("q_rot"), atol=1e-5, rtol=1e-5)
    # token by token against a cache == the causal pass over the whole sequence
    attn = A.AttentionOracle(t("Wq"), t("Wk"), t("Wv"), t("Wo"), nh, nkv, hd, max_len=T, theta=theta, round_to=None)
    for pos in range(T):
        o = attn.step(x[pos:pos + 1], pos)
        assert torch.allclose(o[0], t("attn_out")[pos], atol=2e-5, rtol=1e-4), pos
        h_mid = h[pos:pos + 1] + o
        assert torch.allclose(h_mid[0], t("h_mid")[pos], atol=2e-5, rtol=1e-4)
        assert torch.allclose(A.rms_norm(h_mid, t("ln_post"), eps)[0], t("x_post")[pos], atol=5e-5, rtol=1e-4)
    assert torch.allclose(attn.kc[:, :T], t("k_rot"), atol=1e-5, rtol=1e-5)
