"""Generate the golden fixtures in this directory from the reference's own code.

Run where a checkout of the reference is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's src/packing.py, src/custom_layers.py,
src/expert_cache.py and src/expert_wrapper.py on the CPU under ref_shim.py
(hqq is absent; see that file) and records, with fixed seeds:

  packing.npz     codes -> reference pack_*_common -> reference unpack_*_common
  layer_{2,3,4}bit.npz  a small quantized linear: every tensor the reference layer
                  holds after quantize()+repack(), its dequantize() (fp16) and
                  x @ dequantize().T
  expert_moe.npz  one MixtralBLockSparseTop2MLP_HQQ forward and one SparseMoeWrapper
                  forward over the real ExpertCache (fp16, CPU; forward routed to
                  F.linear(x, dequantize()) because forward_triton needs a GPU)
  slab_layout.json  order / offsets / sizes of the tensors inside an expert's
                  storage slab as MixtralExpertWrapper.replace_layer_storage lays them
  lru_traces.json traces of the real ExpertCache: yield order, residency, hits/misses
"""
from __future__ import annotations

import hashlib
import json
import os
import random
import sys

import numpy as np
import torch
from torch import nn
from torch.nn import functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: python make_golden.py <path of the dvmazur/mixtral-offloading checkout>")
REF = sys.argv[1]
sys.path.insert(0, HERE)
sys.path.insert(0, REF)

import ref_shim  # noqa: E402

ref_shim.install()
torch.UntypedStorage.pin_memory = lambda self, device=None: self      # no driver on the CPU box

from src import packing as rp  # noqa: E402
from src import custom_layers as rcl  # noqa: E402
from src import expert_cache as rec  # noqa: E402
from src import expert_wrapper as rew  # noqa: E402
from src.utils import nested_flatten  # noqa: E402
from transformers.models.mixtral.configuration_mixtral import MixtralConfig  # noqa: E402

# storage-replaced tensors lose the PackedTensor tag (the reference then falls into hqq's
# stock unpackers); the layout in memory is still the "common" one, so point them there.
ref_shim.BitPack.unpack_4bit_u8 = staticmethod(rp.unpack_4bit_u8_common)
ref_shim.BitPack.unpack_2bit_u8 = staticmethod(rp.unpack_2bit_u8_common)
ref_shim.BitPack.unpack_3bit_32 = staticmethod(rp.unpack_3bit_i32_common)
rcl.HQQLinearTritonSavable.forward = lambda self, x: F.linear(x, self.dequantize())


def bf16_bits(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def make_packing():
    g = torch.Generator().manual_seed(0)
    out = {}
    for nbits, rows, pack, unpack in ((4, 64, rp.pack_4bit_u8_common, rp.unpack_4bit_u8_common),
                                      (2, 64, rp.pack_2bit_u8_common, rp.unpack_2bit_u8_common),
                                      (3, 64, rp.pack_3bit_i32_common, rp.unpack_3bit_i32_common),
                                      (3, 60, rp.pack_3bit_i32_common, rp.unpack_3bit_i32_common),
                                      (3, 7, rp.pack_3bit_i32_common, rp.unpack_3bit_i32_common)):
        codes = torch.randint(0, 2 ** nbits, (rows, 48), generator=g, dtype=torch.uint8)
        packed = pack(codes)
        back = unpack(torch.as_tensor(packed))
        assert torch.equal(back[:rows], codes)
        out[f"codes_{nbits}_{rows}"] = codes.numpy()
        out[f"packed_{nbits}_{rows}"] = torch.as_tensor(packed).numpy()
        out[f"unpacked_{nbits}_{rows}"] = back.numpy()
    # known answers for the 3-bit word layout
    sevens = rp.pack_3bit_i32_common(torch.full((10, 1), 7, dtype=torch.uint8))
    first = torch.zeros((10, 1), dtype=torch.uint8)
    first[0] = 7
    out["ka_3bit_ten_sevens"] = torch.as_tensor(sevens).numpy()
    out["ka_3bit_first_seven"] = torch.as_tensor(rp.pack_3bit_i32_common(first)).numpy()
    np.savez_compressed(os.path.join(HERE, "packing.npz"), **out)


def layer_tensors(layer):
    m = layer.meta
    return dict(
        W_q=torch.as_tensor(layer.W_q).numpy(),
        scale_q=m["scale_q"].reshape(-1).numpy(), zero_q=m["zero_q"].reshape(-1).numpy(),
        ms_scale=m["meta_scale"]["scale"].reshape(-1).numpy(), mz_scale=m["meta_scale"]["zero"].reshape(-1).numpy(),
        ms_zero=m["meta_zero"]["scale"].reshape(-1).numpy(), mz_zero=m["meta_zero"]["zero"].reshape(-1).numpy(),
    )


def make_layer(nbits, group, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(5, K, generator=g).to(torch.bfloat16)
    lin = nn.Linear(K, N, bias=False)
    lin.weight.data = W.float()
    cfg = ref_shim.BaseQuantizeConfig(nbits=nbits, group_size=group, quant_zero=True, quant_scale=True)
    layer = rcl.HQQLinearTritonSavable(lin, cfg)
    assert tuple(layer.meta["shape"]) == (N, K) and layer.meta["axis"] == 0
    W_est = layer.dequantize()                                            # fp16, custom_layers.py:95-116
    y = x.float() @ W_est.float().T
    out = layer_tensors(layer)
    out.update(N=N, K=K, nbits=nbits, group_size=group, meta_group=256,
               W_bf16=bf16_bits(W), x_bf16=bf16_bits(x), W_est_f16=W_est.numpy(), y_f32=y.numpy())
    np.savez_compressed(os.path.join(HERE, f"layer_{nbits}bit.npz"), **out)


def fill_expert(expert, seed):
    """Quantise random weights into an empty reference expert (what load_state_dict does in build_model)."""
    g = torch.Generator().manual_seed(seed)
    for name in ("w1", "w2", "w3"):
        lyr = getattr(expert, name)
        N, K = lyr.meta["shape"]
        lin = nn.Linear(K, N, bias=False)
        lin.weight.data = torch.randn(N, K, generator=g) * 0.02
        lyr.bias = None
        lyr.quantize(lin.weight.data, **lyr.quant_config)
    return expert


def make_expert_moe():
    hidden, ffn, n_exp, tokens = 128, 256, 4, 12
    config = MixtralConfig(hidden_size=hidden, intermediate_size=ffn, num_local_experts=n_exp,
                           num_experts_per_tok=2, num_hidden_layers=1, num_attention_heads=4,
                           num_key_value_heads=2, vocab_size=64)
    qcfg = ref_shim.BaseQuantizeConfig(nbits=2, group_size=16, quant_zero=True, quant_scale=True)
    meta1 = rcl.HQQLinearTritonSavable.get_hqq_meta((hidden, ffn), qcfg)
    meta2 = rcl.HQQLinearTritonSavable.get_hqq_meta((ffn, hidden), qcfg)

    def empty():
        return rcl.MixtralBLockSparseTop2MLP_HQQ(config, qcfg, meta1, meta2)

    out = dict(hidden=hidden, ffn=ffn, n_exp=n_exp, tokens=tokens)
    experts = [fill_expert(empty(), 100 + e) for e in range(n_exp)]
    for e, ex in enumerate(experts):
        for name in ("w1", "w2", "w3"):
            for k, v in layer_tensors(getattr(ex, name)).items():
                out[f"e{e}_{name}_{k}"] = v

    g = torch.Generator().manual_seed(7)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    gate_w = (torch.randn(n_exp, hidden, generator=g) * 0.02).to(torch.bfloat16)
    out["x_bf16"], out["gate_bf16"] = bf16_bits(x), bf16_bits(gate_w)
    with torch.inference_mode():
        out["ffn0_y_f16"] = experts[0](x.half()).numpy()                  # custom_layers.py:253-256

    # slab layout as replace_layer_storage produces it (expert_wrapper.py:41-85)
    names, offsets, off = [], [], 0
    state = {f"w{i}": {"W_q": getattr(experts[0], f"w{i}").W_q, "meta": getattr(experts[0], f"w{i}").meta,
                       "bias": getattr(experts[0], f"w{i}").bias} for i in range(1, 4)}

    def walk(d, prefix):
        for k, v in sorted(d.items()):
            if isinstance(v, dict):
                yield from walk(v, prefix + k + ".")
            else:
                yield prefix + k, v
    flat_named = [(n, v) for n, v in walk(state, "") if isinstance(v, torch.Tensor)]
    flat = [v for v in nested_flatten(state) if isinstance(v, torch.Tensor)]
    assert all(a is b for (_, a), b in zip(flat_named, flat))
    for n, v in flat_named:
        names.append(n)
        offsets.append(off)
        off += v.nbytes

    # the MoE block over the real cache: 2 device slots, 2 host slots, 2 buffers
    def make_module():
        return rew.MixtralExpertWrapper(fill_expert(empty(), 0), device=torch.device("cpu"))
    cache = rec.ExpertCache(make_module, main_size=2, offload_size=2, buffer_size=2)
    wrapped0 = None
    for e, ex in enumerate(experts):
        w = rew.MixtralExpertWrapper(ex, device=torch.device("cpu"))
        if e == 0:
            wrapped0 = w
        cache.add_expert((0, e), w, eviction_group=0, offload=(e < 2))
    slab = bytes(wrapped0.storage)
    assert len(slab) == off
    with open(os.path.join(HERE, "slab_layout.json"), "w") as f:
        json.dump(dict(names=names, offsets=offsets, total=off, sha256_expert0=hashlib.sha256(slab).hexdigest()), f,
                  indent=1)

    gate = nn.Linear(hidden, n_exp, bias=False, dtype=torch.float16)
    gate.weight.data = gate_w.half()
    moe = rcl.SparseMoeWrapper(config, 0, gate, cache)
    with torch.inference_mode():
        y, logits = moe(x.half().reshape(1, tokens, hidden))              # custom_layers.py:272-314
    out["moe_y_f16"], out["moe_logits_f16"] = y.reshape(tokens, hidden).numpy(), logits.numpy()
    np.savez_compressed(os.path.join(HERE, "expert_moe.npz"), **out)


class _Slab:
    def __init__(self, size=16):
        self.storage = torch.UntypedStorage(size)


def run_trace(main_size, offload_size, buffer_size, placement, requests):
    """placement: list of (uid, group, offload); requests: list of (uids, unordered)."""
    cache = rec.ExpertCache(lambda: _Slab(), main_size, offload_size, buffer_size)
    for uid, group, offload in placement:
        s = _Slab()
        torch.as_tensor(s.storage, dtype=torch.uint8)[:] = hash(tuple(uid)) % 251
        cache.add_expert_storage(tuple(uid), s.storage, eviction_group=group, offload=offload)
    steps = []
    for uids, unordered in requests:
        order, intact = [], []
        for uid, module in cache.load_experts(*[tuple(u) for u in uids], unordered=unordered):
            # with few buffers the reference can hand out a slab that a later swap already overwrote
            intact.append(int(torch.as_tensor(module.storage, dtype=torch.uint8)[0]) == hash(tuple(uid)) % 251)
            order.append(list(uid))
        group = cache.registered_experts[tuple(uids[0])].eviction_group
        gi = cache.group_infos[group]
        steps.append(dict(request=[list(u) for u in uids], unordered=unordered, order=order, intact=intact,
                          resident=[list(u) for u in gi.main_infos.keys()], hits=gi.hits, misses=gi.misses))
    return dict(main_size=main_size, offload_size=offload_size, buffer_size=buffer_size,
                placement=[[list(u), g, o] for u, g, o in placement], steps=steps)


def make_lru():
    traces = []
    # one layer, experts 0-3 offloaded and 4-7 resident as build_model.py:220 does, 4 buffers
    place = [((0, e), 0, e < 4) for e in range(8)]
    reqs = [([(0, 4), (0, 5)], True), ([(0, 0), (0, 5)], True), ([(0, 1), (0, 2)], True), ([(0, 0), (0, 1)], True),
            ([(0, 6), (0, 7)], True), ([(0, e) for e in range(8)], True), ([(0, 3), (0, 4)], True)]
    traces.append(run_trace(4, 4, 4, place, reqs))
    # ordered requests and a single buffer pair
    traces.append(run_trace(4, 4, 2, place, [([(0, 0), (0, 5), (0, 1)], False), ([(0, 7), (0, 2)], False),
                                             ([(0, e) for e in range(7, -1, -1)], False)]))
    # several layers sharing the pools, random top-2 style traffic
    rng = random.Random(0)
    layers, n_exp, per_layer_off = 3, 8, 5
    place = [((l, e), l, e < per_layer_off) for l in range(layers) for e in range(n_exp)]
    reqs = []
    for _ in range(60):
        l = rng.randrange(layers)
        k = rng.choice([1, 2, 2, 2, 3, 5, 8])
        reqs.append(([(l, e) for e in rng.sample(range(n_exp), k)], rng.random() < 0.8))
    traces.append(run_trace(layers * (n_exp - per_layer_off), layers * per_layer_off, 4, place, reqs))
    with open(os.path.join(HERE, "lru_traces.json"), "w") as f:
        json.dump(traces, f)


if __name__ == "__main__":
    make_packing()
    make_layer(4, 64, 128, 256, seed=1)
    make_layer(2, 16, 128, 256, seed=2)
    make_layer(3, 64, 192, 256, seed=3)
    make_expert_moe()
    make_lru()
    print("golden fixtures written to", HERE)
