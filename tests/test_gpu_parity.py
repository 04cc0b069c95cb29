"""Parity of the CUDA path (through the C ABI) against the CPU oracle and the golden fixtures."""
import ctypes as C
import json
import os
import random

import numpy as np
import pytest
import torch

from mixtral_offloading_b200 import (ExpertCache, HQQLinearTritonSavable, MixtralBLockSparseTop2MLP_HQQ,
                                     MixtralExpertWrapper, SparseMoeWrapper, _cabi, packing)
from oracle import hqq_oracle as O
from tests.helpers import bf16_from_bits, fill_layer, layer_from_oracle, quant_config, random_layer, random_layer_fast

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = 1e-2          # max|y - y_ref| / max|y_ref| per layer, the bound the build targets


def gpu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


# ------------------------------------------------------------------ packing
PACKERS = {2: (packing.pack_2bit_u8_common, packing.unpack_2bit_u8_common),
           3: (packing.pack_3bit_i32_common, packing.unpack_3bit_i32_common),
           4: (packing.pack_4bit_u8_common, packing.unpack_4bit_u8_common)}


@pytest.mark.parametrize("nbits,rows", [(4, 64), (2, 64), (3, 64), (3, 60), (3, 7)])
def test_packing_golden(golden_dir, nbits, rows):
    z = np.load(os.path.join(golden_dir, "packing.npz"))
    pack, unpack = PACKERS[nbits]
    packed = pack(gpu(z[f"codes_{nbits}_{rows}"]))
    assert np.array_equal(packed.cpu().numpy(), z[f"packed_{nbits}_{rows}"])
    assert np.array_equal(unpack(gpu(z[f"packed_{nbits}_{rows}"])).cpu().numpy(), z[f"unpacked_{nbits}_{rows}"])


@pytest.mark.parametrize("nbits,N,K", [(4, 256, 512), (4, 6, 33), (2, 256, 512), (2, 8, 17), (3, 250, 512),
                                       (3, 13, 7), (3, 1, 1), (3, 10, 4), (3, 39, 20), (4, 2, 16), (2, 4, 15)])
def test_packing_oracle_ragged(nbits, N, K):
    rng = np.random.default_rng(N * 1000 + K)
    codes = rng.integers(0, 2 ** nbits, (N, K), dtype=np.uint8)
    pack, unpack = PACKERS[nbits]
    want = O.PACK[nbits](codes)
    got = pack(gpu(codes))
    assert got.dtype == (torch.int32 if nbits == 3 else torch.uint8)
    assert np.array_equal(got.cpu().numpy(), want)
    back = unpack(got)
    assert np.array_equal(back.cpu().numpy(), O.UNPACK[nbits](want))
    assert np.array_equal(back.cpu().numpy()[:N], codes)


def test_packing_empty():
    for nbits, (pack, unpack) in PACKERS.items():
        e = torch.empty((0, 16), dtype=torch.uint8, device=DEV)
        assert pack(e).shape[0] == 0
        p = torch.empty((0, 16), dtype=torch.int32 if nbits == 3 else torch.uint8, device=DEV)
        assert unpack(p).shape[0] == 0


@pytest.mark.parametrize("nbits,N,K", [(4, 4096, 4096), (2, 14336, 4096), (2, 4096, 14336), (3, 14336, 4096)])
def test_packing_full_size_round_trip(nbits, N, K):
    g = torch.Generator(device=DEV).manual_seed(nbits)
    codes = torch.randint(0, 2 ** nbits, (N, K), dtype=torch.uint8, device=DEV, generator=g)
    pack, unpack = PACKERS[nbits]
    packed = pack(codes)
    back = unpack(packed)
    assert torch.equal(back[:N], codes)
    if nbits == 3:
        assert packed.shape == ((N + 9) // 10, K) and int(back[N:].max()) == 0     # zero tail (packing.py:66-77)
        assert int((packed >> 30).abs().max()) == 0                                 # bits 31-30 unused
    # spot-check storage rows against the oracle
    per = O.CODES_PER_WORD[nbits]
    rows = [0, 1, packed.shape[0] // 2, packed.shape[0] - 1]
    for R in rows:
        want = O.PACK[nbits](codes[R * per:(R + 1) * per].cpu().numpy())
        assert np.array_equal(packed[R:R + 1].cpu().numpy(), want[:1])


# ------------------------------------------------------------------ quantized linear
def golden_layer(golden_dir, nbits):
    z = np.load(os.path.join(golden_dir, f"layer_{nbits}bit.npz"))
    od = dict(N=int(z["N"]), K=int(z["K"]), nbits=nbits, group_size=int(z["group_size"]), meta_group=256,
              **{k: z[k] for k in ("W_q", "scale_q", "zero_q", "ms_scale", "mz_scale", "ms_zero", "mz_zero")})
    return z, od


@pytest.mark.parametrize("nbits", [2, 3, 4])
def test_quantize_matches_reference_tensors(golden_dir, nbits):
    """The product's build-time quantiser reproduces the reference layer's tensors bit for bit."""
    z, od = golden_layer(golden_dir, nbits)
    W = bf16_from_bits(z["W_bf16"]).reshape(od["N"], od["K"]).to(DEV)
    lin = torch.nn.Linear(od["K"], od["N"], bias=False, device=DEV)
    lin.weight.data = W.float()
    layer = HQQLinearTritonSavable(lin, quant_config(nbits, od["group_size"]))
    assert np.array_equal(layer.W_q.cpu().numpy(), z["W_q"])
    m = layer.meta
    assert np.array_equal(m["scale_q"].cpu().numpy().reshape(-1), z["scale_q"])
    assert np.array_equal(m["zero_q"].cpu().numpy().reshape(-1), z["zero_q"])
    for a, b in ((m["meta_scale"]["scale"], "ms_scale"), (m["meta_scale"]["zero"], "mz_scale"),
                 (m["meta_zero"]["scale"], "ms_zero"), (m["meta_zero"]["zero"], "mz_zero")):
        assert np.array_equal(a.cpu().numpy().reshape(-1), z[b])
    # repack() from the (group_size, G*K)-packed form the reference's quantize() leaves behind
    per = O.CODES_PER_WORD[nbits]
    g = od["group_size"]
    codes = O.UNPACK[nbits](z["W_q"])[:od["N"]]
    layer.W_q = gpu(O.PACK[nbits](codes.reshape(g, -1)))
    layer.repack()
    assert tuple(layer.W_q.shape) == ((od["N"] + per - 1) // per, od["K"])
    assert np.array_equal(layer.W_q.cpu().numpy(), z["W_q"])


@pytest.mark.parametrize("nbits", [2, 3, 4])
def test_linear_golden(golden_dir, nbits):
    z, od = golden_layer(golden_dir, nbits)
    layer = layer_from_oracle(od, DEV)
    # decode: exact against the fp32 oracle, close to the reference's fp16 dequantize()
    W32 = layer.dequantize(torch.float32).cpu()
    assert torch.equal(W32, O.dequantize(od))
    assert O.rel_err(layer.dequantize(torch.float16).cpu(), torch.from_numpy(z["W_est_f16"])) < 3e-3
    x = bf16_from_bits(z["x_bf16"]).reshape(-1, od["K"])
    y = layer(x.to(DEV)).cpu()
    assert y.dtype == torch.bfloat16 and y.shape == (x.shape[0], od["N"])
    assert O.rel_err(y, torch.from_numpy(z["y_f32"])) < TOL
    assert O.rel_err(y, O.linear(x, od)) < TOL


SHAPES = [
    # nbits, group, N, K
    (4, 64, 128, 256), (4, 64, 512, 1024), (4, 64, 1024, 4096), (4, 32, 64, 128),
    (2, 16, 128, 256), (2, 16, 512, 1024), (2, 16, 1792, 512), (2, 32, 256, 4096), (2, 16, 512, 3584),
    (3, 64, 192, 256), (3, 64, 448, 512), (3, 64, 640, 1024), (3, 32, 160, 256), (3, 64, 1792, 512),
]


@pytest.mark.parametrize("nbits,group,N,K", SHAPES)
@pytest.mark.parametrize("M", [1, 2, 3, 7, 16, 17, 65])
def test_linear_oracle_small(nbits, group, N, K, M):
    od = random_layer(N, K, nbits, group, seed=N + K + nbits)
    layer = layer_from_oracle(od, DEV)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    y = layer(x.to(DEV)).cpu()
    assert O.rel_err(y, O.linear(x, od)) < TOL


def test_tensor_core_path_reports_no_timeout():
    """The tcgen05 GEMM bounds every wait; a wait that ran out would set this flag (and skip work)."""
    od = random_layer(512, 1024, 4, 64, seed=9)
    layer = layer_from_oracle(od, DEV)
    for M in (17, 64, 100, 300):
        x = torch.randn(M, 1024, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16)
        assert O.rel_err(layer(x.to(DEV)).cpu(), O.linear(x, od)) < TOL
    assert _cabi.lib().hqm_device_error() == 0


def test_linear_shapes_and_dtypes():
    od = random_layer(128, 256, 4, 64, seed=5)
    layer = layer_from_oracle(od, DEV)
    x = torch.randn(2, 3, 256).to(torch.bfloat16)
    y = layer(x.to(DEV))
    assert y.shape == (2, 3, 128)
    assert O.rel_err(y.cpu().reshape(6, 128), O.linear(x.reshape(6, 256), od)) < TOL
    y16 = layer(x.to(DEV).half())
    assert y16.dtype == torch.float16
    assert layer(torch.empty(0, 256, dtype=torch.bfloat16, device=DEV)).shape == (0, 128)
    with pytest.raises(RuntimeError):
        layer(x)                                  # CPU tensor: no fallback path
    with pytest.raises(AssertionError):
        layer(torch.zeros(1, 255, dtype=torch.bfloat16, device=DEV))
    # bias
    layer.bias = torch.randn(128).to(torch.bfloat16).to(DEV)
    yb = layer(x.to(DEV)).cpu().float()
    want = O.linear(x.reshape(6, 256), od) + layer.bias.cpu().float()
    assert O.rel_err(yb.reshape(6, 128), want) < TOL


FULL = [(4, 64, 4096, 4096, (1, 16, 64)), (4, 64, 1024, 4096, (1,)), (2, 16, 14336, 4096, (1, 8, 64, 512)),
        (2, 16, 4096, 14336, (1, 8, 64, 512)), (3, 64, 14336, 4096, (1, 4, 16, 128, 300))]


@pytest.mark.parametrize("nbits,group,N,K,Ms", FULL)
def test_linear_full_size(nbits, group, N, K, Ms):
    """BASELINE shapes: quantised from N(0, 0.02^2) weights as the configs say."""
    od = random_layer(N, K, nbits, group, seed=0)
    layer = layer_from_oracle(od, DEV)
    W = O.dequantize(od)
    assert torch.equal(layer.dequantize(torch.float32).cpu(), W)
    for M in Ms:
        g = torch.Generator().manual_seed(M)
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        y = layer(x.to(DEV)).cpu()
        assert O.rel_err(y, x.float() @ W.T) < TOL


def test_linear_is_linear_full_size():
    """Size-independent property at a BASELINE shape: y(a) + y(b) == y(a + b) up to bf16 rounding."""
    od = random_layer_fast(14336, 4096, 2, 16, seed=3)
    layer = layer_from_oracle(od, DEV)
    g = torch.Generator().manual_seed(0)
    a = torch.randn(1, 4096, generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randn(1, 4096, generator=g).to(torch.bfloat16).to(DEV)
    s = (a.float() + b.float()).to(torch.bfloat16)
    ya, yb, ys = layer(a).float(), layer(b).float(), layer(s).float()
    assert float((ya + yb - ys).abs().max() / ys.abs().max()) < 2e-2


# ------------------------------------------------------------------ expert FFN and MoE block
class Cfg:
    def __init__(self, hidden, ffn, n_exp):
        self.hidden_size, self.intermediate_size, self.num_local_experts = hidden, ffn, n_exp
        self.num_experts_per_tok, self.hidden_act = 2, "silu"


def make_expert(hidden, ffn, ods, nbits=2, group=16):
    cfg = quant_config(nbits, group)
    meta1 = HQQLinearTritonSavable.get_hqq_meta((hidden, ffn), cfg)
    meta2 = HQQLinearTritonSavable.get_hqq_meta((ffn, hidden), cfg)
    ex = MixtralBLockSparseTop2MLP_HQQ(Cfg(hidden, ffn, 8), cfg, meta1, meta2)
    if ods is not None:
        for name, od in zip(("w1", "w2", "w3"), ods):
            fill_layer(getattr(ex, name), od, DEV)
    return ex


def golden_experts(golden_dir):
    z = np.load(os.path.join(golden_dir, "expert_moe.npz"))
    hidden, ffn = int(z["hidden"]), int(z["ffn"])
    keys = ("W_q", "scale_q", "zero_q", "ms_scale", "mz_scale", "ms_zero", "mz_zero")
    experts = []
    for e in range(int(z["n_exp"])):
        ws = []
        for name, (N, K) in (("w1", (ffn, hidden)), ("w2", (hidden, ffn)), ("w3", (ffn, hidden))):
            ws.append(dict(N=N, K=K, nbits=2, group_size=16, meta_group=256, **{k: z[f"e{e}_{name}_{k}"] for k in keys}))
        experts.append(tuple(ws))
    return z, hidden, ffn, experts


def test_expert_ffn_golden(golden_dir):
    z, hidden, ffn, experts = golden_experts(golden_dir)
    x = bf16_from_bits(z["x_bf16"]).reshape(-1, hidden)
    ex = make_expert(hidden, ffn, experts[0])
    y = ex(x.to(DEV)).cpu()
    assert O.rel_err(y, torch.from_numpy(z["ffn0_y_f16"])) < TOL
    assert O.rel_err(y, O.expert_ffn(x, *experts[0])) < TOL


@pytest.mark.parametrize("M", [1, 8, 64, 200])
def test_expert_ffn_mid_size(M):
    hidden, ffn = 1024, 3584
    ods = (random_layer(ffn, hidden, 2, 16, 1), random_layer(hidden, ffn, 2, 16, 2), random_layer(ffn, hidden, 2, 16, 3))
    ex = make_expert(hidden, ffn, ods)
    x = torch.randn(M, hidden, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16)
    y = ex(x.to(DEV)).cpu()
    assert O.rel_err(y, O.expert_ffn(x, *ods)) < TOL


@pytest.mark.parametrize("M", [1, 8, 64, 512])
def test_expert_ffn_full_size(M):
    """BASELINE configs[1]: one Mixtral expert (w1, w3 14336 x 4096; w2 4096 x 14336), 2-bit g16, at its own token
    counts; 512 rows cross the 256-row chunking of the tensor-core GEMM and its scatter epilogue."""
    hidden, ffn = 4096, 14336
    ods = (random_layer(ffn, hidden, 2, 16, 1), random_layer(hidden, ffn, 2, 16, 2), random_layer(ffn, hidden, 2, 16, 3))
    ex = make_expert(hidden, ffn, ods)
    x = torch.randn(M, hidden, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16)
    y = ex(x.to(DEV)).cpu()
    assert O.rel_err(y, O.expert_ffn(x, *ods)) < TOL
    assert _cabi.lib().hqm_device_error() == 0


def test_overlapped_launches_give_the_same_bits():
    """A chain of expert FFNs feeding each other, launched back to back with no host work in between: each
    kernel may start while its predecessor is still running.  The result must be bit-identical to plain
    launches, eagerly and replayed from a CUDA graph."""
    hidden, ffn = 1024, 3584
    experts = []
    for e in range(3):
        ods = (random_layer(ffn, hidden, 2, 16, 10 * e + 1), random_layer(hidden, ffn, 2, 16, 10 * e + 2),
               random_layer(ffn, hidden, 2, 16, 10 * e + 3))
        experts.append(make_expert(hidden, ffn, ods))
    x = torch.randn(1, hidden, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(DEV)

    def chain(inp):
        h = inp
        for rep in range(4):
            for ex in experts:
                h = ex(h)
                h = (h.float() / h.float().abs().max().clamp_min(1e-6)).to(torch.bfloat16)   # keep the scale
        return h

    prev = _cabi.lib().hqm_set_overlap(0)
    try:
        plain = chain(x).clone()
        assert _cabi.lib().hqm_set_overlap(1) == 0
        for _ in range(3):
            assert torch.equal(chain(x), plain)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            chain(x)                                   # allocations settle before capture
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = chain(x)
        for _ in range(3):
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, plain)
    finally:
        _cabi.lib().hqm_set_overlap(prev)


def test_expert_ffn_routed_accumulates():
    hidden, ffn, T = 256, 512, 9
    ods = (random_layer(ffn, hidden, 2, 16, 1), random_layer(hidden, ffn, 2, 16, 2), random_layer(ffn, hidden, 2, 16, 3))
    ex = make_expert(hidden, ffn, ods)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, hidden, generator=g).to(torch.bfloat16)
    idx = torch.tensor([7, 2, 5], dtype=torch.int32)
    w = torch.tensor([0.25, 0.5, 0.75])
    base = torch.randn(T, hidden, generator=g).to(torch.bfloat16)
    out = base.clone().to(DEV)
    ex.forward_routed(x.to(DEV), idx.to(DEV), w.to(DEV), out, accumulate=True)
    want = base.float().clone()
    want[idx.long()] += O.expert_ffn(x[idx.long()], *ods) * w[:, None]
    assert O.rel_err(out.cpu(), want) < TOL
    untouched = [t for t in range(T) if t not in idx.tolist()]
    assert torch.equal(out.cpu()[untouched], base[untouched])


def test_router_against_oracle():
    M, K, E = 300, 512, 8
    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    gate = torch.nn.Linear(K, E, bias=False, dtype=torch.bfloat16, device=DEV)
    gate.weight.data = (torch.randn(E, K, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    moe = SparseMoeWrapper(Cfg(K, 2 * K, E), 0, gate, None)
    logits, topk_w, topk_idx, meta, token_idx, token_w = [t.cpu() for t in moe.route(x.to(DEV))]
    ref_logits, ref_w, ref_idx = O.router_top2(x, gate.weight.data.cpu(), round_to=torch.bfloat16)
    assert O.rel_err(logits, ref_logits) < 1e-2
    same = (topk_idx.long() == ref_idx).all(dim=1)
    assert same.float().mean() > 0.98                    # bf16 ties on the rounded logits may legitimately differ
    assert torch.allclose(topk_w[same], ref_w[same].to(torch.bfloat16).float(), atol=1e-2)
    assert torch.allclose(topk_w.sum(1), torch.ones(M), atol=1e-2)
    counts, offsets = meta[:E].tolist(), meta[E:].tolist()
    assert sum(counts) == 2 * M and offsets[0] == 0 and offsets[-1] == 2 * M
    for e in range(E):
        seg = token_idx[offsets[e]:offsets[e + 1]].tolist()
        want = sorted(t for t in range(M) if e in topk_idx[t].tolist())
        assert seg == want and counts[e] == len(want)
        for pos, t in zip(range(offsets[e], offsets[e + 1]), seg):
            slot = topk_idx[t].tolist().index(e)
            assert float(token_w[pos]) == float(topk_w[t, slot])


def build_cache(experts_ods, hidden, ffn, main_size, offload_size, buffer_size, layer_id=0, offload_first=None):
    def make_module():
        ods = (random_layer(ffn, hidden, 2, 16, 91), random_layer(hidden, ffn, 2, 16, 92), random_layer(ffn, hidden, 2, 16, 93))
        return MixtralExpertWrapper(make_expert(hidden, ffn, ods), device=DEV)
    cache = ExpertCache(make_module, main_size=main_size, offload_size=offload_size, buffer_size=buffer_size)
    n_off = offload_size if offload_first is None else offload_first
    for e, ods in enumerate(experts_ods):
        wrapped = MixtralExpertWrapper(make_expert(hidden, ffn, ods), device=DEV)
        cache.add_expert((layer_id, e), wrapped, eviction_group=layer_id, offload=(e < n_off))
    return cache


def test_moe_block_golden(golden_dir):
    z, hidden, ffn, experts = golden_experts(golden_dir)
    x = bf16_from_bits(z["x_bf16"]).reshape(-1, hidden)
    gate_w = bf16_from_bits(z["gate_bf16"]).reshape(-1, hidden)
    cache = build_cache(experts, hidden, ffn, main_size=2, offload_size=2, buffer_size=2)
    gate = torch.nn.Linear(hidden, len(experts), bias=False, dtype=torch.bfloat16, device=DEV)
    gate.weight.data = gate_w.to(DEV)
    moe = SparseMoeWrapper(Cfg(hidden, ffn, len(experts)), 0, gate, cache)
    for _ in range(3):                                  # repeated calls exercise swaps in both directions
        y, logits = moe(x.to(DEV).reshape(1, -1, hidden))
        assert y.shape == (1, x.shape[0], hidden) and logits.shape == (x.shape[0], len(experts))
        want, want_logits = O.moe_forward(x, gate_w, experts)
        assert O.rel_err(logits.cpu(), want_logits) < TOL
        assert O.rel_err(y.cpu().reshape(-1, hidden), want) < TOL
        assert O.rel_err(y.cpu().reshape(-1, hidden), torch.from_numpy(z["moe_y_f16"])) < 2e-2
    gi = cache.group_infos[0]
    assert gi.hits + gi.misses == 3 * len(set(O.router_top2(x, gate_w, round_to=torch.bfloat16)[2].flatten().tolist()))
    assert gi.misses > 0


def test_resident_moe_device_side_routing():
    """All experts resident: the single-token block never tells the host which experts ran, and can be
    replayed from a CUDA graph; several tokens fall back to the per-expert loop.  Both match the oracle."""
    from mixtral_offloading_b200 import ResidentMoe
    hidden, ffn, n_exp = 256, 512, 8
    experts = [tuple(random_layer(n, k, 2, 16, seed=20 * e + i) for i, (n, k) in
                     enumerate(((ffn, hidden), (hidden, ffn), (ffn, hidden)))) for e in range(n_exp)]
    g = torch.Generator().manual_seed(11)
    gate_w = (torch.randn(n_exp, hidden, generator=g) * 0.05).to(torch.bfloat16)
    gate = torch.nn.Linear(hidden, n_exp, bias=False, dtype=torch.bfloat16, device=DEV)
    gate.weight.data = gate_w.to(DEV)
    moe = ResidentMoe(Cfg(hidden, ffn, n_exp), 0, gate, [make_expert(hidden, ffn, ods) for ods in experts])
    router = SparseMoeWrapper(Cfg(hidden, ffn, n_exp), 0, gate, None)
    xs = torch.randn(6, hidden, generator=g).to(torch.bfloat16)
    seen = set()
    for t in range(6):
        x = xs[t:t + 1]
        y, logits = moe(x.to(DEV).reshape(1, 1, hidden))
        _, tw, ti, _, _, _ = router.route(x.to(DEV))
        seen.update(ti.cpu().flatten().tolist())
        want, want_logits = O.moe_forward(x, gate_w, experts, routing=(tw.cpu(), ti.cpu()))
        assert O.rel_err(y.cpu().reshape(1, hidden), want) < TOL
        assert O.rel_err(logits.cpu(), want_logits) < TOL
    assert len(seen) > 2                                  # different tokens really picked different experts
    y, _ = moe(xs.to(DEV).reshape(1, 6, hidden))          # several tokens: host-driven loop
    _, tw, ti, _, _, _ = router.route(xs.to(DEV))
    want, _ = O.moe_forward(xs, gate_w, experts, routing=(tw.cpu(), ti.cpu()))
    assert O.rel_err(y.cpu().reshape(6, hidden), want) < TOL
    # graph replay with a new input: the routing changes inside the graph
    x_static = xs[0:1].to(DEV).reshape(1, 1, hidden).clone()
    moe(x_static)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static, _ = moe(x_static)
    for t in (3, 5):
        x_static.copy_(xs[t:t + 1].to(DEV).reshape(1, 1, hidden))
        graph.replay()
        _, tw, ti, _, _, _ = router.route(xs[t:t + 1].to(DEV))
        want, _ = O.moe_forward(xs[t:t + 1], gate_w, experts, routing=(tw.cpu(), ti.cpu()))
        assert O.rel_err(y_static.cpu().reshape(1, hidden), want) < TOL


def test_expert_cache_moves_the_right_bytes(golden_dir):
    """Replay the reference's recorded requests on real slabs: every yielded module must hold
    its expert's bytes, and residency / hits / misses must follow the reference."""
    hidden, ffn = 128, 256
    traces = json.load(open(os.path.join(golden_dir, "lru_traces.json")))
    tr = traces[0]

    class Raw:
        def __init__(self, fill):
            self.storage = torch.UntypedStorage(4096, device=DEV)
            torch.as_tensor(self.storage, dtype=torch.uint8, device=DEV).fill_(fill)
    cache = ExpertCache(lambda: Raw(255), tr["main_size"], tr["offload_size"], tr["buffer_size"])
    for uid, group, offload in tr["placement"]:
        cache.add_expert_storage(tuple(uid), Raw(uid[1] + 1).storage, eviction_group=group, offload=offload)
    for step in tr["steps"]:
        order = []
        for uid, module in cache.load_experts(*[tuple(u) for u in step["request"]], unordered=step["unordered"]):
            data = torch.as_tensor(module.storage, dtype=torch.uint8, device=DEV)
            junk = torch.empty(1 << 22, device=DEV).normal_()        # keep the compute stream busy
            assert int(data.min()) == uid[1] + 1 and int(data.max()) == uid[1] + 1
            del junk
            order.append(list(uid))
        assert order == step["order"]
        gi = cache.group_infos[0]
        assert [list(u) for u in gi.resident] == step["resident"]
        assert (gi.hits, gi.misses) == (step["hits"], step["misses"])
    h2d, swaps = cache.stats()
    assert swaps == tr["steps"][-1]["misses"] and h2d == swaps * 4096
    # protocol errors surface as the reference's exception types
    with pytest.raises(AssertionError):
        list(cache.load_experts((0, 1), (0, 1)))
    with pytest.raises(AssertionError):
        cache.add_expert_storage((0, 1), Raw(0).storage)
    with pytest.raises(ValueError):
        cache.add_expert_storage((0, 99), Raw(0).storage)


def test_expert_cache_random_traffic_few_buffers():
    rng = random.Random(0)

    class Raw:
        def __init__(self, fill):
            self.storage = torch.UntypedStorage(1 << 16, device=DEV)
            torch.as_tensor(self.storage, dtype=torch.uint8, device=DEV).fill_(fill)
    cache = ExpertCache(lambda: Raw(255), 3, 5, 2)
    for e in range(8):
        cache.add_expert_storage(e, Raw(e + 1).storage, eviction_group=0, offload=(e >= 3))
    for _ in range(100):
        req = rng.sample(range(8), rng.choice([1, 2, 3, 5, 8]))
        got = []
        for uid, module in cache.load_experts(*req, unordered=rng.random() < 0.5):
            data = torch.as_tensor(module.storage, dtype=torch.uint8, device=DEV)
            assert int(data.min()) == uid + 1 and int(data.max()) == uid + 1
            got.append(uid)
        assert sorted(got) == sorted(req)


# ------------------------------------------------------------------ checkpoint format (state-dict hooks)
def test_scale_and_zero_with_different_meta_groups():
    """A checkpoint whose scale is 8-bit quantised in groups of 128 and whose zero is one group for the whole
    tensor (the reference's notebook overrides only the scale's group size, so the two differ in real files): the
    group sizes are read off the tensors, the layer is computed by the shape-agnostic kernel, fp32 decode exact."""
    N, K = 256, 512
    L = (N // 64) * K
    g = torch.Generator().manual_seed(2)
    W = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    od = O.quantize(W, 4, 64, meta_group=128, meta_group_zero=L)
    layer = layer_from_oracle(od, DEV)
    d = layer.descriptor()
    assert (d.meta_group, d.meta_group_zero) == (128, L)
    assert torch.equal(layer.dequantize(torch.float32).cpu(), O.dequantize(od))
    for M in (1, 5, 40):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        assert O.rel_err(layer(x.to(DEV)).cpu(), O.linear(x, od)) < TOL
    # the same tensors through the state-dict hooks into a layer built from the 256 / 256 template
    sd = {k: v.clone() for k, v in layer.state_dict().items()}
    fresh = layer_from_oracle(random_layer(N, K, 4, 64, seed=1), DEV)
    fresh.load_state_dict(sd)
    d2 = fresh.descriptor()
    assert (d2.meta_group, d2.meta_group_zero) == (128, L)
    x = torch.randn(3, K, generator=g).to(torch.bfloat16)
    assert torch.equal(fresh(x.to(DEV)), layer(x.to(DEV)))
    # tensors that do not fit the layer are refused, not read out of bounds
    bad = dict(sd)
    bad["meta.meta_scale.scale"] = sd["meta.meta_scale.scale"].reshape(-1)[:-1].clone()
    fresh.load_state_dict(bad)
    with pytest.raises(ValueError):
        fresh.descriptor()


def test_state_dict_round_trip_of_layer_and_expert_slab():
    """custom_layers.py:136-222 and expert_wrapper.py:23-30: a quantized layer and a whole expert slab saved and
    reloaded give identical bytes and identical outputs."""
    hidden, ffn = 256, 512
    ods = (random_layer(ffn, hidden, 2, 16, 1), random_layer(hidden, ffn, 2, 16, 2), random_layer(ffn, hidden, 2, 16, 3))
    src = MixtralExpertWrapper(make_expert(hidden, ffn, ods), device=DEV)
    sd = src.state_dict()
    assert set(sd) == {"storage"} and sd["storage"].dtype == torch.uint8
    other = (random_layer(ffn, hidden, 2, 16, 11), random_layer(hidden, ffn, 2, 16, 12), random_layer(ffn, hidden, 2, 16, 13))
    dst = MixtralExpertWrapper(make_expert(hidden, ffn, other), device=DEV)
    x = torch.randn(4, hidden, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).to(DEV)
    assert not torch.equal(dst(x), src(x))
    dst.load_state_dict({k: v.cpu() for k, v in sd.items()})            # as read from a file
    assert torch.equal(torch.as_tensor(dst.storage, dtype=torch.uint8, device=DEV).cpu(), sd["storage"].cpu())
    assert torch.equal(dst(x), src(x))
    assert O.rel_err(dst(x).cpu(), O.expert_ffn(x.cpu(), *ods)) < TOL
    # a single layer: W_q arriving in the (group_size, G*K)-packed form is repacked on load (custom_layers.py:222)
    od = ods[0]
    lay = layer_from_oracle(od, DEV)
    sd1 = {k: v.clone() for k, v in lay.state_dict().items()}
    codes = O.UNPACK[2](od["W_q"])[:od["N"]]
    sd1["W_q"] = gpu(O.PACK[2](codes.reshape(od["group_size"], -1)))
    fresh = layer_from_oracle(random_layer(ffn, hidden, 2, 16, 21), DEV)
    fresh.load_state_dict(sd1)
    assert np.array_equal(fresh.W_q.cpu().numpy(), od["W_q"])
    assert torch.equal(fresh(x), lay(x))


def test_many_row_gemm_without_tma_staging():
    """HQM_GEMM_TMA=0 at load time keeps the many-row GEMM on its first-generation kernel (operand tiles filled by
    the producer threads): same oracle, same bound; run in a process of its own because the switch is read once."""
    import subprocess
    import sys
    code = (
        "import torch\n"
        "from oracle import hqq_oracle as O\n"
        "from tests.helpers import layer_from_oracle, random_layer\n"
        "from mixtral_offloading_b200 import _cabi\n"
        "dev = torch.device('cuda:0')\n"
        "for nbits, group, N, K, M in ((2, 16, 1792, 1024, 40), (4, 64, 1024, 2048, 300)):\n"
        "    od = random_layer(N, K, nbits, group, seed=3)\n"
        "    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16)\n"
        "    y = layer_from_oracle(od, dev)(x.to(dev)).cpu()\n"
        "    err = O.rel_err(y, O.linear(x, od))\n"
        "    assert err < 1e-2, err\n"
        "assert _cabi.lib().hqm_device_error() == 0\n"
        "print('ok')\n")
    env = dict(os.environ, HQM_GEMM_TMA="0")
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600,
                         cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr
