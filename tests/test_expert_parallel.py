"""Expert-parallel MoE block: partition and combine logic on CPU ranks (gloo, world size 2), and the
real thing on 2 GPUs when they are there."""
import ctypes as C
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mixtral_offloading_b200.expert_parallel import ExpertParallelMoe, expert_owner, owner_layout
from oracle import hqq_oracle as O
from tests.helpers import random_layer


class Cfg:
    def __init__(self, hidden, ffn, n_exp):
        self.hidden_size, self.intermediate_size, self.num_local_experts = hidden, ffn, n_exp
        self.num_experts_per_tok, self.hidden_act = 2, "silu"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _problem(hidden=128, ffn=256, n_exp=4, tokens=7):
    experts = [tuple(random_layer(n, k, 2, 16, seed=10 * e + i) for i, (n, k) in
                     enumerate(((ffn, hidden), (hidden, ffn), (ffn, hidden)))) for e in range(n_exp)]
    g = torch.Generator().manual_seed(3)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)
    gate_w = (torch.randn(n_exp, hidden, generator=g) * 0.02).to(torch.bfloat16)
    return hidden, ffn, n_exp, experts, x, gate_w


def test_owner_layout_and_partition():
    per, perm = owner_layout(7, 4)
    assert per == 2 and sorted(perm.tolist()) == sorted(set(perm.tolist())) and int(perm.max()) < 8
    for t in range(7):
        assert perm[t] // per == t % 4                      # grouped by owner
    assert [expert_owner(e, 8, 4) for e in range(8)] == [0, 0, 1, 1, 2, 2, 3, 3]
    with pytest.raises(AssertionError):
        expert_owner(0, 8, 3)


class OracleRankMoe(ExpertParallelMoe):
    """The same module with the device pieces replaced by the CPU oracle, so that the sharding and
    the collectives can run as gloo ranks."""

    def __init__(self, *a, experts=None, gate_w=None, **k):
        super().__init__(*a, **k)
        self._experts, self._gate_w = experts, gate_w

    def route(self, x2d):
        logits, w, idx = O.router_top2(x2d, self._gate_w, round_to=torch.bfloat16)
        w = w.to(torch.bfloat16).float()
        E = self.num_experts
        counts, offsets, tok, tw = [], [0], [], []
        for e in range(E):
            t, slot = torch.where(idx == e)
            order = torch.argsort(t)
            tok += t[order].tolist()
            tw += w[t[order], slot[order]].tolist()
            counts.append(len(t))
            offsets.append(offsets[-1] + len(t))
        return logits.to(torch.bfloat16), counts, offsets, torch.tensor(tok, dtype=torch.int32), torch.tensor(tw)

    def run_expert(self, e, x_rows, row_idx, row_w, out):
        rows = row_idx.long()
        y = O.expert_ffn(x_rows[rows], *self._experts[e]) * row_w[:, None].to(torch.bfloat16).float()
        out[rows] = (out[rows].float() + y.to(torch.bfloat16).float()).to(out.dtype)


def _cpu_rank(rank, world, port, combine, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hidden, ffn, n_exp, experts, x, gate_w = _problem()
        local = {e: None for e in range(n_exp) if expert_owner(e, n_exp, world) == rank}
        moe = OracleRankMoe(Cfg(hidden, ffn, n_exp), 0, None, local, combine=combine, experts=experts, gate_w=gate_w)
        y, logits = moe(x.reshape(1, -1, hidden))
        want, want_logits = O.moe_forward(x, gate_w, experts)
        err = O.rel_err(y.reshape(-1, hidden), want)
        assert err < 1e-2, err
        assert O.rel_err(logits, want_logits) < 1e-2
        if rank == 0:
            result.put(float(err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("combine", ["all_reduce", "all_to_all"])
def test_two_cpu_ranks_match_the_single_process_block(combine):
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cpu_rank, args=(r, 2, port, combine, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert result.get(timeout=5) < 1e-2


def _gpu_rank(rank, world, port, combine, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from tests.test_gpu_parity import make_expert
        import tests.test_gpu_parity as tp
        tp.DEV = dev
        hidden, ffn, n_exp, experts, x, gate_w = _problem(hidden=256, ffn=512, n_exp=4, tokens=37)
        local = {e: make_expert(hidden, ffn, experts[e]) for e in range(n_exp) if expert_owner(e, n_exp, world) == rank}
        gate = torch.nn.Linear(hidden, n_exp, bias=False, dtype=torch.bfloat16, device=dev)
        gate.weight.data = gate_w.to(dev)
        moe = ExpertParallelMoe(Cfg(hidden, ffn, n_exp), 0, gate, local, combine=combine)
        for tokens in (37, 1):
            y, _ = moe(x[:tokens].to(dev).reshape(1, tokens, hidden))
            # the device's own routing decision goes into the oracle: a near-tie of two bf16-rounded
            # logits may legitimately be broken differently, and would swamp the comparison
            _, tw, ti, _, _, _ = moe.router.route(x[:tokens].to(dev))
            want, _ = O.moe_forward(x[:tokens], gate_w, experts, routing=(tw.cpu(), ti.cpu()))
            err = O.rel_err(y.cpu().reshape(-1, hidden), want)
            assert err < 1e-2, (tokens, err)
        if rank == 0:
            result.put(float(err))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("combine", ["all_reduce", "all_to_all"])
def test_two_gpu_ranks_match_the_oracle(combine):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_rank, args=(r, 2, port, combine, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert result.get(timeout=5) < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
def test_expert_parallel_decoder_layer_on_one_gpu(ranks):
    """The expert-parallel decoder layer with its ranks emulated one after the other on ONE GPU (each "rank" holds
    only its experts; the all-reduce is a sum of the ranks' fp32 shares): residual stream, next-layer input, router
    logits and cache rows are bit for bit those of the single-GPU layer, for every partition of the 8 experts."""
    from mixtral_offloading_b200 import (AttentionDecode, DecoderLayerDecode, ExpertParallelDecoderLayer, ResidentMoe,
                                         _cabi, add_rmsnorm)
    from tests.helpers import layer_from_oracle, random_layer
    from tests.test_gpu_parity import Cfg, make_expert
    dev = torch.device("cuda:0")
    HD, n_heads, n_kv, ffn, E, max_len = 128, 8, 2, 3584, 8, 16
    hidden = n_heads * HD
    g = torch.Generator().manual_seed(ranks)
    shapes = [(hidden, hidden), (n_kv * HD, hidden), (n_kv * HD, hidden), (hidden, hidden)]
    attn_ods = [random_layer(N, K, 4, 64, 40 + i, std=0.05) for i, (N, K) in enumerate(shapes)]
    lns = [(1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(dev) for _ in range(3)]

    def attention():
        return AttentionDecode(*[layer_from_oracle(od, dev) for od in attn_ods], lns[0], lns[1], n_heads, n_kv, HD, max_len)
    experts = [make_expert(hidden, ffn, (random_layer(ffn, hidden, 2, 16, 100 + 3 * e), random_layer(hidden, ffn, 2, 16, 101 + 3 * e),
                                         random_layer(ffn, hidden, 2, 16, 102 + 3 * e))) for e in range(E)]
    gate = torch.nn.Linear(hidden, E, bias=False, dtype=torch.bfloat16, device=dev)
    gate.weight.data.copy_((0.5 * torch.randn(E, hidden, generator=g)).to(torch.bfloat16))
    single = DecoderLayerDecode(attention(), ResidentMoe(Cfg(hidden, ffn, E), 0, gate, experts), lns[2])
    per = E // ranks
    parts = [ExpertParallelDecoderLayer(attention(), gate, experts[r * per:(r + 1) * per], r * per, E, lns[2])
             for r in range(ranks)]
    lib = _cabi.lib()
    pos = torch.zeros(1, dtype=torch.int32, device=dev)
    seen = set()
    for step in range(6):
        h0 = torch.randn(1, hidden, generator=g).to(torch.bfloat16).to(dev)
        h_a = h0.clone()
        x_a = add_rmsnorm(h_a, None, lns[0], 1e-5)
        logits_a = single(h_a, x_a, pos)
        seen.update(logits_a.float().view(-1).topk(2).indices.tolist())
        # every rank: attention half + its experts' share; then the sum of the shares finishes the layer on each
        states, shares = [], []
        for layer in parts:
            h = h0.clone()
            x = add_rmsnorm(h, None, lns[0], 1e-5)
            d = layer._descriptor(dev)
            need = lib.hqm_decode_layer_ep_scratch_bytes(C.byref(d), per)
            assert need > 0
            from mixtral_offloading_b200.custom_layers import _scratch
            ws = _scratch(dev, need)
            logits = torch.empty((1, E), dtype=torch.bfloat16, device=dev)
            _cabi.check(lib.hqm_decode_layer_ep(_cabi.ptr(h), _cabi.ptr(x), _cabi.ptr(logits), _cabi.ptr(layer.y_partial),
                                                None, C.byref(d), layer.expert_lo, per, _cabi.ptr(pos), _cabi.ptr(ws),
                                                ws.numel(), _cabi.stream_ptr(dev)))
            states.append((h, x, logits))
            shares.append(layer.y_partial.clone())
        total = torch.stack(shares).sum(0)
        assert sum(int((s != 0).any()) for s in shares) <= 2          # at most two ranks own a routed expert
        for r, (h, x, logits) in enumerate(states):
            _cabi.check(lib.hqm_add_f32_rmsnorm(_cabi.ptr(h), _cabi.ptr(total), _cabi.ptr(lns[2]), _cabi.ptr(x), hidden,
                                                1e-5, _cabi.stream_ptr(dev)))
            assert torch.equal(logits, logits_a), (step, r)
            assert torch.equal(h, h_a) and torch.equal(x, x_a), (step, r)
            assert torch.equal(parts[r].attention.k_cache[:, step], single.attention.k_cache[:, step])
        pos += 1
    assert len(seen) > 2
    assert lib.hqm_device_error() == 0


def _decode_problem(dev):
    """A small decoder layer (8 heads, 8 experts of 3584) from fixed seeds: the same tensors on every rank."""
    from mixtral_offloading_b200 import AttentionDecode
    from tests.helpers import layer_from_oracle
    from tests.test_gpu_parity import make_expert
    import tests.test_gpu_parity as tp
    tp.DEV = dev
    HD, n_heads, n_kv, ffn, E, max_len = 128, 8, 2, 3584, 8, 16
    hidden = n_heads * HD
    g = torch.Generator().manual_seed(77)
    shapes = [(hidden, hidden), (n_kv * HD, hidden), (n_kv * HD, hidden), (hidden, hidden)]
    attn_ods = [random_layer(N, K, 4, 64, 40 + i, std=0.05) for i, (N, K) in enumerate(shapes)]
    lns = [(1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(dev) for _ in range(3)]
    attn = AttentionDecode(*[layer_from_oracle(od, dev) for od in attn_ods], lns[0], lns[1], n_heads, n_kv, HD, max_len)
    gate = torch.nn.Linear(hidden, E, bias=False, dtype=torch.bfloat16, device=dev)
    gate.weight.data.copy_((0.5 * torch.randn(E, hidden, generator=g)).to(torch.bfloat16))
    hs = [torch.randn(1, hidden, generator=g).to(torch.bfloat16) for _ in range(6)]

    def expert(e):
        return make_expert(hidden, ffn, (random_layer(ffn, hidden, 2, 16, 100 + 3 * e), random_layer(hidden, ffn, 2, 16, 101 + 3 * e),
                                         random_layer(ffn, hidden, 2, 16, 102 + 3 * e)))
    return hidden, ffn, E, attn, gate, lns, hs, expert


def _gpu_decode_rank(rank, world, port, use_peer, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from mixtral_offloading_b200 import (DecoderLayerDecode, ExpertParallelDecoderLayer, PeerExchange, ResidentMoe, _cabi,
                                         add_rmsnorm)
    from tests.test_gpu_parity import Cfg as GCfg
    hidden, ffn, E, attn, gate, lns, hs, expert = _decode_problem(dev)
    per = E // world
    mine = [expert(e) for e in range(rank * per, (rank + 1) * per)]
    exchange = PeerExchange(dist.group.WORLD, hidden, dev) if use_peer else None
    layer = ExpertParallelDecoderLayer(attn, gate, mine, rank * per, E, lns[2], group=dist.group.WORLD, exchange=exchange)
    pos = torch.zeros(1, dtype=torch.int32, device=dev)
    outs = []
    for h0 in hs:
        h = h0.clone().to(dev)
        x = add_rmsnorm(h, None, lns[0], 1e-5)
        logits = layer(h, x, pos)
        outs.append((h.cpu(), x.cpu(), logits.cpu()))
        pos += 1
    torch.cuda.synchronize(dev)
    assert _cabi.lib().hqm_device_error() == 0
    if rank == 0:
        # the single-GPU layer over all experts, on this rank's GPU, with a fresh cache
        _, _, _, attn1, gate1, lns1, _, expert1 = _decode_problem(dev)
        single = DecoderLayerDecode(attn1, ResidentMoe(GCfg(hidden, ffn, E), 0, gate1, [expert1(e) for e in range(E)]), lns1[2])
        pos.zero_()
        same = True
        for h0, (h_ep, x_ep, lg_ep) in zip(hs, outs):
            h = h0.clone().to(dev)
            x = add_rmsnorm(h, None, lns1[0], 1e-5)
            lg = single(h, x, pos)
            same = same and torch.equal(h.cpu(), h_ep) and torch.equal(x.cpu(), x_ep) and torch.equal(lg.cpu(), lg_ep)
            pos += 1
        result.put(bool(same))
    dist.barrier()
    torch.cuda.synchronize(dev)
    os._exit(0)          # (destroying the group after peer mappings / captured collectives has blocked for minutes)


@pytest.mark.gpu
@pytest.mark.parametrize("use_peer", [False, True])
def test_two_gpu_ranks_decode_layer_equals_one_gpu(use_peer):
    """ExpertParallelDecoderLayer on two GPUs (NCCL all-reduce, and the peer-memory exchange from inside the
    kernels) gives bit for bit the residual stream, next input and router logits of the single-GPU layer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gpu_decode_rank, args=(r, 2, port, use_peer, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        if p.is_alive():
            p.kill()
        assert p.exitcode == 0
    assert result.get(timeout=5) is True
