"""The single-token attention block (hqm_attn_decode) and the fused residual-add + RMSNorm against a torch
restatement of the Hugging Face decoder-layer arithmetic on the oracle's dequantised weights."""
import math

import pytest
import torch

from mixtral_offloading_b200 import (AttentionDecode, DecoderLayerDecode, MixtralDecodeModel, ResidentMoe,
                                     add_rmsnorm)
from oracle import hqq_oracle as O
from tests.helpers import layer_from_oracle, random_layer

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
HD = 128


def bf(x):
    return x.to(torch.bfloat16).float()


def rms_ref(h, w, eps):
    v = h.float()
    return bf(w.float() * bf(v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)))


def rope_ref(t, pos, theta):                       # t: (heads, HD) float holding bf16 values
    inv = theta ** (-torch.arange(0, HD, 2, dtype=torch.float32) / HD)
    ang = pos * inv
    cos, sin = bf(torch.cat([ang.cos(), ang.cos()])), bf(torch.cat([ang.sin(), ang.sin()]))
    rot = torch.cat([-t[:, HD // 2:], t[:, :HD // 2]], -1)
    return bf(bf(t * cos) + bf(rot * sin))


class RefLayer:
    """Float restatement of one attention block with its own cache."""

    def __init__(self, ods, ln_in, ln_post, n_heads, n_kv, max_len, theta, eps):
        self.W = [O.dequantize(od).float() for od in ods]          # q, k, v, o as (N, K)
        self.ln_in, self.ln_post = ln_in.float(), ln_post.float()
        self.nh, self.nkv, self.theta, self.eps = n_heads, n_kv, theta, eps
        self.kc = torch.zeros(n_kv, max_len, HD)
        self.vc = torch.zeros(n_kv, max_len, HD)

    def step(self, h, pos, delta=None):
        h = h.float()
        if delta is not None:
            h = bf(h + delta.float())
        x = rms_ref(h, self.ln_in, self.eps)
        q = bf(x @ self.W[0].t()).view(self.nh, HD)
        k = bf(x @ self.W[1].t()).view(self.nkv, HD)
        v = bf(x @ self.W[2].t()).view(self.nkv, HD)
        q, k = rope_ref(q, pos, self.theta), rope_ref(k, pos, self.theta)
        self.kc[:, pos], self.vc[:, pos] = k, v
        grp = self.nh // self.nkv
        K = self.kc[:, :pos + 1].repeat_interleave(grp, 0)          # (nh, len, HD)
        V = self.vc[:, :pos + 1].repeat_interleave(grp, 0)
        p = torch.softmax(torch.einsum("hd,hld->hl", q, K) / math.sqrt(HD), -1)
        ctx = bf(torch.einsum("hl,hld->hd", p, V)).reshape(1, -1)
        h = bf(h + bf(ctx @ self.W[3].t()))
        return h, rms_ref(h, self.ln_post, self.eps)


def build(n_heads, n_kv, max_len, seed, theta=1e6, eps=1e-5):
    hidden = n_heads * HD
    shapes = [(hidden, hidden), (n_kv * HD, hidden), (n_kv * HD, hidden), (hidden, hidden)]
    ods = [random_layer(N, K, 4, 64, seed + i, std=0.05) for i, (N, K) in enumerate(shapes)]
    g = torch.Generator().manual_seed(seed + 99)
    ln_in = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    ln_post = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    layers = [layer_from_oracle(od, DEV) for od in ods]
    mod = AttentionDecode(*layers, ln_in.to(DEV), ln_post.to(DEV), n_heads, n_kv, HD, max_len, theta, eps)
    return mod, RefLayer(ods, ln_in, ln_post, n_heads, n_kv, max_len, theta, eps), hidden


def rel(a, b):
    return float((a.float().cpu() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-9))


@pytest.mark.parametrize("n_heads,n_kv", [(4, 2), (8, 8), (8, 1)])
def test_attention_decode_follows_the_reference_over_several_positions(n_heads, n_kv):
    mod, ref, hidden = build(n_heads, n_kv, max_len=48, seed=11 * n_heads + n_kv)
    g = torch.Generator().manual_seed(3)
    pos = torch.zeros(1, dtype=torch.int32, device=DEV)
    h_ref = torch.randn(1, hidden, generator=g).to(torch.bfloat16)
    h = h_ref.clone().to(DEV)
    for step in range(40):
        delta = (0.3 * torch.randn(1, hidden, generator=g)).to(torch.bfloat16) if step % 2 else None
        x = mod(h, pos, None if delta is None else delta.to(DEV))
        h_ref, x_ref = ref.step(h_ref, step, delta)
        assert rel(h, h_ref) < 2e-2, step
        assert rel(x, x_ref) < 2e-2, step
        h_ref = h.cpu().clone()                      # keep the two residual streams from drifting apart
        # the cache rows the kernel wrote are what the reference wrote
        assert rel(mod.k_cache[:, step], ref.kc[:, step]) < 2e-2
        assert rel(mod.v_cache[:, step], ref.vc[:, step]) < 2e-2
        ref.kc[:, step], ref.vc[:, step] = mod.k_cache[:, step].float().cpu(), mod.v_cache[:, step].float().cpu()
        pos += 1


def test_attention_decode_full_size_long_context_in_a_graph():
    """Mixtral shape (32 / 8 heads), 700 cached positions, captured and replayed with an advancing position."""
    n_heads, n_kv, max_len, ctx_len = 32, 8, 768, 700
    mod, ref, hidden = build(n_heads, n_kv, max_len, seed=5)
    g = torch.Generator().manual_seed(8)
    kc = torch.randn(n_kv, ctx_len, HD, generator=g).to(torch.bfloat16)
    vc = torch.randn(n_kv, ctx_len, HD, generator=g).to(torch.bfloat16)
    mod.k_cache[:, :ctx_len], mod.v_cache[:, :ctx_len] = kc.to(DEV), vc.to(DEV)
    ref.kc[:, :ctx_len], ref.vc[:, :ctx_len] = kc.float(), vc.float()
    pos = torch.full((1,), ctx_len, dtype=torch.int32, device=DEV)
    h0 = torch.randn(1, hidden, generator=g).to(torch.bfloat16)
    h = h0.clone().to(DEV)
    h_in = h0.clone().to(DEV)

    def step():
        h.copy_(h_in)
        x = mod(h, pos)
        pos.add_(1)
        return x

    step()                                            # settle allocations
    pos.fill_(ctx_len)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        x = step()
    pos.fill_(ctx_len)
    for i in range(3):
        graph.replay()
        torch.cuda.synchronize()
        h_ref, x_ref = ref.step(h0, ctx_len + i)
        assert rel(h, h_ref) < 2e-2 and rel(x, x_ref) < 2e-2, i
        ref.kc[:, ctx_len + i] = mod.k_cache[:, ctx_len + i].float().cpu()
        ref.vc[:, ctx_len + i] = mod.v_cache[:, ctx_len + i].float().cpu()
    assert int(pos.item()) == ctx_len + 3


def test_position_outside_the_cache_is_reported_not_written():
    from mixtral_offloading_b200 import _cabi
    mod, _, hidden = build(4, 2, max_len=8, seed=2)
    h = torch.randn(1, hidden).to(torch.bfloat16).to(DEV)
    before = mod.k_cache.clone()
    mod(h, torch.full((1,), 8, dtype=torch.int32, device=DEV))
    assert _cabi.lib().hqm_device_error() == 2
    assert torch.equal(mod.k_cache, before)
    assert _cabi.lib().hqm_device_error() == 0           # reading the flag cleared it


def test_add_rmsnorm():
    g = torch.Generator().manual_seed(1)
    for hidden in (512, 4096, 5120):
        h = torch.randn(1, hidden, generator=g).to(torch.bfloat16)
        d = torch.randn(1, hidden, generator=g).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
        hd = h.clone().to(DEV)
        x = add_rmsnorm(hd, d.to(DEV), w.to(DEV), 1e-5)
        h_ref = bf(h.float() + d.float())
        assert torch.equal(hd.cpu().float(), h_ref)
        assert rel(x, rms_ref(h_ref, w, 1e-5)) < 1e-2
        hd2 = h.clone().to(DEV)
        x2 = add_rmsnorm(hd2, None, w.to(DEV), 1e-5)
        assert torch.equal(hd2.cpu(), h) and rel(x2, rms_ref(h, w, 1e-5)) < 1e-2


class _Cfg:
    def __init__(self, hidden, ffn, n_exp):
        self.hidden_size, self.intermediate_size, self.num_local_experts = hidden, ffn, n_exp
        self.num_experts_per_tok, self.hidden_act = 2, "silu"


def test_fused_decoder_layer_matches_the_two_separate_calls():
    """hqm_decode_layer against AttentionDecode + ResidentMoe + add_rmsnorm on the same weights, over several
    positions: same residual stream, same next-layer input, same router logits, same cache rows."""
    from tests.test_gpu_parity import make_expert
    n_heads, n_kv, ffn, E, max_len = 8, 2, 3584, 8, 32
    hidden = n_heads * HD
    mod, _, _ = build(n_heads, n_kv, max_len, seed=21)
    mod2, _, _ = build(n_heads, n_kv, max_len, seed=21)                 # same weights, own cache
    experts = [make_expert(hidden, ffn, (random_layer(ffn, hidden, 2, 16, 100 + 3 * e), random_layer(hidden, ffn, 2, 16, 101 + 3 * e),
                                         random_layer(ffn, hidden, 2, 16, 102 + 3 * e))) for e in range(E)]
    g = torch.Generator().manual_seed(4)
    gate = torch.nn.Linear(hidden, E, bias=False, dtype=torch.bfloat16, device=DEV)
    gate.weight.data.copy_((0.5 * torch.randn(E, hidden, generator=g)).to(torch.bfloat16))
    moe = ResidentMoe(_Cfg(hidden, ffn, E), 0, gate, experts)
    next_ln = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(DEV)
    fused = DecoderLayerDecode(mod2, moe, next_ln)
    pos = torch.zeros(1, dtype=torch.int32, device=DEV)
    for step in range(12):
        h0 = torch.randn(1, hidden, generator=g).to(torch.bfloat16).to(DEV)
        # separate calls
        h_a = h0.clone()
        x_moe = mod(h_a, pos)                                            # norm(ln_in) inside
        y, logits_a = moe(x_moe.view(1, 1, hidden))
        x_a = add_rmsnorm(h_a, y.view(1, hidden), next_ln, 1e-5)
        # fused layer: the caller provides the normalised input
        h_b = h0.clone()
        x_b = add_rmsnorm(h_b, None, mod.ln_in, 1e-5)
        logits_b = fused(h_b, x_b, pos)
        assert rel(logits_b, logits_a.float().cpu()) < 1e-2, step
        if set(logits_a.float().view(-1).topk(2).indices.tolist()) == set(logits_b.float().view(-1).topk(2).indices.tolist()):
            assert rel(h_b, h_a.float().cpu()) < 1e-2, step
            assert rel(x_b, x_a.float().cpu()) < 1e-2, step
        assert rel(mod2.k_cache[:, step], mod.k_cache[:, step].float().cpu()) < 1e-2
        assert rel(mod2.v_cache[:, step], mod.v_cache[:, step].float().cpu()) < 1e-2
        pos += 1


def test_generate_graph_and_eager_agree_and_repeat():
    """Two small layers, greedy generation: replaying the captured step gives the tokens of the eager step, twice."""
    from tests.test_gpu_parity import make_expert
    n_heads, n_kv, ffn, E, max_len, vocab, L = 4, 2, 1792, 8, 64, 500, 2
    hidden = n_heads * HD
    g = torch.Generator().manual_seed(12)
    lns = [(1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(DEV) for _ in range(L + 1)]
    layers = []
    for l in range(L):
        attn, _, _ = build(n_heads, n_kv, max_len, seed=31 + 7 * l)
        experts = [make_expert(hidden, ffn, (random_layer(ffn, hidden, 2, 16, 300 + 30 * l + 3 * e),
                                             random_layer(hidden, ffn, 2, 16, 301 + 30 * l + 3 * e),
                                             random_layer(ffn, hidden, 2, 16, 302 + 30 * l + 3 * e))) for e in range(E)]
        gate = torch.nn.Linear(hidden, E, bias=False, dtype=torch.bfloat16, device=DEV)
        gate.weight.data.copy_((0.5 * torch.randn(E, hidden, generator=g)).to(torch.bfloat16))
        layers.append(DecoderLayerDecode(attn, ResidentMoe(_Cfg(hidden, ffn, E), l, gate, experts), lns[l + 1]))
    embed = torch.randn(vocab, hidden, generator=g).to(torch.bfloat16).to(DEV)
    head = (0.05 * torch.randn(vocab, hidden, generator=g)).to(torch.bfloat16).to(DEV)
    model = MixtralDecodeModel(embed, layers, lns[0], head)
    prompt = [3, 141, 59, 26, 5]
    eager = model.generate(prompt, 12, use_graph=False)
    graphed = model.generate(prompt, 12, use_graph=True)
    # a larger workspace request after the capture (a long prompt, say) must not pull the captured step's
    # workspace from under it: the outgrown buffer stays alive
    from mixtral_offloading_b200.custom_layers import _SCRATCH, _scratch
    old_buf = _SCRATCH[("cuda", 0)]
    new_buf = _scratch(DEV, 4 * old_buf.numel())
    assert new_buf.data_ptr() != old_buf.data_ptr() and new_buf.numel() >= 4 * old_buf.numel()
    new_buf.fill_(0xFF)
    _cabi_lib = __import__("mixtral_offloading_b200")._cabi
    _cabi_lib.check(_cabi_lib.lib().hqm_scratch_init(_cabi_lib.ptr(new_buf), _cabi_lib.stream_ptr(DEV)))   # its header: zero again
    again = model.generate(prompt, 12, use_graph=True)
    assert len(eager) == 12 and all(0 <= t < vocab for t in eager)
    assert graphed == eager and again == eager
    assert int(model.position.item()) == len(prompt) + 11
    with pytest.raises(ValueError):
        model.generate(prompt, max_len)


def test_prefill_matches_feeding_the_prompt_token_by_token():
    """prefill() fills the caches and predicts the next token like the single-token step fed with the prompt."""
    from tests.test_gpu_parity import make_expert
    n_heads, n_kv, ffn, E, max_len, vocab, L = 4, 2, 1792, 8, 64, 300, 2
    hidden = n_heads * HD
    g = torch.Generator().manual_seed(77)
    lns = [(1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(DEV) for _ in range(L + 1)]
    layers = []
    for l in range(L):
        attn, _, _ = build(n_heads, n_kv, max_len, seed=51 + 7 * l)
        experts = [make_expert(hidden, ffn, (random_layer(ffn, hidden, 2, 16, 500 + 30 * l + 3 * e),
                                             random_layer(hidden, ffn, 2, 16, 501 + 30 * l + 3 * e),
                                             random_layer(ffn, hidden, 2, 16, 502 + 30 * l + 3 * e))) for e in range(E)]
        gate = torch.nn.Linear(hidden, E, bias=False, dtype=torch.bfloat16, device=DEV)
        gate.weight.data.copy_((0.5 * torch.randn(E, hidden, generator=g)).to(torch.bfloat16))
        layers.append(DecoderLayerDecode(attn, ResidentMoe(_Cfg(hidden, ffn, E), l, gate, experts), lns[l + 1]))
    embed = torch.randn(vocab, hidden, generator=g).to(torch.bfloat16).to(DEV)
    head = (0.05 * torch.randn(vocab, hidden, generator=g)).to(torch.bfloat16).to(DEV)
    model = MixtralDecodeModel(embed, layers, lns[0], head)
    prompt = [int(v) for v in torch.randint(0, vocab, (20,), generator=g)]
    # token by token
    model.position.zero_()
    for tkn in prompt:
        model.token.fill_(tkn)
        logits_step = model.step().float().cpu()
    caches_step = [(l.attention.k_cache[:, :20].float().cpu(), l.attention.v_cache[:, :20].float().cpu()) for l in layers]
    # one pass
    logits_pre = model.prefill(prompt).float().cpu()
    assert int(model.position.item()) == 20
    # bf16 noise compounds through the layers and a router near-tie may flip for some token: compare loosely
    assert rel(caches_step[0][0], layers[0].attention.k_cache[:, :20].float().cpu()) < 2e-2   # layer 0 sees equal inputs
    assert rel(caches_step[0][1], layers[0].attention.v_cache[:, :20].float().cpu()) < 2e-2
    assert rel(logits_pre, logits_step) < 0.15
    assert len(model.generate(prompt, 5, prefill=True)) == 5


def test_row_kernels_against_the_oracle():
    """hqm_add_rmsnorm_rows and hqm_rope_append_rows (a prompt's layout and a batch's) against the pinned oracle's
    RMSNorm and rotary embedding with bf16 rounding where the Hugging Face bf16 model rounds."""
    from mixtral_offloading_b200 import _cabi
    from mixtral_offloading_b200.decoder import rms_norm_rows, rope_append_rows
    from oracle import attention_oracle as A
    g = torch.Generator().manual_seed(5)
    T, n_heads, n_kv, max_len, theta = 37, 4, 2, 64, 1e6
    hidden = n_heads * HD
    h = (3 * torch.randn(T, hidden, generator=g)).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    x = rms_norm_rows(h.to(DEV), w.to(DEV), 1e-5).float().cpu()
    want = A.rms_norm(h.float(), w.float(), 1e-5, torch.bfloat16)
    assert rel(x, want) < 4e-3                                     # one bf16 step where the fp32 normalisation differs
    q = torch.randn(T, n_heads * HD, generator=g).to(torch.bfloat16)
    k = torch.randn(T, n_kv * HD, generator=g).to(torch.bfloat16)
    v = torch.randn(T, n_kv * HD, generator=g).to(torch.bfloat16)
    pos0 = 11
    cos, sin = A.rope_cos_sin(torch.arange(pos0, pos0 + T), HD, theta, torch.bfloat16)
    q_ref = A.apply_rope(q.float().view(T, n_heads, HD), cos[:, None, :], sin[:, None, :], torch.bfloat16)
    k_ref = A.apply_rope(k.float().view(T, n_kv, HD), cos[:, None, :], sin[:, None, :], torch.bfloat16)
    # a prompt: one cache, consecutive positions
    qd = q.clone().to(DEV)
    kc = torch.zeros(n_kv, max_len, HD, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    rope_append_rows(qd, k.to(DEV), v.to(DEV), kc, vc, n_heads, n_kv, HD, theta, pos0, 1)
    assert rel(qd.view(T, n_heads, HD), q_ref) < 1e-2
    assert rel(kc[:, pos0:pos0 + T].transpose(0, 1), k_ref) < 1e-2
    assert torch.equal(vc[:, pos0:pos0 + T].transpose(0, 1).cpu(), v.view(T, n_kv, HD))
    assert float(kc[:, :pos0].abs().max()) == 0 and float(kc[:, pos0 + T:].abs().max()) == 0
    # a batch: one cache per token, all at the position held in device memory
    B, pos = 5, 23
    cosb, sinb = A.rope_cos_sin(pos, HD, theta, torch.bfloat16)
    kb_ref = A.apply_rope(k[:B].float().view(B, n_kv, HD), cosb, sinb, torch.bfloat16)
    qd = q[:B].clone().to(DEV)
    kcb = torch.zeros(B, n_kv, max_len, HD, dtype=torch.bfloat16, device=DEV)
    vcb = torch.zeros_like(kcb)
    rope_append_rows(qd, k[:B].contiguous().to(DEV), v[:B].contiguous().to(DEV), kcb, vcb, n_heads, n_kv, HD, theta,
                     torch.tensor([pos], dtype=torch.int64, device=DEV), 0)
    assert rel(kcb[:, :, pos], kb_ref) < 1e-2
    assert torch.equal(vcb[:, :, pos].cpu(), v[:B].view(B, n_kv, HD))
    assert _cabi.lib().hqm_device_error() == 0
    # a position outside the cache is reported, nothing is written
    rope_append_rows(qd, k[:B].contiguous().to(DEV), v[:B].contiguous().to(DEV), kcb, vcb, n_heads, n_kv, HD, theta,
                     torch.tensor([max_len], dtype=torch.int64, device=DEV), 0)
    assert _cabi.lib().hqm_device_error() == 2


def _small_model(max_len=96, vocab=300, seed=91):
    from tests.test_gpu_parity import make_expert
    n_heads, n_kv, ffn, E, L = 4, 2, 1792, 8, 2
    hidden = n_heads * HD
    g = torch.Generator().manual_seed(seed)
    lns = [(1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).to(DEV) for _ in range(L + 1)]
    layers = []
    for l in range(L):
        attn, _, _ = build(n_heads, n_kv, max_len, seed=seed + 7 * l)
        experts = [make_expert(hidden, ffn, (random_layer(ffn, hidden, 2, 16, 700 + 30 * l + 3 * e),
                                             random_layer(hidden, ffn, 2, 16, 701 + 30 * l + 3 * e),
                                             random_layer(ffn, hidden, 2, 16, 702 + 30 * l + 3 * e))) for e in range(E)]
        gate = torch.nn.Linear(hidden, E, bias=False, dtype=torch.bfloat16, device=DEV)
        gate.weight.data.copy_((0.5 * torch.randn(E, hidden, generator=g)).to(torch.bfloat16))
        layers.append(DecoderLayerDecode(attn, ResidentMoe(_Cfg(hidden, ffn, E), l, gate, experts), lns[l + 1]))
    embed = torch.randn(vocab, hidden, generator=g).to(torch.bfloat16).to(DEV)
    head = (0.05 * torch.randn(vocab, hidden, generator=g)).to(torch.bfloat16).to(DEV)
    return MixtralDecodeModel(embed, layers, lns[0], head), vocab


def test_generate_sampling_and_multi_turn():
    """The demo's generation settings (do_sample, temperature 0.9, top_p 0.9) and its multi-turn loop (the caches are
    kept and the next turn is appended): sampled tokens are reproducible under a seeded generator, and a second
    turn behind kept caches equals feeding the whole conversation from empty caches."""
    model, vocab = _small_model()
    p1, p2 = [5, 17, 250, 9, 33], [7, 120, 64]
    out1 = model.generate(p1, 4)
    out2 = model.generate([out1[-1]] + p2, 3, continue_cache=True)           # the last chosen token has not been fed yet
    assert model.generate(p1 + out1 + p2, 3) == out2
    assert model.generate(p1 + out1 + p2, 3, prefill=True, use_graph=False)[0] in range(vocab)
    draws = []
    for _ in range(2):
        g = torch.Generator(device=DEV).manual_seed(11)
        draws.append(model.generate(p1, 12, do_sample=True, temperature=0.9, top_p=0.9, generator=g))
    assert draws[0] == draws[1] and len(draws[0]) == 12 and all(0 <= t < vocab for t in draws[0])
    assert draws[0] != model.generate(p1, 12)                                 # flat random logits: sampling differs from greedy
    eos = model.generate(p1, 12)[2]
    assert model.generate(p1, 12, eos_token_id=eos)[-1] == eos and len(model.generate(p1, 12, eos_token_id=eos)) <= 3
