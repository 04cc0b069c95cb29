"""The whole decoder layer for one token (hqm_decode_layer) at the Mixtral shape against the CPU oracle.

BASELINE configs[3] / [4]: hidden 4096, 32 query / 8 key-value heads of 128, RoPE theta 1e6, RMSNorm eps 1e-5,
4-bit g64 attention projections, router 4096 -> 8, eight 2-bit g16 experts of 14336, a KV cache holding 512
positions before the token.  The oracle (oracle/attention_oracle.py, pinned against transformers, with the
reference's MoE block from oracle/hqq_oracle.py) computes in fp32 on the dequantised weights and rounds to bf16
where the Hugging Face bf16 model would.  The routing is forced to the device's choice so that a near-tie of
two bf16 router logits cannot turn the comparison into one between different experts.

Bounds (max|a - b| / max|b|):
  * the two blocks' own outputs (attention + o_proj, MoE block): 1e-2, the per-layer bound the build targets;
  * the residual stream h after the layer: 1.6e-2.  h is bf16 and |h| reaches 4..8 here, where one bf16 step is
    2^-5 = 0.031, i.e. 0.6e-2 .. 0.8e-2 of max|h|: an element whose pre-rounding value differs from the
    oracle's by far less than the 1e-2 target can still land on the neighbouring bf16 value, and the layer
    rounds h twice (after each residual add).  Two such flips on one element are 1.6e-2; the block outputs, which
    are small next to h, carry the real error and are held to 1e-2;
  * final logits after two teacher-forced layers (each layer fed the oracle's input): 2e-2.
"""
import pytest
import torch

from mixtral_offloading_b200 import AttentionDecode, DecoderLayerDecode, ResidentMoe, _cabi, add_rmsnorm
from oracle import attention_oracle as A
from oracle import hqq_oracle as O
from tests.helpers import layer_from_oracle, random_layer
from tests.test_gpu_parity import make_expert

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
H, NH, NKV, HD, FFN, E = 4096, 32, 8, 128, 14336, 8
CONTEXT, THETA, EPS = 512, 1e6, 1e-5
N_DISTINCT = 3            # distinct expert weight sets per layer (expert e uses set e % 3): quantising 8 takes minutes


class _Cfg:
    hidden_size, intermediate_size, num_local_experts, num_experts_per_tok, hidden_act = H, FFN, E, 2, "silu"


def rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-9))


def build_layer(seed, next_ln):
    """(product layer, oracle layer).  Expert e of the layer points at weight set e % N_DISTINCT."""
    g = torch.Generator().manual_seed(seed)
    attn_ods = [random_layer(n, k, 4, 64, seed=seed + i) for i, (n, k) in
                enumerate(((NH * HD, H), (NKV * HD, H), (NKV * HD, H), (H, NH * HD)))]
    sets = [(random_layer(FFN, H, 2, 16, seed + 10 + 3 * s), random_layer(H, FFN, 2, 16, seed + 11 + 3 * s),
             random_layer(FFN, H, 2, 16, seed + 12 + 3 * s)) for s in range(N_DISTINCT)]
    ln_in = (1 + 0.05 * torch.randn(H, generator=g)).to(torch.bfloat16)
    ln_post = (1 + 0.05 * torch.randn(H, generator=g)).to(torch.bfloat16)
    gate_w = (0.02 * torch.randn(E, H, generator=g)).to(torch.bfloat16)
    kc = torch.randn(NKV, CONTEXT, HD, generator=g).to(torch.bfloat16)
    vc = torch.randn(NKV, CONTEXT, HD, generator=g).to(torch.bfloat16)
    attn = AttentionDecode(*[layer_from_oracle(od, DEV) for od in attn_ods], ln_in.to(DEV), ln_post.to(DEV), NH, NKV, HD,
                           CONTEXT + 264, THETA, EPS)
    attn.k_cache[:, :CONTEXT], attn.v_cache[:, :CONTEXT] = kc.to(DEV), vc.to(DEV)
    dev_sets = [make_expert(H, FFN, ods) for ods in sets]
    gate = torch.nn.Linear(H, E, bias=False, dtype=torch.bfloat16, device=DEV)
    gate.weight.data.copy_(gate_w)
    moe = ResidentMoe(_Cfg, 0, gate, [dev_sets[e % N_DISTINCT] for e in range(E)])
    layer = DecoderLayerDecode(attn, moe, next_ln.to(DEV))
    ref = A.DecoderLayerOracle(attn_ods, ln_in.float(), ln_post.float(), gate_w, [sets[e % N_DISTINCT] for e in range(E)],
                               NH, NKV, HD, CONTEXT + 264, THETA, EPS, round_to=torch.bfloat16)
    ref.attn.kc[:, :CONTEXT], ref.attn.vc[:, :CONTEXT] = kc.float(), vc.float()
    return layer, ref


def device_routing(logits_bf16):
    """The choice the device made, recomputed from the router logits it returned (custom_layers.py:278-282)."""
    lg = logits_bf16.float().cpu().reshape(1, -1)
    p = torch.softmax(lg, dim=1, dtype=torch.float32)
    w, idx = torch.topk(p, 2, dim=-1)
    return w / w.sum(-1, keepdim=True), idx


def run_layer(layer, ref, h0, next_ln):
    """One token at position CONTEXT through both; returns the figures of the comparison."""
    pos = torch.full((1,), CONTEXT, dtype=torch.int32, device=DEV)
    h = h0.clone().to(DEV)
    x = add_rmsnorm(h, None, layer.attention.ln_in, EPS)
    x_in_dev = x.clone()
    logits = layer(h, x, pos)
    assert _cabi.lib().hqm_device_error() == 0
    x_ref_in = A.rms_norm(h0.float(), ref.ln_in, EPS, torch.bfloat16)
    h_ref, parts = ref.step(h0.float(), CONTEXT, routing=device_routing(logits), x_in=x_ref_in)
    x_next_ref = A.rms_norm(h_ref, next_ln.float(), EPS, torch.bfloat16)
    out = dict(
        x_in=rel(x_in_dev, x_ref_in), logits=rel(logits, parts["router_logits"]), h=rel(h, h_ref), x_next=rel(x, x_next_ref),
        k_row=rel(layer.attention.k_cache[:, CONTEXT], ref.attn.kc[:, CONTEXT]),
        v_row=rel(layer.attention.v_cache[:, CONTEXT], ref.attn.vc[:, CONTEXT]))
    return out, h, h_ref


@pytest.fixture(scope="module")
def two_layers():
    g = torch.Generator().manual_seed(9)
    lns = [(1 + 0.05 * torch.randn(H, generator=g)).to(torch.bfloat16) for _ in range(2)]
    return lns, [build_layer(seed=300 + 50 * l, next_ln=lns[l]) for l in range(2)]


@pytest.mark.parametrize("tma_mode", [1, 2])
def test_decoder_layer_full_shape_against_the_oracle(two_layers, tma_mode):
    lib = _cabi.lib()
    prev = lib.hqm_set_tma_mode(tma_mode)
    try:
        g = torch.Generator().manual_seed(5)
        next_ln = two_layers[0][0]
        layer, ref = two_layers[1][0]
        worst = {}
        for trial in range(3):
            h0 = torch.randn(1, H, generator=g).to(torch.bfloat16)
            fig, _, _ = run_layer(layer, ref, h0, next_ln)
            for k, v in fig.items():
                worst[k] = max(worst.get(k, 0.0), v)
            # the cache row written by this trial is overwritten by the next (same position)
        print("decoder layer vs oracle (max rel diff):", {k: round(v, 5) for k, v in worst.items()})
        assert worst["x_in"] < 1e-2 and worst["logits"] < 1e-2
        assert worst["k_row"] < 1e-2 and worst["v_row"] < 1e-2
        assert worst["h"] < 1.6e-2 and worst["x_next"] < 1.6e-2, "bf16 residual stream: see the module docstring"
    finally:
        lib.hqm_set_tma_mode(prev)


def test_blocks_of_the_layer_full_shape(two_layers):
    """The same layer as two calls (hqm_attn_decode, hqm_moe_decode), which expose what each block produces: the
    residual stream after the attention half (one bf16 rounding) and the MoE block's output on the device's own
    input, each within 1e-2 of the oracle."""
    lns, built = two_layers
    layer, ref = built[0]
    g = torch.Generator().manual_seed(23)
    pos = torch.full((1,), CONTEXT, dtype=torch.int32, device=DEV)
    for trial in range(3):
        h0 = torch.randn(1, H, generator=g).to(torch.bfloat16)
        h = h0.clone().to(DEV)
        x_moe = layer.attention(h, pos)                               # h += attention; returns norm(h) * ln_post
        x_ref = A.rms_norm(h0.float(), ref.ln_in, EPS, torch.bfloat16)
        h_mid_ref = A._rnd(h0.float() + ref.attn.step(x_ref, CONTEXT), torch.bfloat16)
        assert rel(h, h_mid_ref) < 1e-2, trial
        assert rel(x_moe, A.rms_norm(h_mid_ref, ref.ln_post, EPS, torch.bfloat16)) < 1e-2, trial
        y, logits = layer.moe(x_moe.view(1, 1, H))
        want, want_logits = O.moe_forward(x_moe.float().cpu(), ref.gate_w, ref.experts, routing=device_routing(logits))
        assert rel(logits, want_logits) < 1e-2, trial
        assert rel(y.view(1, H), want) < 1e-2, trial
    assert _cabi.lib().hqm_device_error() == 0


@pytest.mark.parametrize("T", [32, 256])
def test_decoder_layer_many_tokens_behind_a_filled_cache(two_layers, T):
    """BASELINE configs[3]: the layer at 32 and 256 new tokens on a cache of 512 positions
    (DecoderLayerDecode.forward_tokens: tensor-core linears, torch attention over the cache, per-expert MoE)."""
    lns, built = two_layers
    layer, ref = built[1]
    g = torch.Generator().manual_seed(100 + T)
    h0 = torch.randn(T, H, generator=g).to(torch.bfloat16)
    h_dev, logits = layer.forward_tokens(h0.to(DEV), CONTEXT)
    assert _cabi.lib().hqm_device_error() == 0
    # oracle: the attention half token by token against the cache, then the MoE block for all tokens at once
    h_mid = torch.empty(T, H)
    for t in range(T):
        x = A.rms_norm(h0[t:t + 1].float(), ref.ln_in, EPS, torch.bfloat16)
        h_mid[t] = A._rnd(h0[t:t + 1].float() + ref.attn.step(x, CONTEXT + t), torch.bfloat16)[0]
    x_moe = A.rms_norm(h_mid, ref.ln_post, EPS, torch.bfloat16)
    lg = logits.float().cpu()
    p = torch.softmax(lg, dim=1, dtype=torch.float32)
    w, idx = torch.topk(p, 2, dim=-1)
    moe_out, want_logits = O.moe_forward(x_moe, ref.gate_w, ref.experts, routing=(w / w.sum(-1, keepdim=True), idx))
    h_ref = A._rnd(h_mid + A._rnd(moe_out, torch.bfloat16), torch.bfloat16)
    fig = dict(h=rel(h_dev, h_ref), logits=rel(logits, want_logits),
               k_rows=rel(layer.attention.k_cache[:, CONTEXT:CONTEXT + T], ref.attn.kc[:, CONTEXT:CONTEXT + T]),
               v_rows=rel(layer.attention.v_cache[:, CONTEXT:CONTEXT + T], ref.attn.vc[:, CONTEXT:CONTEXT + T]))
    print(f"decoder layer, {T} tokens behind {CONTEXT} cached positions (max rel diff):", {k: round(v, 5) for k, v in fig.items()})
    # the rotated keys are bf16 values of magnitude 4..8 that went through three bf16 roundings (two products and a
    # sum): over 256 x 1024 of them one lands two bf16 steps from the oracle's (2 x 2^-5 = 1.03e-2 of max|k|)
    assert fig["k_rows"] < 1.6e-2 and fig["v_rows"] < 1e-2 and fig["logits"] < 1e-2
    assert fig["h"] < 1.6e-2


def test_two_layers_teacher_forced_logits(two_layers):
    """Each layer is fed the oracle's input of that layer; the logits of the product's last layer output through
    the final norm and a 32000 x 4096 lm_head stay within 2e-2 of the oracle's."""
    g = torch.Generator().manual_seed(19)
    lns, built = two_layers
    lm_head = (0.02 * torch.randn(32000, H, generator=g)).to(torch.bfloat16)
    h_in = torch.randn(1, H, generator=g).to(torch.bfloat16)
    for l, (layer, ref) in enumerate(built):
        fig, h_dev, h_ref = run_layer(layer, ref, h_in, lns[l])
        assert fig["h"] < 1.6e-2 and fig["logits"] < 1e-2, (l, fig)
        if l + 1 < len(built):
            h_in = h_ref.to(torch.bfloat16)                 # teacher forcing: the next layer sees the oracle's stream
    x_dev = A.rms_norm(h_dev.float().cpu(), lns[-1].float(), EPS, torch.bfloat16)
    x_ref = A.rms_norm(h_ref, lns[-1].float(), EPS, torch.bfloat16)
    logits_dev = x_dev @ lm_head.float().t()
    logits_ref = x_ref @ lm_head.float().t()
    err = rel(logits_dev, logits_ref)
    print("teacher-forced final logits max rel diff:", round(err, 5))
    assert err < 2e-2


def test_batch_of_eight_sequences_against_the_oracle(two_layers):
    """BASELINE configs[4] at batch 8: eight sequences, each one token behind its own 512-position cache, through
    one full-shape layer, the final norm and a 1000 x 4096 head (BatchDecode); every sequence against the oracle."""
    from mixtral_offloading_b200 import BatchDecode, MixtralDecodeModel
    B = 8
    g = torch.Generator().manual_seed(29)
    lns, built = two_layers
    layer, ref = built[0]
    embed = torch.randn(B, H, generator=g).to(torch.bfloat16)                 # row b = the stream of sequence b
    lm_head = (0.02 * torch.randn(1000, H, generator=g)).to(torch.bfloat16)
    model = MixtralDecodeModel(embed.to(DEV), [layer], layer.attention.ln_in, lm_head.to(DEV), rms_eps=EPS)
    batch = BatchDecode(model, B, CONTEXT + 8)
    prefix_k, prefix_v = ref.attn.kc[:, :CONTEXT].clone(), ref.attn.vc[:, :CONTEXT].clone()
    for b in range(B):          # sequence b sees the prefix rolled by b positions: eight different histories
        batch.k_caches[0][b, :, :CONTEXT] = prefix_k.roll(b, 1).to(torch.bfloat16).to(DEV)
        batch.v_caches[0][b, :, :CONTEXT] = prefix_v.roll(b, 1).to(torch.bfloat16).to(DEV)
    logits = batch.step(torch.arange(B, device=DEV), CONTEXT).float().cpu()
    assert _cabi.lib().hqm_device_error() == 0
    router = batch.router_logits[0].float().cpu()
    k_row = batch.k_caches[0][:, :, CONTEXT].clone()
    batch.capture()                                  # the same step from recorded segments: identical results
    batch.k_caches[0][:, :, CONTEXT] = 0
    again = batch.step(torch.arange(B, device=DEV), CONTEXT).float().cpu()
    assert torch.equal(again, logits) and torch.equal(batch.k_caches[0][:, :, CONTEXT], k_row)
    worst = dict(logits=0.0, router=0.0, k=0.0)
    for b in range(B):
        ref.attn.kc[:, :CONTEXT], ref.attn.vc[:, :CONTEXT] = prefix_k.roll(b, 1), prefix_v.roll(b, 1)
        h_ref, parts = ref.step(embed[b:b + 1].float(), CONTEXT, routing=device_routing(router[b:b + 1].to(torch.bfloat16)))
        want = A.rms_norm(h_ref, lns[0].float(), EPS, torch.bfloat16) @ lm_head.float().t()
        worst["logits"] = max(worst["logits"], rel(logits[b:b + 1], want))
        worst["router"] = max(worst["router"], rel(router[b:b + 1], parts["router_logits"]))
        worst["k"] = max(worst["k"], rel(batch.k_caches[0][b, :, CONTEXT], ref.attn.kc[:, CONTEXT]))
    ref.attn.kc[:, :CONTEXT], ref.attn.vc[:, :CONTEXT] = prefix_k, prefix_v
    print("batch of 8, worst sequence:", {k: round(v, 5) for k, v in worst.items()})
    assert worst["logits"] < 2e-2 and worst["router"] < 1e-2 and worst["k"] < 1e-2
