// Expert FFN: w2( silu(w1 x) * w3 x ), with the gather of the routed rows in
// front and the routing-weight scale + accumulate into the MoE output behind
// (MixtralBLockSparseTop2MLP_HQQ.forward and the per-expert body of
// SparseMoeWrapper.forward in the reference's custom_layers.py).
#include "common.cuh"
#include "kernels.cuh"

namespace hqm {

// h = silu(a) * b, in place in a.  Both operands are the bf16 outputs of the
// w1 / w3 linears, the product is rounded to bf16 as the reference rounds to fp16.
__global__ void silu_mul_kernel(uint16_t* __restrict__ a, const uint16_t* __restrict__ b, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float av = bf16_bits_to_float(a[i]), bv = bf16_bits_to_float(b[i]);
        const float act = round_bf16(av / (1.f + __expf(-av)));
        a[i] = float_to_bf16_bits(act * bv);
    }
}

// out[t] = (accumulate ? out[t] : 0) + w_i * y[i]; one expert touches a token at
// most once, so plain read-modify-write is race free.
__global__ void scale_scatter_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ y,
                                     const int32_t* __restrict__ token_idx, const float* __restrict__ route_w,
                                     int64_t M, int H, int accumulate) {
    const int64_t total = M * H;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / H;
        const int h = (int)(i % H);
        const int64_t t = token_idx ? token_idx[m] : m;
        const float wgt = route_w ? route_w[m] : 1.f;
        const float v = round_bf16(bf16_bits_to_float(y[i]) * wgt);
        uint16_t* dst = out + t * H + h;
        *dst = float_to_bf16_bits(accumulate ? bf16_bits_to_float(*dst) + v : v);
    }
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static bool same_format(const hqm_weight* a, const hqm_weight* b) {
    return a->N == b->N && a->K == b->K && a->nbits == b->nbits && a->group_size == b->group_size &&
           a->meta_group == b->meta_group;
}

// The tensor-core path for a whole expert (many rows): [w1; w3] GEMM -> silu * mul -> w2 GEMM -> scatter.
struct TcPlan {
    int G1, C1, G2, C2;
    size_t up_bytes, h_bytes, down_bytes;
    size_t gather_bytes;      // the routed rows of x made contiguous (the TMA-staged GEMM copies x by tiles)
};
static bool tc_plan(int64_t M, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3, const void* x,
                    TcPlan* tp) {
    if (force_generic() || M < TC_MIN_ROWS || !same_format(w1, w3)) return false;
    if (check_weight(w1, &tp->G1, &tp->C1) != HQM_OK || check_weight(w3, &tp->G1, &tp->C1) != HQM_OK ||
        check_weight(w2, &tp->G2, &tp->C2) != HQM_OK)
        return false;
    if (x && (reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;
    if (!gemm_tc_supported(w1, tp->G1, tp->C1, M) || !gemm_tc_supported(w3, tp->G1, tp->C1, M) ||
        !gemm_tc_supported(w2, tp->G2, tp->C2, M))
        return false;
    tp->up_bytes = align_up((size_t)M * 2 * w1->N * sizeof(float), 256);
    tp->h_bytes = align_up((size_t)M * w1->N * 2, 256);
    tp->down_bytes = align_up((size_t)M * w2->N * sizeof(float), 256);
    tp->gather_bytes = gemm_tma_supported(w1, tp->G1, tp->C1, M) ? align_up((size_t)M * w1->K * 2, 256) : 0;
    return true;
}

// The streaming path for a whole expert: w1 and w3 in one launch, then w2.
struct FusedPlan {
    StreamPlan up, down;
    int G1, C1, G2, C2;
    size_t up_bytes, h_bytes, down_bytes;
};
static bool fused_plan(int64_t M, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3, const void* x,
                       FusedPlan* fp) {
    if (force_generic() || !same_format(w1, w3)) return false;
    if (check_weight(w1, &fp->G1, &fp->C1) != HQM_OK || check_weight(w3, &fp->G1, &fp->C1) != HQM_OK ||
        check_weight(w2, &fp->G2, &fp->C2) != HQM_OK)
        return false;
    if (x && (reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;
    const hqm_weight* up[2] = {w1, w3};
    const hqm_weight* down[1] = {w2};
    if (!gemv_stream_plan(up, 2, M, &fp->up) || !gemv_stream_plan(down, 1, M, &fp->down)) return false;
    fp->up_bytes = align_up(gemv_stream_scratch_bytes(fp->up, M), 256);
    fp->h_bytes = align_up((size_t)M * w1->N * 2, 256);
    fp->down_bytes = align_up(gemv_stream_scratch_bytes(fp->down, M), 256);
    return true;
}

}  // namespace hqm

extern "C" {

size_t hqm_expert_ffn_scratch_bytes(int64_t M, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3) {
    if (!w1 || !w2 || !w3 || M <= 0) return 0;
    const size_t H = hqm::SCRATCH_HEADER;
    hqm::TcPlan tp;
    if (hqm::tc_plan(M, w1, w2, w3, nullptr, &tp)) return H + tp.up_bytes + tp.h_bytes + tp.down_bytes + tp.gather_bytes;
    hqm::FusedPlan fp;
    if (hqm::fused_plan(M, w1, w2, w3, nullptr, &fp)) return H + fp.up_bytes + fp.h_bytes + fp.down_bytes;
    const size_t a = hqm::align_up((size_t)M * (size_t)w1->N * 2, 256);
    const size_t b = hqm::align_up((size_t)M * (size_t)w3->N * 2, 256);
    const size_t c = hqm::align_up((size_t)M * (size_t)w2->N * 2, 256);
    size_t lin = hqm::linear_scratch_bytes(M, w1);
    lin = lin > hqm::linear_scratch_bytes(M, w3) ? lin : hqm::linear_scratch_bytes(M, w3);
    lin = lin > hqm::linear_scratch_bytes(M, w2) ? lin : hqm::linear_scratch_bytes(M, w2);
    return H + a + b + c + lin;
}

int hqm_expert_ffn(uint16_t* out, const uint16_t* x, int64_t M, const int32_t* token_idx, const float* route_w,
                   int accumulate, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3, void* scratch,
                   size_t scratch_bytes, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(M >= 0 && M <= INT32_MAX, "expert_ffn: bad row count %lld", (long long)M);
    if (M == 0) return HQM_OK;
    HQM_CHECK_ARG(out && x && w1 && w2 && w3, "expert_ffn: null pointer");
    HQM_CHECK_ARG(w1->N == w3->N && w1->K == w3->K, "expert_ffn: w1 (%d,%d) and w3 (%d,%d) differ", w1->N, w1->K,
                  w3->N, w3->K);
    HQM_CHECK_ARG(w2->K == w1->N && w2->N == w1->K, "expert_ffn: w2 (%d,%d) does not map (%d) back to (%d)", w2->N,
                  w2->K, w1->N, w1->K);
    const size_t need = hqm_expert_ffn_scratch_bytes(M, w1, w2, w3);
    if (scratch == nullptr || scratch_bytes < need) {
        set_error("expert_ffn: scratch of %zu bytes given, %zu needed", scratch_bytes, need);
        return HQM_ERR_SCRATCH;
    }
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "expert_ffn: scratch must be 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int F = w1->N, H = w2->N;
    uint32_t* counters = (uint32_t*)scratch;
    uint8_t* p = (uint8_t*)scratch + SCRATCH_HEADER;
    TcPlan tp;
    if (tc_plan(M, w1, w2, w3, x, &tp)) {
        float* up = (float*)p;
        uint16_t* h = (uint16_t*)(p + tp.up_bytes);
        float* down = (float*)(p + tp.up_bytes + tp.h_bytes);
        int rc;
        if (token_idx && tp.gather_bytes) {
            uint16_t* xg = (uint16_t*)(p + tp.up_bytes + tp.h_bytes + tp.down_bytes);
            rc = launch_gather_rows(xg, x, token_idx, M, w1->K, st);
            if (rc != HQM_OK) return rc;
            rc = launch_gemm_tc(up, xg, nullptr, M, w1, w3, tp.G1, tp.C1, st);
        } else {
            rc = launch_gemm_tc(up, x, token_idx, M, w1, w3, tp.G1, tp.C1, st);
        }
        if (rc != HQM_OK) return rc;
        rc = launch_silu_mul_from_sums(h, up, M, F, st);
        if (rc != HQM_OK) return rc;
        rc = launch_gemm_tc(down, h, nullptr, M, w2, nullptr, tp.G2, tp.C2, st);
        if (rc != HQM_OK) return rc;
        return launch_scatter_from_sums(out, down, token_idx, route_w, accumulate, M, H, st);
    }
    FusedPlan fp;
    if (fused_plan(M, w1, w2, w3, x, &fp)) {
        // 4 launches: [w1;w3] partials -> h = silu(a) * b -> w2 partials -> scale / accumulate into out
        float* up = (float*)p;
        uint16_t* h = (uint16_t*)(p + fp.up_bytes);
        float* down = (float*)(p + fp.up_bytes + fp.h_bytes);
        StreamJob gate_up{}, down_proj{};
        gate_up.w[0] = w1;
        gate_up.w[1] = w3;
        down_proj.w[0] = w2;
        gate_up.counters = down_proj.counters = counters;
        int rc = launch_gemv_stream(up, x, token_idx, M, gate_up, fp.up, st);
        if (rc != HQM_OK) return rc;
        rc = launch_finalize_silu_mul(h, up, M, fp.up, st);
        if (rc != HQM_OK) return rc;
        rc = launch_gemv_stream(down, h, nullptr, M, down_proj, fp.down, st);
        if (rc != HQM_OK) return rc;
        return launch_finalize_scatter(out, down, token_idx, route_w, accumulate, M, fp.down, st);
    }
    uint16_t* a = (uint16_t*)p;
    p += align_up((size_t)M * F * 2, 256);
    uint16_t* b = (uint16_t*)p;
    p += align_up((size_t)M * F * 2, 256);
    uint16_t* c = (uint16_t*)p;
    p += align_up((size_t)M * H * 2, 256);
    void* lin = p;
    const size_t lin_bytes = scratch_bytes - (size_t)(p - (uint8_t*)scratch);

    int rc = launch_linear(a, x, token_idx, M, w1, nullptr, counters, lin, lin_bytes, st);
    if (rc != HQM_OK) return rc;
    rc = launch_linear(b, x, token_idx, M, w3, nullptr, counters, lin, lin_bytes, st);
    if (rc != HQM_OK) return rc;
    const int64_t nf = M * F;
    silu_mul_kernel<<<(int)((nf + 255) / 256 > 148 * 8 ? 148 * 8 : (nf + 255) / 256), 256, 0, st>>>(a, b, nf);
    HQM_LAUNCH_CHECK();
    rc = launch_linear(c, a, nullptr, M, w2, nullptr, counters, lin, lin_bytes, st);
    if (rc != HQM_OK) return rc;
    const int64_t nh = M * H;
    scale_scatter_kernel<<<(int)((nh + 255) / 256 > 148 * 8 ? 148 * 8 : (nh + 255) / 256), 256, 0, st>>>(
        out, c, token_idx, route_w, M, H, accumulate);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

// ---- single-token MoE block with every expert resident: the host never learns the routing ----------
// Both experts of the token share every launch: [w1; w3] of expert A and of expert B in one streaming
// launch (4 layers), one silu-mul over both, the two w2 in one launch (2 layers, each reading its own h
// row), one weighted sum.
}  // extern "C"

namespace hqm {
bool moe_decode_plan(int E, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3, MoeDecodePlan* mp) {
    return moe_decode_plan_slots(E, 2, w1, w2, w3, mp);
}
bool moe_decode_plan_slots(int E, int slots, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3,
                           MoeDecodePlan* mp) {
    const hqm_weight* up[4] = {w1, w3, w1, w3};
    const hqm_weight* down[2] = {w2, w2};
    if (slots < 1 || slots > 2) return false;
    if (!same_format(w1, w3) || !gemv_stream_plan(up, 2 * slots, 1, &mp->up) || !gemv_stream_plan(down, slots, 1, &mp->down))
        return false;
    mp->router_bytes = align_up((size_t)(4 + 4 + 2 * E + 1 + 4) * 4, 256);
    mp->up_bytes = align_up(gemv_stream_scratch_bytes(mp->up, 1), 256);
    mp->h_bytes = align_up((size_t)slots * w1->N * 2, 256);
    mp->down_bytes = align_up(gemv_stream_scratch_bytes(mp->down, 1), 256);
    return true;
}
}  // namespace hqm

extern "C" {

size_t hqm_moe_decode_scratch_bytes(int32_t E, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3) {
    if (!w1 || !w2 || !w3 || E < 2) return 0;
    hqm::MoeDecodePlan mp;
    if (!hqm::moe_decode_plan(E, w1, w2, w3, &mp)) return 0;
    return hqm::SCRATCH_HEADER + mp.router_bytes + mp.up_bytes + mp.h_bytes + mp.down_bytes;
}

int hqm_moe_decode(uint16_t* out, uint16_t* router_logits, const uint16_t* x, const uint16_t* gate_w, int32_t E,
                   const void* table, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3,
                   void* scratch, size_t scratch_bytes, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(out && router_logits && x && gate_w && table && w1 && w2 && w3, "moe_decode: null pointer");
    HQM_CHECK_ARG(E >= 2 && E <= 32, "moe_decode: %d experts not supported (2..32)", E);
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(x) & 15u) == 0, "moe_decode: x must be 16-byte aligned");
    MoeDecodePlan mp;
    HQM_CHECK_ARG(moe_decode_plan(E, w1, w2, w3, &mp), "moe_decode: these expert shapes are outside the streaming path");
    const size_t need = SCRATCH_HEADER + mp.router_bytes + mp.up_bytes + mp.h_bytes + mp.down_bytes;
    if (scratch == nullptr || scratch_bytes < need) {
        set_error("moe_decode: scratch of %zu bytes given, %zu needed", scratch_bytes, need);
        return HQM_ERR_SCRATCH;
    }
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "moe_decode: scratch must be 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    // router outputs live at the head of the scratch buffer (behind the library's header)
    uint32_t* counters = (uint32_t*)scratch;
    scratch = (uint8_t*)scratch + SCRATCH_HEADER;
    float* topk_w = (float*)scratch;                    // [2] (+2 pad)
    int32_t* topk_idx = (int32_t*)(topk_w + 4);         // [2] (+2 pad)
    int rc = launch_router_top2(router_logits, topk_w, topk_idx, x, gate_w, 1, w1->K, E, st);
    if (rc != HQM_OK) return rc;
    uint8_t* p = (uint8_t*)scratch + mp.router_bytes;
    float* up = (float*)p;
    uint16_t* h = (uint16_t*)(p + mp.up_bytes);         // [2][F]: one row per chosen expert
    float* down = (float*)(p + mp.up_bytes + mp.h_bytes);
    // the experts are whatever the router wrote to topk_idx[0..1]; their descriptors come from the table
    StreamJob gate_up{}, down_proj{};
    gate_up.table = down_proj.table = static_cast<const StreamEntry*>(table);
    gate_up.counters = down_proj.counters = counters;
    for (int slot = 0; slot < 2; ++slot) {
        gate_up.w[2 * slot] = w1;
        gate_up.w[2 * slot + 1] = w3;
        gate_up.sel[2 * slot] = gate_up.sel[2 * slot + 1] = topk_idx + slot;
        gate_up.which[2 * slot] = 0;
        gate_up.which[2 * slot + 1] = 2;
        down_proj.w[slot] = w2;
        down_proj.sel[slot] = topk_idx + slot;
        down_proj.which[slot] = 1;
        down_proj.xrow[slot] = slot;
    }
    // the down projections may read the router's choice and start on their weights while the silu kernel runs:
    // that kernel releases its successor only after the gate / up launch (and so the router) has completed
    down_proj.sel_settled = 1;
    rc = launch_gemv_stream(up, x, nullptr, 1, gate_up, mp.up, st);
    if (rc != HQM_OK) return rc;
    rc = launch_finalize_silu_mul(h, up, 1, mp.up, st, /*late_trigger=*/true);
    if (rc != HQM_OK) return rc;
    rc = launch_gemv_stream(down, h, nullptr, 1, down_proj, mp.down, st);
    if (rc != HQM_OK) return rc;
    return launch_finalize_scatter(out, down, nullptr, topk_w, /*accumulate=*/0, 1, mp.down, st);
}

}  // extern "C"
