// Top-2 router of the MoE block: gate linear, fp32 softmax, top-2, renormalise
// (SparseMoeWrapper.forward, custom_layers.py:276-282) and, on the device, the
// per-expert token lists that the reference builds with one_hot / where /
// .tolist() (custom_layers.py:290-302).  The only thing the host needs back is
// counts[E] (which experts are active).
#include "common.cuh"

namespace hqm {

// One warp per token.  EMAX bounds the number of experts held in registers.
template <int EMAX>
__global__ void __launch_bounds__(256)
router_logits_top2_kernel(uint16_t* __restrict__ logits_out, float* __restrict__ topk_w, int32_t* __restrict__ topk_idx,
                          const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate_w, int M, int K, int E) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= M) return;
    float acc[EMAX];
#pragma unroll
    for (int e = 0; e < EMAX; ++e) acc[e] = 0.f;
    const uint16_t* xr = x + (int64_t)t * K;
    for (int k = lane; k < K; k += 32) {
        const float xv = bf16_bits_to_float(xr[k]);
#pragma unroll
        for (int e = 0; e < EMAX; ++e)
            if (e < E) acc[e] = fmaf(xv, bf16_bits_to_float(gate_w[(int64_t)e * K + k]), acc[e]);
    }
    // The gate is a linear layer in the activation dtype: its output is rounded
    // before the fp32 softmax sees it.
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
        acc[e] = round_bf16(warp_sum(acc[e]));
        if (e < E) mx = fmaxf(mx, acc[e]);
    }
    if (lane != 0) return;
    float p[EMAX], sum = 0.f;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
        p[e] = (e < E) ? expf(acc[e] - mx) : 0.f;
        sum += p[e];
    }
    int i0 = 0, i1 = -1;
    float p0 = -1.f, p1 = -1.f;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
        if (e < E) {
            const float pe = p[e] / sum;
            logits_out[(int64_t)t * E + e] = float_to_bf16_bits(acc[e]);
            if (pe > p0) { p1 = p0; i1 = i0; p0 = pe; i0 = e; }
            else if (pe > p1) { p1 = pe; i1 = e; }
        }
    }
    if (i1 < 0) { i1 = i0; p1 = 0.f; }   // E == 1
    const float norm = p0 + p1;
    topk_w[2 * t] = round_bf16(p0 / norm);
    topk_w[2 * t + 1] = round_bf16(p1 / norm);
    topk_idx[2 * t] = i0;
    topk_idx[2 * t + 1] = i1;
}

// One CTA, one warp per expert: count, exclusive scan, then a stable (token
// ascending) list of the rows routed to each expert with their weights.
__global__ void router_lists_kernel(int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                    int32_t* __restrict__ token_idx, float* __restrict__ token_w,
                                    const float* __restrict__ topk_w, const int32_t* __restrict__ topk_idx, int M,
                                    int E) {
    __shared__ int s_count[32];
    __shared__ int s_off[33];
    const int lane = threadIdx.x & 31, e = threadIdx.x >> 5;
    int cnt = 0;
    for (int t0 = 0; t0 < M; t0 += 32) {
        const int t = t0 + lane;
        const bool hit = t < M && (topk_idx[2 * t] == e || topk_idx[2 * t + 1] == e);
        cnt += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) s_count[e] = cnt;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < E; ++i) {
            s_off[i] = run;
            offsets[i] = run;
            counts[i] = s_count[i];
            run += s_count[i];
        }
        s_off[E] = run;
        offsets[E] = run;
    }
    __syncthreads();
    int base = s_off[e];
    for (int t0 = 0; t0 < M; t0 += 32) {
        const int t = t0 + lane;
        int slot = -1;
        if (t < M) {
            if (topk_idx[2 * t] == e) slot = 0;
            else if (topk_idx[2 * t + 1] == e) slot = 1;
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, slot >= 0);
        if (slot >= 0) {
            const int pos = base + __popc(ballot & ((1u << lane) - 1u));
            token_idx[pos] = t;
            token_w[pos] = topk_w[2 * t + slot];
        }
        base += __popc(ballot);
    }
}

}  // namespace hqm

extern "C" int hqm_router_top2(uint16_t* router_logits, float* topk_w, int32_t* topk_idx, int32_t* counts,
                               int32_t* offsets, int32_t* token_idx, float* token_w, const uint16_t* x,
                               const uint16_t* gate_w, int64_t M, int64_t K, int32_t E, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(E >= 1 && E <= 32, "router: %d experts not supported (1..32)", E);
    HQM_CHECK_ARG(M >= 0 && M <= (1 << 24) && K > 0 && K <= INT32_MAX, "router: bad shape (%lld, %lld)", (long long)M,
                  (long long)K);
    HQM_CHECK_ARG(counts && offsets, "router: null counts/offsets");
    cudaStream_t st = (cudaStream_t)stream;
    if (M > 0) {
        HQM_CHECK_ARG(router_logits && topk_w && topk_idx && token_idx && token_w && x && gate_w,
                      "router: null pointer");
        const int blocks = (int)((M + 7) / 8);
        if (E <= 8)
            router_logits_top2_kernel<8><<<blocks, 256, 0, st>>>(router_logits, topk_w, topk_idx, x, gate_w, (int)M,
                                                                  (int)K, E);
        else
            router_logits_top2_kernel<32><<<blocks, 256, 0, st>>>(router_logits, topk_w, topk_idx, x, gate_w, (int)M,
                                                                   (int)K, E);
        HQM_LAUNCH_CHECK();
    }
    router_lists_kernel<<<1, 32 * E, 0, st>>>(counts, offsets, token_idx, token_w, topk_w, topk_idx, (int)M, E);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}
