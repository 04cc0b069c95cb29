// Top-2 router of the MoE block: gate linear, fp32 softmax, top-2, renormalise
// (SparseMoeWrapper.forward, custom_layers.py:276-282) and, on the device, the
// per-expert token lists that the reference builds with one_hot / where /
// .tolist() (custom_layers.py:290-302).  The only thing the host needs back is
// counts[E] (which experts are active).
#include <cooperative_groups.h>

#include "common.cuh"

namespace hqm {

namespace cg = cooperative_groups;

// A cluster of ROUTER_CTAS CTAs per token: the hidden dimension is dealt to the cluster's threads in 16-byte
// pieces (8 columns of x against the same 8 columns of every expert's gate row: all loads of a thread are
// independent), the E dot products are reduced per CTA in shared memory and across the cluster through
// distributed shared memory, and the first CTA's thread 0 finishes softmax / top-2.  EMAX bounds the
// experts held in registers.
constexpr int ROUTER_CTAS = 8;

template <int EMAX>
__global__ void __launch_bounds__(256)
router_logits_top2_kernel(uint16_t* __restrict__ logits_out, float* __restrict__ topk_w, int32_t* __restrict__ topk_idx,
                          const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate_w, int M, int K, int E) {
    __shared__ float s_part[8][EMAX];
    __shared__ float s_cta[EMAX];
    cg::cluster_group cluster = cg::this_cluster();
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int t = blockIdx.x / ROUTER_CTAS, part = blockIdx.x % ROUTER_CTAS;
    const int tid = part * 256 + threadIdx.x;                 // thread within the cluster
    float acc[EMAX];
#pragma unroll
    for (int e = 0; e < EMAX; ++e) acc[e] = 0.f;
    const uint16_t* xr = x + (int64_t)t * K;
    const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(gate_w)) & 15u) == 0;
    if (vec) {
        for (int k = 8 * tid; k < K; k += 8 * 256 * ROUTER_CTAS) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xr + k);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int e0 = 0; e0 < EMAX; e0 += 8) {           // eight gate rows in flight at a time
                uint4 gv[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    gv[e] = (e0 + e < E) ? *reinterpret_cast<const uint4*>(gate_w + (int64_t)(e0 + e) * K + k)
                                         : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t gw[4] = {gv[e].x, gv[e].y, gv[e].z, gv[e].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[e0 + e] = fmaf(__uint_as_float(xw[j] << 16), __uint_as_float(gw[j] << 16), acc[e0 + e]);
                        acc[e0 + e] = fmaf(__uint_as_float(xw[j] & 0xffff0000u), __uint_as_float(gw[j] & 0xffff0000u),
                                           acc[e0 + e]);
                    }
                }
            }
        }
    } else {
        for (int k = tid; k < K; k += 256 * ROUTER_CTAS) {
            const float xv = bf16_bits_to_float(xr[k]);
#pragma unroll
            for (int e = 0; e < EMAX; ++e)
                if (e < E) acc[e] = fmaf(xv, bf16_bits_to_float(gate_w[(int64_t)e * K + k]), acc[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
        const float v = warp_sum(acc[e]);
        if (lane == 0) s_part[wi][e] = v;
    }
    __syncthreads();
    if (threadIdx.x < EMAX) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += s_part[w][threadIdx.x];
        s_cta[threadIdx.x] = v;
    }
    cluster.sync();
    if (part == 0 && threadIdx.x == 0) {
        // The gate is a linear layer in the activation dtype: its output is rounded
        // before the fp32 softmax sees it.
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < EMAX; ++e) {
            float v = 0.f;
#pragma unroll
            for (int r = 0; r < ROUTER_CTAS; ++r) v += cluster.map_shared_rank(s_cta, r)[e];
            acc[e] = round_bf16(v);
            if (e < E) mx = fmaxf(mx, acc[e]);
        }
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
    cluster.sync();                                     // nobody leaves while its shared memory may still be read
}

// One CTA, one warp per expert: count, exclusive scan, then a stable (token
// ascending) list of the rows routed to each expert with their weights.
__global__ void router_lists_kernel(int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                    int32_t* __restrict__ token_idx, float* __restrict__ token_w,
                                    const float* __restrict__ topk_w, const int32_t* __restrict__ topk_idx, int M,
                                    int E) {
    __shared__ int s_count[32];
    __shared__ int s_off[33];
    grid_launch_dependents();
    grid_dependency_wait();
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

namespace hqm {
// Logits, top-2 indices and weights only (no per-expert lists): what the single-token MoE block needs.
int launch_router_top2(uint16_t* router_logits, float* topk_w, int32_t* topk_idx, const uint16_t* x,
                       const uint16_t* gate_w, int64_t M, int64_t K, int32_t E, cudaStream_t st) {
    if (E <= 8)
        launch_overlapped_cluster(router_logits_top2_kernel<8>, (int)M * ROUTER_CTAS, 256, 0, ROUTER_CTAS, st,
                                  router_logits, topk_w, topk_idx, x, gate_w, (int)M, (int)K, (int)E);
    else
        launch_overlapped_cluster(router_logits_top2_kernel<32>, (int)M * ROUTER_CTAS, 256, 0, ROUTER_CTAS, st,
                                  router_logits, topk_w, topk_idx, x, gate_w, (int)M, (int)K, (int)E);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
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
        const int rc = launch_router_top2(router_logits, topk_w, topk_idx, x, gate_w, M, K, E, st);
        if (rc != HQM_OK) return rc;
    }
    launch_overlapped(router_lists_kernel, 1, 32 * E, 0, st, counts, offsets, token_idx, token_w, (const float*)topk_w,
                      (const int32_t*)topk_idx, (int)M, (int)E);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}
