// The attention half of a decoder layer for ONE new token (batch 1 decode), as a fixed sequence of
// launches with no host involvement:
//
//     h += delta                      (the previous block's output, optional)
//     x  = rmsnorm(h) * ln_in
//     q, k, v = quantized projections of x      one streaming launch, three layers
//     q, k = rope(q, k, pos);  k_cache[pos] = k;  v_cache[pos] = v
//     ctx = softmax(q K^T / sqrt(d)) V          over positions 0..pos, grouped-query heads
//     h += o_proj(ctx)                          streaming launch
//     x_out = rmsnorm(h) * ln_post              the MoE block's input
//
// In the reference these steps are the Hugging Face Mixtral decoder layer around the MoE block that
// build_model.py patches (build_model.py:166-241 builds the model, the four projections are
// HQQLinearTritonSavable modules, custom_layers.py:49-92); here they are the step either side of the
// MoE block so that a whole decode step is a replayable launch sequence.  Arithmetic follows the
// Hugging Face implementation: RMSNorm in fp32 with the product by the weight in bf16, rotate-half
// RoPE with bf16 cos / sin, fp32 softmax, bf16 residual adds.
#include <cooperative_groups.h>
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"
#include "stream_split.cuh"

namespace hqm {

namespace cg = cooperative_groups;

constexpr int HEAD_DIM = 128;

// ---- RMSNorm over a thread-block cluster -----------------------------------------------------------
// The hidden vector is split over NORM_CTAS CTAs of one cluster; the sum of squares is exchanged through
// distributed shared memory (each CTA publishes its part, reads everybody's after a cluster barrier).
constexpr int NORM_CTAS = 8;
constexpr int NORM_THREADS = 512;
constexpr int NORM_PER_THREAD = 4;          // hidden <= 8 * 512 * 4

__device__ __forceinline__ float cluster_sum(float v, float* red, float* mine) {
    cg::cluster_group cluster = cg::this_cluster();
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    if (lane == 0) red[wi] = v;
    __syncthreads();
    if (wi == 0) {
        float t = (lane < NORM_THREADS / 32) ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) *mine = t;
    }
    cluster.sync();                                   // every CTA's part is published
    float total = 0.f;
#pragma unroll
    for (int r = 0; r < NORM_CTAS; ++r) total += *cluster.map_shared_rank(mine, r);
    cluster.sync();                                   // nobody leaves while its shared memory may still be read
    return total;
}

// h = bf16(h + delta) (if delta), x = bf16(w * bf16(h * rsqrt(mean(h^2) + eps))).  One cluster.
__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_kernel(uint16_t* __restrict__ h,
                                                                   const uint16_t* __restrict__ delta,
                                                                   const uint16_t* __restrict__ w,
                                                                   uint16_t* __restrict__ x, int H, float eps) {
    __shared__ float red[32];
    __shared__ float mine;
    grid_launch_dependents();
    grid_dependency_wait();
    const int stride = NORM_CTAS * NORM_THREADS, first = blockIdx.x * NORM_THREADS + threadIdx.x;
    float v[NORM_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        v[j] = 0.f;
        if (i < H) {
            v[j] = bf16_bits_to_float(h[i]);
            if (delta) {
                v[j] = round_bf16(v[j] + bf16_bits_to_float(delta[i]));
                h[i] = float_to_bf16_bits(v[j]);
            }
        }
        ss += v[j] * v[j];
    }
    const float rstd = rsqrtf(cluster_sum(ss, red, &mine) / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        if (i < H) x[i] = float_to_bf16_bits(bf16_bits_to_float(w[i]) * round_bf16(v[j] * rstd));
    }
}

// h = bf16(h + bf16(o-projection sums)), x = rmsnorm(h) * w.  One cluster; the sums are the partial row-sets
// of a streaming launch.
__global__ void __launch_bounds__(NORM_THREADS) finalize_add_rmsnorm_kernel(uint16_t* __restrict__ h,
                                                                            const float* __restrict__ partial,
                                                                            const uint16_t* __restrict__ w,
                                                                            uint16_t* __restrict__ x, int H, float eps,
                                                                            Split sp, ColMap cm) {
    __shared__ float red[32];
    __shared__ float mine;
    grid_launch_dependents();
    grid_dependency_wait();
    const int stride = NORM_CTAS * NORM_THREADS, first = blockIdx.x * NORM_THREADS + threadIdx.x;
    float v[NORM_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        v[j] = 0.f;
        if (i < H) {
            const float y = round_bf16(partial_sum(partial, sp, cm, 0, i, H, H));
            v[j] = round_bf16(bf16_bits_to_float(h[i]) + y);
            h[i] = float_to_bf16_bits(v[j]);
        }
        ss += v[j] * v[j];
    }
    const float rstd = rsqrtf(cluster_sum(ss, red, &mine) / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        if (i < H) x[i] = float_to_bf16_bits(bf16_bits_to_float(w[i]) * round_bf16(v[j] * rstd));
    }
}

// One CTA of 64 threads per head of the [q | k | v] partial row: sums the partials, rounds to bf16 (the
// projection's output), rotates q and k by the position's angles and writes q to `qbuf`, k and v to the
// caches at `pos`.  A position outside the cache sets the error flag and writes nothing.
__global__ void __launch_bounds__(64) finalize_qkv_rope_kernel(uint16_t* __restrict__ qbuf, uint16_t* __restrict__ k_cache,
                                                               uint16_t* __restrict__ v_cache,
                                                               const float* __restrict__ partial,
                                                               const int32_t* __restrict__ pos_ptr, int n_heads,
                                                               int n_kv, int max_len, float theta, int row, Split sp,
                                                               ColMap cm, int* __restrict__ error_flag) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int head = blockIdx.x, d = threadIdx.x;        // d in [0, 64): pairs (d, d + 64)
    const int pos = pos_ptr[0];
    if (pos < 0 || pos >= max_len) {
        if (d == 0 && head == 0 && error_flag) atomicExch(error_flag, 2);
        return;
    }
    const int col = head * HEAD_DIM + d;                 // q heads, then k heads, then v heads: the row's order
    const float a = round_bf16(partial_sum(partial, sp, cm, 0, col, row, row));
    const float b = round_bf16(partial_sum(partial, sp, cm, 0, col + HEAD_DIM / 2, row, row));
    float o0 = a, o1 = b;
    if (head < n_heads + n_kv) {
        const float inv_freq = powf(theta, -(float)(2 * d) / (float)HEAD_DIM);
        float sn, cs;
        sincosf((float)pos * inv_freq, &sn, &cs);
        sn = round_bf16(sn);
        cs = round_bf16(cs);
        o0 = round_bf16(round_bf16(a * cs) + round_bf16(-b * sn));
        o1 = round_bf16(round_bf16(b * cs) + round_bf16(a * sn));
    }
    uint16_t* dst;
    if (head < n_heads) dst = qbuf + head * HEAD_DIM;
    else if (head < n_heads + n_kv) dst = k_cache + ((int64_t)(head - n_heads) * max_len + pos) * HEAD_DIM;
    else dst = v_cache + ((int64_t)(head - n_heads - n_kv) * max_len + pos) * HEAD_DIM;
    dst[d] = float_to_bf16_bits(o0);
    dst[d + HEAD_DIM / 2] = float_to_bf16_bits(o1);
}

// A cluster of ATTN_SPLIT CTAs per query head, 8 warps each; the cached positions are dealt round-robin to
// the cluster's 8 * ATTN_SPLIT warps, eight at a time per warp: lane l holds 4 of the 128 dimensions, a
// score is a warp reduction, the running (max, sum, weighted V) are kept per warp, merged per CTA in shared
// memory, and the CTAs' results are merged by the cluster's first CTA through distributed shared memory.
constexpr int ATTN_SPLIT = 4;

__global__ void __launch_bounds__(256) attn_decode_kernel(uint16_t* __restrict__ ctx, const uint16_t* __restrict__ qbuf,
                                                          const uint16_t* __restrict__ k_cache,
                                                          const uint16_t* __restrict__ v_cache,
                                                          const int32_t* __restrict__ pos_ptr, int group, int max_len) {
    __shared__ float s_m[8], s_l[8];
    __shared__ float s_acc[8][HEAD_DIM];
    __shared__ float c_m, c_l;                          // this CTA's merged state, read by the cluster's first CTA
    __shared__ float c_acc[HEAD_DIM];
    cg::cluster_group cluster = cg::this_cluster();
    grid_launch_dependents();
    grid_dependency_wait();
    const int head = blockIdx.x / ATTN_SPLIT, part = blockIdx.x % ATTN_SPLIT;
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int len = min(max(pos_ptr[0] + 1, 0), max_len);
    const int kvh = head / group;
    const uint16_t* K = k_cache + (int64_t)kvh * max_len * HEAD_DIM + 4 * lane;
    const uint16_t* V = v_cache + (int64_t)kvh * max_len * HEAD_DIM + 4 * lane;
    const float scale = rsqrtf((float)HEAD_DIM);
    float q[4];
    {
        const uint2 qv = *reinterpret_cast<const uint2*>(qbuf + head * HEAD_DIM + 4 * lane);
        q[0] = __uint_as_float(qv.x << 16) * scale;
        q[1] = __uint_as_float(qv.x & 0xffff0000u) * scale;
        q[2] = __uint_as_float(qv.y << 16) * scale;
        q[3] = __uint_as_float(qv.y & 0xffff0000u) * scale;
    }
    constexpr int WARPS = 8 * ATTN_SPLIT;               // warps sharing the head
    float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    constexpr int U = 8;                                // positions per warp and iteration
    for (int j0 = part * 8 + wi; j0 < len; j0 += U * WARPS) {
        float s[U];
        uint2 vv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = j0 + WARPS * u;
            const bool ok = j < len;
            const uint2 kv = ok ? *reinterpret_cast<const uint2*>(K + (int64_t)j * HEAD_DIM) : make_uint2(0u, 0u);
            vv[u] = ok ? *reinterpret_cast<const uint2*>(V + (int64_t)j * HEAD_DIM) : make_uint2(0u, 0u);
            s[u] = q[0] * __uint_as_float(kv.x << 16) + q[1] * __uint_as_float(kv.x & 0xffff0000u) +
                   q[2] * __uint_as_float(kv.y << 16) + q[3] * __uint_as_float(kv.y & 0xffff0000u);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < U; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
        }
        float m_new = m;
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (j0 + WARPS * u < len) m_new = fmaxf(m_new, s[u]);
        const float corr = __expf(m - m_new);           // 0 on the first chunk (m = -inf)
        l *= corr;
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[c] *= corr;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (j0 + WARPS * u < len) {
                const float p = __expf(s[u] - m_new);
                l += p;
                acc[0] += p * __uint_as_float(vv[u].x << 16);
                acc[1] += p * __uint_as_float(vv[u].x & 0xffff0000u);
                acc[2] += p * __uint_as_float(vv[u].y << 16);
                acc[3] += p * __uint_as_float(vv[u].y & 0xffff0000u);
            }
        }
        m = m_new;
    }
    if (lane == 0) {
        s_m[wi] = m;
        s_l[wi] = l;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) s_acc[wi][4 * lane + c] = acc[c];
    __syncthreads();
    if (threadIdx.x < HEAD_DIM) {                       // merge the CTA's 8 warps
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 8; ++w) mm = fmaxf(mm, s_m[w]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float f = (s_m[w] == -INFINITY) ? 0.f : __expf(s_m[w] - mm);
            num += f * s_acc[w][threadIdx.x];
            den += f * s_l[w];
        }
        c_acc[threadIdx.x] = num;
        if (threadIdx.x == 0) {
            c_m = mm;
            c_l = den;
        }
    }
    cluster.sync();
    if (part == 0 && threadIdx.x < HEAD_DIM) {          // merge the cluster's CTAs
        float pm[ATTN_SPLIT], mm = -INFINITY;
#pragma unroll
        for (int r = 0; r < ATTN_SPLIT; ++r) {
            pm[r] = *cluster.map_shared_rank(&c_m, r);
            mm = fmaxf(mm, pm[r]);
        }
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int r = 0; r < ATTN_SPLIT; ++r) {
            const float f = (pm[r] == -INFINITY) ? 0.f : __expf(pm[r] - mm);
            num += f * cluster.map_shared_rank(c_acc, r)[threadIdx.x];
            den += f * *cluster.map_shared_rank(&c_l, r);
        }
        ctx[head * HEAD_DIM + threadIdx.x] = float_to_bf16_bits(den > 0.f ? num / den : 0.f);
    }
    cluster.sync();                                     // nobody leaves while its shared memory may still be read
}

struct AttnPlan {
    StreamPlan qkv, o;
    size_t x_bytes, qkv_bytes, q_bytes, ctx_bytes, o_bytes;
    size_t total() const { return x_bytes + qkv_bytes + q_bytes + ctx_bytes + o_bytes; }
};
static inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

static int attn_plan(const hqm_attn_layer* L, AttnPlan* ap) {
    HQM_CHECK_ARG(L != nullptr, "attn_decode: null layer");
    HQM_CHECK_ARG(L->head_dim == HEAD_DIM, "attn_decode: head_dim = %d isn't supported (128)", L->head_dim);
    HQM_CHECK_ARG(L->n_heads > 0 && L->n_kv_heads > 0 && L->n_heads % L->n_kv_heads == 0,
                  "attn_decode: %d query heads do not group over %d key/value heads", L->n_heads, L->n_kv_heads);
    const int hidden = L->q.K;
    HQM_CHECK_ARG(L->q.N == L->n_heads * HEAD_DIM && L->k.N == L->n_kv_heads * HEAD_DIM && L->v.N == L->k.N &&
                      L->k.K == hidden && L->v.K == hidden && L->o.K == L->q.N && L->o.N == hidden,
                  "attn_decode: projection shapes do not fit %d heads / %d key-value heads of %d", L->n_heads,
                  L->n_kv_heads, HEAD_DIM);
    HQM_CHECK_ARG(hidden <= NORM_CTAS * NORM_THREADS * NORM_PER_THREAD, "attn_decode: hidden size %d too large", hidden);
    HQM_CHECK_ARG(L->max_len > 0 && L->k_cache && L->v_cache && L->ln_in && L->ln_post, "attn_decode: null tensor");
    const hqm_weight* qkv[3] = {&L->q, &L->k, &L->v};
    const hqm_weight* o[1] = {&L->o};
    HQM_CHECK_ARG(gemv_stream_plan(qkv, 3, 1, &ap->qkv) && gemv_stream_plan(o, 1, 1, &ap->o),
                  "attn_decode: these projections are outside the streaming path");
    ap->x_bytes = up256((size_t)hidden * 2);
    ap->qkv_bytes = up256(gemv_stream_scratch_bytes(ap->qkv, 1));
    ap->q_bytes = up256((size_t)L->q.N * 2);
    ap->ctx_bytes = up256((size_t)L->q.N * 2);
    ap->o_bytes = up256(gemv_stream_scratch_bytes(ap->o, 1));
    return HQM_OK;
}

}  // namespace hqm

extern "C" {

int hqm_add_rmsnorm(uint16_t* h, const uint16_t* delta, const uint16_t* weight, uint16_t* x_out, int32_t hidden,
                    float eps, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(h && weight && x_out && hidden > 0 && hidden <= NORM_CTAS * NORM_THREADS * NORM_PER_THREAD,
                  "add_rmsnorm: null pointer or hidden size %d outside (0, %d]", hidden,
                  NORM_CTAS * NORM_THREADS * NORM_PER_THREAD);
    launch_overlapped_cluster(add_rmsnorm_kernel, NORM_CTAS, NORM_THREADS, 0, NORM_CTAS, (cudaStream_t)stream, h, delta,
                              weight, x_out, (int)hidden, eps);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

size_t hqm_attn_decode_scratch_bytes(const hqm_attn_layer* L) {
    hqm::AttnPlan ap;
    if (hqm::attn_plan(L, &ap) != HQM_OK) return 0;
    return ap.total();
}

int hqm_attn_decode(uint16_t* h, uint16_t* x_out, const uint16_t* delta, const hqm_attn_layer* L, const int32_t* pos,
                    void* scratch, size_t scratch_bytes, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(h && x_out && pos, "attn_decode: null pointer");
    AttnPlan ap;
    int rc = attn_plan(L, &ap);
    if (rc != HQM_OK) return rc;
    if (scratch == nullptr || scratch_bytes < ap.total()) {
        set_error("attn_decode: scratch of %zu bytes given, %zu needed", scratch_bytes, ap.total());
        return HQM_ERR_SCRATCH;
    }
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "attn_decode: scratch must be 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int hidden = L->q.K;
    uint8_t* p = (uint8_t*)scratch;
    uint16_t* x = (uint16_t*)p;
    float* qkv_part = (float*)(p + ap.x_bytes);
    uint16_t* qbuf = (uint16_t*)(p + ap.x_bytes + ap.qkv_bytes);
    uint16_t* ctx = (uint16_t*)(p + ap.x_bytes + ap.qkv_bytes + ap.q_bytes);
    float* o_part = (float*)(p + ap.x_bytes + ap.qkv_bytes + ap.q_bytes + ap.ctx_bytes);

    launch_overlapped_cluster(add_rmsnorm_kernel, NORM_CTAS, NORM_THREADS, 0, NORM_CTAS, st, h, delta, L->ln_in, x, hidden,
                              L->rms_eps);
    HQM_LAUNCH_CHECK();
    StreamJob qkv{}, oj{};
    qkv.w[0] = &L->q;
    qkv.w[1] = &L->k;
    qkv.w[2] = &L->v;
    oj.w[0] = &L->o;
    rc = launch_gemv_stream(qkv_part, x, nullptr, 1, qkv, ap.qkv, st);
    if (rc != HQM_OK) return rc;
    const int heads = L->n_heads + 2 * L->n_kv_heads;
    launch_overlapped(finalize_qkv_rope_kernel, heads, 64, 0, st, qbuf, L->k_cache, L->v_cache,
                      (const float*)qkv_part, pos, (int)L->n_heads, (int)L->n_kv_heads, (int)L->max_len, L->rope_theta,
                      ap.qkv.col0[3], split_of(ap.qkv), colmap_of(ap.qkv), tc_error_ptr());
    HQM_LAUNCH_CHECK();
    launch_overlapped_cluster(attn_decode_kernel, (int)L->n_heads * ATTN_SPLIT, 256, 0, ATTN_SPLIT, st, ctx, (const uint16_t*)qbuf,
                      (const uint16_t*)L->k_cache, (const uint16_t*)L->v_cache, pos, (int)(L->n_heads / L->n_kv_heads),
                      (int)L->max_len);
    HQM_LAUNCH_CHECK();
    rc = launch_gemv_stream(o_part, ctx, nullptr, 1, oj, ap.o, st);
    if (rc != HQM_OK) return rc;
    launch_overlapped_cluster(finalize_add_rmsnorm_kernel, NORM_CTAS, NORM_THREADS, 0, NORM_CTAS, st, h,
                              (const float*)o_part, L->ln_post, x_out, hidden, L->rms_eps, split_of(ap.o),
                              colmap_of(ap.o));
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

}  // extern "C"
