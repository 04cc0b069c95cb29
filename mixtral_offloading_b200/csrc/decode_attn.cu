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

// The same for many rows (a prompt, a batch of sequences): one CTA per row of h (rows, H), two passes over the row
// (the second re-reads the bf16 values the first one wrote or left in place).
__global__ void __launch_bounds__(256) add_rmsnorm_rows_kernel(uint16_t* __restrict__ h, const uint16_t* __restrict__ delta,
                                                               const uint16_t* __restrict__ w, uint16_t* __restrict__ x,
                                                               int H, float eps) {
    __shared__ float red[8];
    __shared__ float s_rstd;
    uint16_t* hr = h + (int64_t)blockIdx.x * H;
    const uint16_t* dr = delta ? delta + (int64_t)blockIdx.x * H : nullptr;
    uint16_t* xr = x + (int64_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = bf16_bits_to_float(hr[i]);
        if (dr) {
            v = round_bf16(v + bf16_bits_to_float(dr[i]));
            hr[i] = float_to_bf16_bits(v);
        }
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) s_rstd = rsqrtf(t / (float)H + eps);
    }
    __syncthreads();
    const float rstd = s_rstd;
    for (int i = threadIdx.x; i < H; i += 256)
        xr[i] = float_to_bf16_bits(bf16_bits_to_float(w[i]) * round_bf16(bf16_bits_to_float(hr[i]) * rstd));
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
            const float y = round_bf16(partial_sum<true>(partial, sp, cm, 0, i, H, H));
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

// finalize_add_rmsnorm_kernel followed by the top-2 router on its result, in one launch: every thread multiplies
// the x values it holds with the E gate rows, the E dot products are reduced over the cluster like the sum of
// squares, and the first CTA finishes softmax / top-2 exactly as router_logits_top2_kernel does.  E <= 8.
constexpr int ROUTER_EMAX = 8;
__global__ void __launch_bounds__(NORM_THREADS) finalize_add_rmsnorm_router_kernel(
    uint16_t* __restrict__ h, const float* __restrict__ partial, const uint16_t* __restrict__ w, uint16_t* __restrict__ x,
    int H, float eps, Split sp, ColMap cm, const uint16_t* __restrict__ gate_w, int E, uint16_t* __restrict__ logits_out,
    float* __restrict__ topk_w, int32_t* __restrict__ topk_idx, int ep_lo, int ep_n, int ep_slots,
    float* __restrict__ local_w, int32_t* __restrict__ local_idx) {
    __shared__ float red[32];
    __shared__ float mine;
    __shared__ float s_part[NORM_THREADS / 32][ROUTER_EMAX];
    __shared__ float s_cta[ROUTER_EMAX];
    cg::cluster_group cluster = cg::this_cluster();
    grid_launch_dependents();
    const int stride = NORM_CTAS * NORM_THREADS, first = blockIdx.x * NORM_THREADS + threadIdx.x;
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    // the norm weight and the gate rows of this thread's columns are weights: they are fetched while the launch in
    // front is still finishing
    uint16_t wv[NORM_PER_THREAD], gv[NORM_PER_THREAD][ROUTER_EMAX];
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        wv[j] = 0;
#pragma unroll
        for (int e = 0; e < ROUTER_EMAX; ++e) gv[j][e] = 0;
        if (i < H) {
            wv[j] = w[i];
#pragma unroll
            for (int e = 0; e < ROUTER_EMAX; ++e)
                if (e < E) gv[j][e] = gate_w[(int64_t)e * H + i];
        }
    }
    grid_dependency_wait();
    float v[NORM_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        v[j] = 0.f;
        if (i < H) {
            const float y = round_bf16(partial_sum<true>(partial, sp, cm, 0, i, H, H));
            v[j] = round_bf16(bf16_bits_to_float(h[i]) + y);
            h[i] = float_to_bf16_bits(v[j]);
        }
        ss += v[j] * v[j];
    }
    const float rstd = rsqrtf(cluster_sum(ss, red, &mine) / (float)H + eps);
    float acc[ROUTER_EMAX];
#pragma unroll
    for (int e = 0; e < ROUTER_EMAX; ++e) acc[e] = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        if (i < H) {
            const uint16_t xb = float_to_bf16_bits(bf16_bits_to_float(wv[j]) * round_bf16(v[j] * rstd));
            x[i] = xb;
            const float xv = bf16_bits_to_float(xb);
#pragma unroll
            for (int e = 0; e < ROUTER_EMAX; ++e) acc[e] = fmaf(xv, bf16_bits_to_float(gv[j][e]), acc[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < ROUTER_EMAX; ++e) {
        const float t = warp_sum(acc[e]);
        if (lane == 0) s_part[wi][e] = t;
    }
    __syncthreads();
    if (threadIdx.x < ROUTER_EMAX) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < NORM_THREADS / 32; ++q) t += s_part[q][threadIdx.x];
        s_cta[threadIdx.x] = t;
    }
    cluster.sync();
    if (blockIdx.x == 0 && wi == 0) {
        // lane e adds expert e's dot product over the cluster's CTAs (in rank order, as one thread would); every
        // lane then holds all E logits and runs the same softmax / top-2
        float mine_e = 0.f;
        if (lane < ROUTER_EMAX) {
#pragma unroll
            for (int r = 0; r < NORM_CTAS; ++r) mine_e += cluster.map_shared_rank(s_cta, r)[lane];
            mine_e = round_bf16(mine_e);                // the gate's output in the activation dtype
        }
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < ROUTER_EMAX; ++e) {
            acc[e] = __shfl_sync(0xffffffffu, mine_e, e);
            if (e < E) mx = fmaxf(mx, acc[e]);
        }
        float p[ROUTER_EMAX], sum = 0.f;
#pragma unroll
        for (int e = 0; e < ROUTER_EMAX; ++e) {
            p[e] = (e < E) ? expf(acc[e] - mx) : 0.f;
            sum += p[e];
        }
        int i0 = 0, i1 = -1;
        float p0 = -1.f, p1 = -1.f;
#pragma unroll
        for (int e = 0; e < ROUTER_EMAX; ++e) {
            if (e < E) {
                const float pe = p[e] / sum;
                if (pe > p0) { p1 = p0; i1 = i0; p0 = pe; i0 = e; }
                else if (pe > p1) { p1 = pe; i1 = e; }
            }
        }
        if (lane < E) logits_out[lane] = float_to_bf16_bits(mine_e);
        if (i1 < 0) { i1 = i0; p1 = 0.f; }
        const float norm = p0 + p1;
        const float w0 = round_bf16(p0 / norm), w1 = round_bf16(p1 / norm);
        if (lane == 0) {
            topk_w[0] = w0;
            topk_w[1] = w1;
            topk_idx[0] = i0;
            topk_idx[1] = i1;
            if (local_idx) {
                // expert-parallel rank owning experts [ep_lo, ep_lo + ep_n): the chosen experts it owns, in the
                // router's order, packed into its `ep_slots` launch slots (index into the rank's own table); -1 =
                // slot unused
                int n = 0;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int e = c == 0 ? i0 : i1;
                    if (e >= ep_lo && e < ep_lo + ep_n && n < ep_slots) {
                        local_idx[n] = e - ep_lo;
                        local_w[n] = c == 0 ? w0 : w1;
                        ++n;
                    }
                }
                for (; n < ep_slots; ++n) {
                    local_idx[n] = -1;
                    local_w[n] = 0.f;
                }
            }
        }
    }
    cluster.sync();
}

// The end of the MoE block and the start of the next layer in one launch: y = sum over the launch's layers l of
// bf16(route_w[l] * bf16(partial sums of layer l)) (bf16 rounding after each add, as finalize_scatter_kernel),
// h = bf16(h + y), x = rmsnorm(h) * w.
__global__ void __launch_bounds__(NORM_THREADS) finalize_scatter_add_rmsnorm_kernel(
    uint16_t* __restrict__ h, const float* __restrict__ partial, const float* __restrict__ route_w,
    const uint16_t* __restrict__ w, uint16_t* __restrict__ x, int H, int row, float eps, Split sp, ColMap cm) {
    __shared__ float red[32];
    __shared__ float mine;
    grid_launch_dependents();
    const int stride = NORM_CTAS * NORM_THREADS, first = blockIdx.x * NORM_THREADS + threadIdx.x;
    uint16_t wv[NORM_PER_THREAD];                 // the norm weight is fetched while the launch in front finishes
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        wv[j] = i < H ? w[i] : (uint16_t)0;
    }
    grid_dependency_wait();
    float v[NORM_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        v[j] = 0.f;
        if (i < H) {
            // the launch holds the token's two experts: both sums are requested together
            float s0, s1;
            partial_sum_pair<true>(partial, sp, cm, 0, cm.col0[0] + i, cm.col0[1] + i, row, row, s0, s1);
            const float y = round_bf16(round_bf16(round_bf16(s0) * route_w[0]) + round_bf16(round_bf16(s1) * route_w[1]));
            v[j] = round_bf16(bf16_bits_to_float(h[i]) + y);
            h[i] = float_to_bf16_bits(v[j]);
        }
        ss += v[j] * v[j];
    }
    const float rstd = rsqrtf(cluster_sum(ss, red, &mine) / (float)H + eps);
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        if (i < H) x[i] = float_to_bf16_bits(bf16_bits_to_float(wv[j]) * round_bf16(v[j] * rstd));
    }
}

// y[i] = sum over the launch's layers l of bf16(route_w[l] * bf16(sums of layer l)), in fp32: what one expert-parallel
// rank contributes to the MoE block's output.  Every term is a bf16 value and at most two ranks' terms are non-zero,
// so adding the ranks' vectors in fp32 and rounding to bf16 gives exactly what finalize_scatter_add_rmsnorm_kernel
// computes on one GPU.
__global__ void __launch_bounds__(256) finalize_weighted_f32_kernel(float* __restrict__ y, const float* __restrict__ partial,
                                                                    const float* __restrict__ route_w, int H, int row,
                                                                    Split sp, ColMap cm) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) {
        float acc = 0.f;
#pragma unroll
        for (int l = 0; l < STREAM_MAX_LAYERS; ++l) {
            if (l < cm.count) {
                const float v = round_bf16(round_bf16(partial_sum<true>(partial, sp, cm, 0, layer_col0(cm, l) + i, row, row)) * route_w[l]);
                acc = (l == 0) ? v : round_bf16(acc + v);
            }
        }
        y[i] = acc;
    }
}

// ---- the expert-parallel exchange over peer memory ---------------------------------------------------
// Every rank keeps a buffer [2][world][hidden] fp32 ("shares": one row per rank, two generations) and flags
// [2][world][EP_MAX_CHUNKS] that its peers write with plain stores over NVLink.  An exchange has a number s
// (1, 2, ...; every rank counts its own in device memory and all ranks make the same calls, so the numbers agree):
// the publish kernel writes this rank's row of generation s & 1 into EVERY rank's buffer, fences, and then stores
// s into the matching flags, one per 256-element chunk; the combine kernel waits until the flags of all ranks for
// the chunks it reads show s, adds the rows in rank order and goes on with the residual add and the norm.  A rank
// cannot publish exchange s + 1 before it has combined s, which needs every peer's share of s, which a peer
// publishes only after combining s - 1: nobody is more than one exchange ahead, so two generations are enough.
// Waits are bounded: when a flag does not arrive the kernel records error 4 and goes on with what is there.
constexpr int EP_CHUNK = 256;
constexpr int EP_MAX_CHUNKS = 64;
constexpr uint32_t EP_SPIN_LIMIT = 1u << 21;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// finalize_weighted_f32_kernel whose result goes to every rank's share buffer instead of local memory.
// One CTA per chunk of EP_CHUNK elements.
__global__ void __launch_bounds__(EP_CHUNK) finalize_weighted_publish_kernel(const float* __restrict__ partial,
                                                                             const float* __restrict__ route_w, int H,
                                                                             int row, Split sp, ColMap cm, hqm_ep_comm comm) {
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t s = *reinterpret_cast<volatile uint32_t*>(comm.seq) + 1u;
    const int gen = (int)(s & 1u);
    const int i = blockIdx.x * EP_CHUNK + threadIdx.x;
    if (i < H) {
        float acc = 0.f;
#pragma unroll
        for (int l = 0; l < STREAM_MAX_LAYERS; ++l) {
            if (l < cm.count) {
                const float v = round_bf16(round_bf16(partial_sum<true>(partial, sp, cm, 0, layer_col0(cm, l) + i, row, row)) * route_w[l]);
                acc = (l == 0) ? v : round_bf16(acc + v);
            }
        }
        const size_t at = ((size_t)gen * comm.world + comm.rank) * (size_t)H + i;
        for (int r = 0; r < comm.world; ++r) comm.shares[r][at] = acc;
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < comm.world)
        st_release_sys(comm.flags[threadIdx.x] + ((size_t)gen * comm.world + comm.rank) * EP_MAX_CHUNKS + blockIdx.x, s);
}

// h = bf16(h + bf16(sum over ranks of their shares of exchange s)), x = rmsnorm(h) * w; closes exchange s.
__global__ void __launch_bounds__(NORM_THREADS) ep_combine_add_rmsnorm_kernel(uint16_t* __restrict__ h,
                                                                              const uint16_t* __restrict__ w,
                                                                              uint16_t* __restrict__ x, int H, float eps,
                                                                              hqm_ep_comm comm, int* __restrict__ error_flag) {
    __shared__ float red[32];
    __shared__ float mine;
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t s = *reinterpret_cast<volatile uint32_t*>(comm.seq) + 1u;
    const int gen = (int)(s & 1u);
    const float* shares = comm.shares[comm.rank] + (size_t)gen * comm.world * H;
    const uint32_t* flags = comm.flags[comm.rank] + (size_t)gen * comm.world * EP_MAX_CHUNKS;
    const int stride = NORM_CTAS * NORM_THREADS, first = blockIdx.x * NORM_THREADS + threadIdx.x;
    float v[NORM_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_PER_THREAD; ++j) {
        const int i = first + j * stride;
        v[j] = 0.f;
        if (i < H) {
            const int chunk = i / EP_CHUNK;
            float sum = 0.f;
            for (int r = 0; r < comm.world; ++r) {
                const uint32_t* f = flags + r * EP_MAX_CHUNKS + chunk;
                uint32_t spins = 0;
                while (ld_acquire_sys(f) != s) {
                    if (++spins > EP_SPIN_LIMIT) {
                        if (error_flag) atomicExch(error_flag, 4);
                        break;
                    }
                    __nanosleep(100);
                }
                sum += __ldcg(shares + (size_t)r * H + i);
            }
            v[j] = round_bf16(bf16_bits_to_float(h[i]) + round_bf16(sum));
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
    if (blockIdx.x == 0 && threadIdx.x == 0) *comm.seq = s;            // every CTA read the counter before cluster_sum's barriers
}

// h = bf16(h + bf16(delta)) with delta in fp32 (the all-reduced expert-parallel partials), x = rmsnorm(h) * w.
__global__ void __launch_bounds__(NORM_THREADS) add_f32_rmsnorm_kernel(uint16_t* __restrict__ h,
                                                                       const float* __restrict__ delta,
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
            v[j] = round_bf16(bf16_bits_to_float(h[i]) + round_bf16(delta[i]));
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
    float a, b;
    partial_sum_pair<true>(partial, sp, cm, 0, col, col + HEAD_DIM / 2, row, row, a, b);
    a = round_bf16(a);
    b = round_bf16(b);
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
//
// FUSED = true folds the step in front into the kernel (one launch less per layer): every CTA sums the
// projection partials of its head's q and of its key/value head's new k and v itself, rotates q and k, keeps
// them in shared memory, and attends to the cached positions 0..pos-1 plus the new position from shared
// memory; one CTA per key/value head also appends k and v to the cache.
constexpr int ATTN_SPLIT = 4;

struct QkvSource {                 // FUSED only: where q, k, v of this token come from
    const float* partial;
    int n_heads, n_kv, row;
    float theta;
    Split sp;
    ColMap cm;
    int* error_flag;
};

// rotate-half RoPE of the pair (a, b) = (t[d], t[d + 64]) at position pos, bf16 arithmetic as Hugging Face does it
__device__ __forceinline__ void rope_pair(float a, float b, int d, int pos, float theta, float& o0, float& o1) {
    const float inv_freq = powf(theta, -(float)(2 * d) / (float)HEAD_DIM);
    float sn, cs;
    sincosf((float)pos * inv_freq, &sn, &cs);
    sn = round_bf16(sn);
    cs = round_bf16(cs);
    o0 = round_bf16(round_bf16(a * cs) + round_bf16(-b * sn));
    o1 = round_bf16(round_bf16(b * cs) + round_bf16(a * sn));
}

// RoPE and cache append for many tokens at once (a prompt: token t at position pos0 + t in ONE cache; a batch of
// sequences: token t at the same position in ITS cache, batch_stride elements further on).  One CTA per token:
// q (T, n_heads, 128) is rotated in place, k rotated and v copied into row `pos` of the key / value caches
// (n_kv, max_len, 128).  A position outside the cache sets the error flag and leaves the token untouched.
__global__ void __launch_bounds__(256) rope_append_rows_kernel(uint16_t* __restrict__ q, const uint16_t* __restrict__ k,
                                                               const uint16_t* __restrict__ v,
                                                               uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache,
                                                               int n_heads, int n_kv, int max_len, int64_t batch_stride,
                                                               const int64_t* __restrict__ pos_ptr, int pos0, int pos_step,
                                                               float theta, int* error_flag) {
    const int t = blockIdx.x;
    const int pos = (pos_ptr ? (int)pos_ptr[0] : pos0) + t * pos_step;
    if (pos < 0 || pos >= max_len) {
        if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
        return;
    }
    constexpr int HALF = HEAD_DIM / 2;
    uint16_t* qt = q + (int64_t)t * n_heads * HEAD_DIM;
    for (int i = threadIdx.x; i < n_heads * HALF; i += 256) {
        const int head = i / HALF, d = i % HALF;
        uint16_t* p = qt + head * HEAD_DIM + d;
        float o0, o1;
        rope_pair(bf16_bits_to_float(p[0]), bf16_bits_to_float(p[HALF]), d, pos, theta, o0, o1);
        p[0] = float_to_bf16_bits(o0);
        p[HALF] = float_to_bf16_bits(o1);
    }
    const uint16_t* kt = k + (int64_t)t * n_kv * HEAD_DIM;
    const uint16_t* vt = v + (int64_t)t * n_kv * HEAD_DIM;
    for (int i = threadIdx.x; i < n_kv * HALF; i += 256) {
        const int head = i / HALF, d = i % HALF;
        const int64_t row = (int64_t)t * batch_stride + ((int64_t)head * max_len + pos) * HEAD_DIM + d;
        float o0, o1;
        rope_pair(bf16_bits_to_float(kt[head * HEAD_DIM + d]), bf16_bits_to_float(kt[head * HEAD_DIM + d + HALF]), d, pos, theta,
                  o0, o1);
        k_cache[row] = float_to_bf16_bits(o0);
        k_cache[row + HALF] = float_to_bf16_bits(o1);
        v_cache[row] = vt[head * HEAD_DIM + d];
        v_cache[row + HALF] = vt[head * HEAD_DIM + d + HALF];
    }
}

template <bool FUSED>
__global__ void __launch_bounds__(256) attn_decode_kernel(uint16_t* __restrict__ ctx, const uint16_t* __restrict__ qbuf,
                                                          uint16_t* __restrict__ k_cache, uint16_t* __restrict__ v_cache,
                                                          const int32_t* __restrict__ pos_ptr, int group, int max_len,
                                                          QkvSource src) {
    __shared__ float s_q[HEAD_DIM], s_kn[HEAD_DIM], s_vn[HEAD_DIM];
    __shared__ float s_m[8], s_l[8];
    __shared__ float s_acc[8][HEAD_DIM];
    __shared__ float c_m, c_l;                          // this CTA's merged state, read by the cluster's first CTA
    __shared__ float c_acc[HEAD_DIM];
    cg::cluster_group cluster = cg::this_cluster();
    grid_launch_dependents();
    const int head = blockIdx.x / ATTN_SPLIT, part = blockIdx.x % ATTN_SPLIT;
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int pos = pos_ptr[0];
    const int kvh = head / group;
    const float scale = rsqrtf((float)HEAD_DIM);
    {
        // The cached rows below `pos` were written by earlier steps and the position is not touched inside a step:
        // this warp's rows are requested into L2 while the launch in front (the q / k / v projections) is still
        // running.  A row is 256 bytes = two 128-byte lines; lane -> (row lane / 2 of each batch of 16, line lane % 2).
        constexpr int WARPS_ALL = 8 * ATTN_SPLIT;
        const int n = min(max(pos, 0), max_len);
        const char* kb = reinterpret_cast<const char*>(k_cache + (int64_t)kvh * max_len * HEAD_DIM);
        const char* vb = reinterpret_cast<const char*>(v_cache + (int64_t)kvh * max_len * HEAD_DIM);
        for (int j = part * 8 + wi + WARPS_ALL * (lane >> 1); j < n; j += WARPS_ALL * 16) {
            const int64_t off = (int64_t)j * (HEAD_DIM * 2) + 128 * (lane & 1);
            asm volatile("prefetch.global.L2 [%0];" ::"l"(kb + off));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(vb + off));
        }
    }
    grid_dependency_wait();
    int len;                                            // positions read from the cache
    bool fresh = false;                                 // the new position is attended to from shared memory
    float q[4];
    if constexpr (FUSED) {
        const bool pos_ok = pos >= 0 && pos < max_len;
        if (!pos_ok && blockIdx.x == 0 && threadIdx.x == 0 && src.error_flag) atomicExch(src.error_flag, 2);
        const int which = threadIdx.x >> 6, d = threadIdx.x & 63;     // 0: q, 1: k, 2: v;  pair (d, d + 64)
        if (which < 3) {
            const int col = (which == 0 ? head : (which == 1 ? src.n_heads + kvh : src.n_heads + src.n_kv + kvh)) * HEAD_DIM + d;
            float a, b;
            partial_sum_pair<true>(src.partial, src.sp, src.cm, 0, col, col + HEAD_DIM / 2, src.row, src.row, a, b);
            a = round_bf16(a);
            b = round_bf16(b);
            float o0 = a, o1 = b;
            if (which < 2) rope_pair(a, b, d, pos, src.theta, o0, o1);
            float* dst = which == 0 ? s_q : (which == 1 ? s_kn : s_vn);
            dst[d] = o0;
            dst[d + HEAD_DIM / 2] = o1;
            if (which > 0 && pos_ok && part == 0 && head % group == 0) {     // one CTA per key/value head appends
                uint16_t* row = (which == 1 ? k_cache : v_cache) + ((int64_t)kvh * max_len + pos) * HEAD_DIM;
                row[d] = float_to_bf16_bits(o0);
                row[d + HEAD_DIM / 2] = float_to_bf16_bits(o1);
            }
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = s_q[4 * lane + c] * scale;
        len = min(max(pos, 0), max_len);
        fresh = pos_ok && part == 0 && wi == 0;
    } else {
        len = min(max(pos + 1, 0), max_len);
        const uint2 qv = *reinterpret_cast<const uint2*>(qbuf + head * HEAD_DIM + 4 * lane);
        q[0] = __uint_as_float(qv.x << 16) * scale;
        q[1] = __uint_as_float(qv.x & 0xffff0000u) * scale;
        q[2] = __uint_as_float(qv.y << 16) * scale;
        q[3] = __uint_as_float(qv.y & 0xffff0000u) * scale;
    }
    const uint16_t* K = k_cache + (int64_t)kvh * max_len * HEAD_DIM + 4 * lane;
    const uint16_t* V = v_cache + (int64_t)kvh * max_len * HEAD_DIM + 4 * lane;
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
    if (fresh) {                                        // the new token's own key and value
        float sc = q[0] * s_kn[4 * lane] + q[1] * s_kn[4 * lane + 1] + q[2] * s_kn[4 * lane + 2] + q[3] * s_kn[4 * lane + 3];
        sc = warp_sum(sc);
        const float m_new = fmaxf(m, sc);
        const float corr = __expf(m - m_new), p = __expf(sc - m_new);
        l = l * corr + p;
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[c] = acc[c] * corr + p * s_vn[4 * lane + c];
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

int hqm_add_rmsnorm_rows(uint16_t* h, const uint16_t* delta, const uint16_t* weight, uint16_t* x_out, int64_t rows,
                         int32_t hidden, float eps, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(rows >= 0 && rows <= INT32_MAX && hidden > 0, "add_rmsnorm_rows: bad shape (%lld, %d)", (long long)rows,
                  hidden);
    if (rows == 0) return HQM_OK;
    HQM_CHECK_ARG(h && weight && x_out, "add_rmsnorm_rows: null pointer");
    add_rmsnorm_rows_kernel<<<(int)rows, 256, 0, (cudaStream_t)stream>>>(h, delta, weight, x_out, (int)hidden, eps);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

int hqm_rope_append_rows(uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* k_cache, uint16_t* v_cache,
                         int64_t tokens, int32_t n_heads, int32_t n_kv_heads, int32_t head_dim, int32_t max_len,
                         int64_t batch_stride, const int64_t* pos_device, int32_t pos0, int32_t pos_step, float rope_theta,
                         void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(tokens >= 0 && tokens <= INT32_MAX, "rope_append_rows: bad token count %lld", (long long)tokens);
    if (tokens == 0) return HQM_OK;
    HQM_CHECK_ARG(q && k && v && k_cache && v_cache, "rope_append_rows: null pointer");
    HQM_CHECK_ARG(head_dim == HEAD_DIM && n_heads > 0 && n_kv_heads > 0 && max_len > 0,
                  "rope_append_rows: head_dim %d (only %d), %d / %d heads, cache of %d", head_dim, HEAD_DIM, n_heads,
                  n_kv_heads, max_len);
    rope_append_rows_kernel<<<(int)tokens, 256, 0, (cudaStream_t)stream>>>(q, k, v, k_cache, v_cache, n_heads, n_kv_heads,
                                                                           max_len, batch_stride, pos_device, pos0,
                                                                           pos_step, rope_theta, tc_error_ptr());
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

size_t hqm_attn_decode_scratch_bytes(const hqm_attn_layer* L) {
    hqm::AttnPlan ap;
    if (hqm::attn_plan(L, &ap) != HQM_OK) return 0;
    return hqm::SCRATCH_HEADER + ap.total();
}

int hqm_attn_decode(uint16_t* h, uint16_t* x_out, const uint16_t* delta, const hqm_attn_layer* L, const int32_t* pos,
                    void* scratch, size_t scratch_bytes, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(h && x_out && pos, "attn_decode: null pointer");
    AttnPlan ap;
    int rc = attn_plan(L, &ap);
    if (rc != HQM_OK) return rc;
    if (scratch == nullptr || scratch_bytes < SCRATCH_HEADER + ap.total()) {
        set_error("attn_decode: scratch of %zu bytes given, %zu needed", scratch_bytes, SCRATCH_HEADER + ap.total());
        return HQM_ERR_SCRATCH;
    }
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "attn_decode: scratch must be 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int hidden = L->q.K;
    uint32_t* counters = (uint32_t*)scratch;
    uint8_t* p = (uint8_t*)scratch + SCRATCH_HEADER;
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
    qkv.counters = oj.counters = counters;
    rc = launch_gemv_stream(qkv_part, x, nullptr, 1, qkv, ap.qkv, st);
    if (rc != HQM_OK) return rc;
    const int heads = L->n_heads + 2 * L->n_kv_heads;
    launch_overlapped(finalize_qkv_rope_kernel, heads, 64, 0, st, qbuf, L->k_cache, L->v_cache,
                      (const float*)qkv_part, pos, (int)L->n_heads, (int)L->n_kv_heads, (int)L->max_len, L->rope_theta,
                      ap.qkv.col0[3], split_of(ap.qkv), colmap_of(ap.qkv), tc_error_ptr());
    HQM_LAUNCH_CHECK();
    launch_overlapped_cluster(attn_decode_kernel<false>, (int)L->n_heads * ATTN_SPLIT, 256, 0, ATTN_SPLIT, st, ctx,
                              (const uint16_t*)qbuf, L->k_cache, L->v_cache, pos, (int)(L->n_heads / L->n_kv_heads),
                              (int)L->max_len, QkvSource{});
    HQM_LAUNCH_CHECK();
    rc = launch_gemv_stream(o_part, ctx, nullptr, 1, oj, ap.o, st);
    if (rc != HQM_OK) return rc;
    launch_overlapped_cluster(finalize_add_rmsnorm_kernel, NORM_CTAS, NORM_THREADS, 0, NORM_CTAS, st, h,
                              (const float*)o_part, L->ln_post, x_out, hidden, L->rms_eps, split_of(ap.o),
                              colmap_of(ap.o));
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

// ---- a whole decoder layer for one token: 8 launches -------------------------------------------------
// `slots` expert launch slots: 2 on one GPU (both routed experts); an expert-parallel rank has min(2, experts it
// owns) and fills them on the device with the routed experts that are its own.
static int decoder_layer_plan(const hqm_decoder_layer* L, int slots, hqm::AttnPlan* ap, hqm::MoeDecodePlan* mp) {
    using namespace hqm;
    HQM_CHECK_ARG(L != nullptr, "decode_layer: null layer");
    int rc = attn_plan(&L->attn, ap);
    if (rc != HQM_OK) return rc;
    HQM_CHECK_ARG(L->gate_w && L->table && L->next_ln, "decode_layer: null tensor");
    HQM_CHECK_ARG(L->n_experts >= 2 && L->n_experts <= ROUTER_EMAX, "decode_layer: %d experts not supported (2..%d)",
                  L->n_experts, ROUTER_EMAX);
    HQM_CHECK_ARG(L->w1.K == L->attn.q.K && L->w2.N == L->attn.q.K, "decode_layer: expert shapes do not fit the hidden size");
    HQM_CHECK_ARG(moe_decode_plan_slots(L->n_experts, slots, &L->w1, &L->w2, &L->w3, mp),
                  "decode_layer: these expert shapes are outside the streaming path");
    return HQM_OK;
}

static size_t decoder_layer_bytes(const hqm::AttnPlan& ap, const hqm::MoeDecodePlan& mp) {
    return hqm::SCRATCH_HEADER + ap.total() + mp.router_bytes + mp.up_bytes + mp.h_bytes + mp.down_bytes;
}

// y_partial == nullptr: one GPU, the layer is finished (residual add, next norm).  Otherwise the rank's fp32
// contribution to the MoE block's output goes to y_partial and h / x are left as they are after the attention half.
static int decode_layer_run(uint16_t* h, uint16_t* x, uint16_t* router_logits, float* y_partial, const hqm_ep_comm* comm,
                            const hqm_decoder_layer* L, int ep_lo, int ep_n, int slots, const int32_t* pos, void* scratch,
                            size_t scratch_bytes, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(h && x && router_logits && pos, "decode_layer: null pointer");
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(x) & 15u) == 0, "decode_layer: x must be 16-byte aligned");
    AttnPlan ap;
    MoeDecodePlan mp;
    int rc = decoder_layer_plan(L, slots, &ap, &mp);
    if (rc != HQM_OK) return rc;
    const size_t need = decoder_layer_bytes(ap, mp);
    if (scratch == nullptr || scratch_bytes < need) {
        set_error("decode_layer: scratch of %zu bytes given, %zu needed", scratch_bytes, need);
        return HQM_ERR_SCRATCH;
    }
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "decode_layer: scratch must be 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const hqm_attn_layer* A = &L->attn;
    const int hidden = A->q.K, E = L->n_experts;
    uint32_t* counters = (uint32_t*)scratch;
    uint8_t* p = (uint8_t*)scratch + SCRATCH_HEADER;
    uint16_t* x2 = (uint16_t*)p;                                   // the MoE block's input
    float* qkv_part = (float*)(p + ap.x_bytes);
    uint16_t* ctx = (uint16_t*)(p + ap.x_bytes + ap.qkv_bytes + ap.q_bytes);
    float* o_part = (float*)(p + ap.x_bytes + ap.qkv_bytes + ap.q_bytes + ap.ctx_bytes);
    uint8_t* m0 = p + ap.total();
    float* topk_w = (float*)m0;                                    // [2] (+2 pad)
    int32_t* topk_idx = (int32_t*)(topk_w + 4);                    // [2] (+2 pad)
    float* local_w = topk_w + 8;                                   // [slots] (+pad): the launch slots' routing weights
    int32_t* local_idx = (int32_t*)(topk_w + 12);                  // [slots]: index into `table`, -1 = unused
    float* up = (float*)(m0 + mp.router_bytes);
    uint16_t* hh = (uint16_t*)(m0 + mp.router_bytes + mp.up_bytes);    // [slots][F]
    float* down = (float*)(m0 + mp.router_bytes + mp.up_bytes + mp.h_bytes);

    // 1. q, k, v projections of x
    StreamJob qkv{}, oj{};
    qkv.w[0] = &A->q;
    qkv.w[1] = &A->k;
    qkv.w[2] = &A->v;
    oj.w[0] = &A->o;
    qkv.counters = oj.counters = counters;
    rc = launch_gemv_stream(qkv_part, x, nullptr, 1, qkv, ap.qkv, st);
    if (rc != HQM_OK) return rc;
    // 2. RoPE, cache append and attention
    QkvSource src{qkv_part, (int)A->n_heads, (int)A->n_kv_heads, ap.qkv.col0[3], A->rope_theta, split_of(ap.qkv),
                  colmap_of(ap.qkv), tc_error_ptr()};
    launch_overlapped_cluster(attn_decode_kernel<true>, (int)A->n_heads * ATTN_SPLIT, 256, 0, ATTN_SPLIT, st, ctx,
                              (const uint16_t*)nullptr, A->k_cache, A->v_cache, pos, (int)(A->n_heads / A->n_kv_heads),
                              (int)A->max_len, src);
    HQM_LAUNCH_CHECK();
    // 3. output projection
    rc = launch_gemv_stream(o_part, ctx, nullptr, 1, oj, ap.o, st);
    if (rc != HQM_OK) return rc;
    // 4. residual add, post-attention norm, router (and the rank's launch slots)
    launch_overlapped_cluster(finalize_add_rmsnorm_router_kernel, NORM_CTAS, NORM_THREADS, 0, NORM_CTAS, st, h,
                              (const float*)o_part, A->ln_post, x2, hidden, A->rms_eps, split_of(ap.o), colmap_of(ap.o),
                              L->gate_w, E, router_logits, topk_w, topk_idx, ep_lo, ep_n, slots, local_w, local_idx);
    HQM_LAUNCH_CHECK();
    // 5.-7. the slots' experts: [w1; w3] per slot, silu * mul, w2 per slot
    StreamJob gate_up{}, down_proj{};
    gate_up.table = down_proj.table = static_cast<const StreamEntry*>(L->table);
    gate_up.counters = down_proj.counters = counters;
    for (int slot = 0; slot < slots; ++slot) {
        gate_up.w[2 * slot] = &L->w1;
        gate_up.w[2 * slot + 1] = &L->w3;
        gate_up.sel[2 * slot] = gate_up.sel[2 * slot + 1] = local_idx + slot;
        gate_up.which[2 * slot] = 0;
        gate_up.which[2 * slot + 1] = 2;
        down_proj.w[slot] = &L->w2;
        down_proj.sel[slot] = local_idx + slot;
        down_proj.which[slot] = 1;
        down_proj.xrow[slot] = slot;
    }
    down_proj.sel_settled = 1;
    rc = launch_gemv_stream(up, x2, nullptr, 1, gate_up, mp.up, st);
    if (rc != HQM_OK) return rc;
    rc = launch_finalize_silu_mul(hh, up, 1, mp.up, st, /*late_trigger=*/true);
    if (rc != HQM_OK) return rc;
    rc = launch_gemv_stream(down, hh, nullptr, 1, down_proj, mp.down, st);
    if (rc != HQM_OK) return rc;
    if (comm) {
        // 8''. this rank's weighted share, written straight into every rank's exchange buffer
        launch_overlapped(finalize_weighted_publish_kernel, (hidden + EP_CHUNK - 1) / EP_CHUNK, EP_CHUNK, 0, st,
                          (const float*)down, (const float*)local_w, hidden, mp.down.col0[slots], split_of(mp.down),
                          colmap_of(mp.down), *comm);
        HQM_LAUNCH_CHECK();
        return HQM_OK;
    }
    if (y_partial) {
        // 8'. this rank's weighted share of the block's output, fp32; the caller adds the ranks' shares
        launch_overlapped(finalize_weighted_f32_kernel, (hidden + 255) / 256, 256, 0, st, y_partial, (const float*)down,
                          (const float*)local_w, hidden, mp.down.col0[slots], split_of(mp.down), colmap_of(mp.down));
        HQM_LAUNCH_CHECK();
        return HQM_OK;
    }
    // 8. weighted sum of the two experts, residual add, the next layer's input norm
    launch_overlapped_cluster(finalize_scatter_add_rmsnorm_kernel, NORM_CTAS, NORM_THREADS, 0, NORM_CTAS, st, h,
                              (const float*)down, (const float*)local_w, L->next_ln, x, hidden, mp.down.col0[2],
                              A->rms_eps, split_of(mp.down), colmap_of(mp.down));
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

size_t hqm_decode_layer_scratch_bytes(const hqm_decoder_layer* L) {
    hqm::AttnPlan ap;
    hqm::MoeDecodePlan mp;
    if (decoder_layer_plan(L, 2, &ap, &mp) != HQM_OK) return 0;
    return decoder_layer_bytes(ap, mp);
}

int hqm_decode_layer(uint16_t* h, uint16_t* x, uint16_t* router_logits, const hqm_decoder_layer* L, const int32_t* pos,
                     void* scratch, size_t scratch_bytes, void* stream) {
    return decode_layer_run(h, x, router_logits, nullptr, nullptr, L, 0, L ? L->n_experts : 0, 2, pos, scratch,
                            scratch_bytes, stream);
}

static int ep_slots(int n_local) { return n_local < 2 ? 1 : 2; }

size_t hqm_decode_layer_ep_scratch_bytes(const hqm_decoder_layer* L, int32_t n_local) {
    hqm::AttnPlan ap;
    hqm::MoeDecodePlan mp;
    if (n_local < 1 || decoder_layer_plan(L, ep_slots(n_local), &ap, &mp) != HQM_OK) return 0;
    return decoder_layer_bytes(ap, mp);
}

static int check_comm(const hqm_ep_comm* comm, int hidden) {
    using namespace hqm;
    HQM_CHECK_ARG(comm->world >= 1 && comm->world <= 8 && comm->rank >= 0 && comm->rank < comm->world && comm->seq,
                  "ep exchange: rank %d of %d (at most 8) or null counter", comm->rank, comm->world);
    HQM_CHECK_ARG(comm->hidden == hidden && (hidden + EP_CHUNK - 1) / EP_CHUNK <= EP_MAX_CHUNKS,
                  "ep exchange: buffers sized for hidden = %d, layer has %d (at most %d)", comm->hidden, hidden,
                  EP_CHUNK * EP_MAX_CHUNKS);
    for (int r = 0; r < comm->world; ++r)
        HQM_CHECK_ARG(comm->shares[r] && comm->flags[r], "ep exchange: null buffer of rank %d", r);
    return HQM_OK;
}

size_t hqm_ep_exchange_bytes(int32_t world, int32_t hidden) {
    if (world < 1 || world > 8 || hidden < 1) return 0;
    return (size_t)2 * world * hidden * sizeof(float) + (size_t)2 * world * hqm::EP_MAX_CHUNKS * sizeof(uint32_t);
}

size_t hqm_ep_exchange_flags_offset(int32_t world, int32_t hidden) { return (size_t)2 * world * hidden * sizeof(float); }

int hqm_decode_layer_ep(uint16_t* h, uint16_t* x_moe_unused, uint16_t* router_logits, float* y_partial,
                        const hqm_ep_comm* comm, const hqm_decoder_layer* L, int32_t expert_lo, int32_t n_local,
                        const int32_t* pos, void* scratch, size_t scratch_bytes, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(y_partial != nullptr || comm != nullptr, "decode_layer_ep: neither an output nor an exchange");
    HQM_CHECK_ARG(L && n_local >= 1 && expert_lo >= 0 && expert_lo + n_local <= L->n_experts,
                  "decode_layer_ep: experts [%d, %d) are not a range of the layer's experts", expert_lo, expert_lo + n_local);
    if (comm) {
        const int rc = check_comm(comm, L->attn.q.K);
        if (rc != HQM_OK) return rc;
    }
    return decode_layer_run(h, x_moe_unused, router_logits, y_partial, comm, L, expert_lo, n_local, ep_slots(n_local), pos,
                            scratch, scratch_bytes, stream);
}

int hqm_ep_combine_add_rmsnorm(uint16_t* h, const hqm_ep_comm* comm, const uint16_t* weight, uint16_t* x_out,
                               int32_t hidden, float eps, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(h && comm && weight && x_out && hidden > 0 && hidden <= NORM_CTAS * NORM_THREADS * NORM_PER_THREAD,
                  "ep_combine: null pointer or hidden size %d outside (0, %d]", hidden,
                  NORM_CTAS * NORM_THREADS * NORM_PER_THREAD);
    const int rc = check_comm(comm, hidden);
    if (rc != HQM_OK) return rc;
    launch_overlapped_cluster(ep_combine_add_rmsnorm_kernel, NORM_CTAS, NORM_THREADS, 0, NORM_CTAS, (cudaStream_t)stream, h,
                              weight, x_out, (int)hidden, eps, *comm, tc_error_ptr());
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

int hqm_add_f32_rmsnorm(uint16_t* h, const float* delta, const uint16_t* weight, uint16_t* x_out, int32_t hidden,
                        float eps, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(h && delta && weight && x_out && hidden > 0 && hidden <= NORM_CTAS * NORM_THREADS * NORM_PER_THREAD,
                  "add_f32_rmsnorm: null pointer or hidden size %d outside (0, %d]", hidden,
                  NORM_CTAS * NORM_THREADS * NORM_PER_THREAD);
    launch_overlapped_cluster(add_f32_rmsnorm_kernel, NORM_CTAS, NORM_THREADS, 0, NORM_CTAS, (cudaStream_t)stream, h, delta,
                              weight, x_out, (int)hidden, eps);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

}  // extern "C"
