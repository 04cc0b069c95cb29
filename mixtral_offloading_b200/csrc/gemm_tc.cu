// Prefill-size quantized GEMM on the 5th-generation tensor cores (tcgen05 + TMEM):
// the path that replaces the reference's Triton kernels (triton_kernels.py:37-131,
// 225-319) when many rows of x are multiplied at once.
//
//   sums[m, n] (+)= sum_k x[m, k] * W_est[n, k]          fp32, one tile of 128 output rows per CTA
//
// The weight is the MMA's A operand (M = 128 rows of W), the tokens are its N dimension
// (64 / 128 / 256 per tile), so a small batch wastes nothing.  Per 64-column k-block a CTA
//   0. requests every global load of the block at once (scale / zero bytes and their fp16
//      meta, the packed words, the x columns: one exposed round trip per block),
//   1. decodes scale and zero (8 bit -> s and -z*s, bf16) for the tile's residues once
//      into shared memory,
//   2. dequantises its 128 x 64 weights straight from the packed words into a
//      K-major, 128-byte-swizzled bf16 tile in shared memory (one LOP3 + one exact
//      subtract + one fused multiply-add per two weights),
//   3. copies the tokens' 64 columns of x into a second swizzled tile,
// and one elected thread issues four tcgen05.mma (K = 16 each) that accumulate into
// TMEM.  A ring of stages with mbarriers lets the dequantisation of block i+1 run while
// the tensor core works on block i; tcgen05.commit releases a stage when its MMAs have
// read it.  After the last block the four producer warps read the accumulator with
// tcgen05.ld and write (or, with split K, atomically add) fp32 sums.
//
// A tile's rows are the rows that share scale/zero columns: all `group_size` members of
// RT consecutive storage-row residues x the PER slots of a byte (RT*group_size*PER = 128).
//
// Every wait on an mbarrier is bounded: after a fraction of a second of polling the kernel sets an error
// flag, skips the rest of its work, still frees its TMEM and returns.
#include "common.cuh"
#include "kernels.cuh"
#include "tc_common.cuh"

namespace hqm {

namespace tc {

// bf16 pairs (128 + code) of one slot for columns (k0,k1) [lo] and (k2,k3) [hi] of a byte-permuted word
// (bytes B0,B2,B1,B3: low byte of each half = k0 / k1, high byte = k2 / k3).  The field is shifted to
// bits 1-0 (2-bit) or 3-0 (4-bit) of each half and OR-ed into the mantissa of 128.0.
template <int NBITS>
__device__ __forceinline__ void slot_pairs(uint32_t u, int s, uint32_t mask, uint32_t magic, uint32_t& lo,
                                           uint32_t& hi) {
    constexpr int PER = codes_per_word(NBITS);
    const int sh = NBITS * (PER - 1 - s);
    lo = lop_and_or(u >> sh, mask, magic);
    hi = lop_and_or(u >> (sh + 8), mask, magic);
}

struct Params {
    hqm_weight w[2];
    int layers;
    const uint16_t* x;         // (rows, K) bf16
    const int32_t* x_idx;      // optional gather
    int M;                     // rows of x in this launch (<= NTOK)
    int m_base;
    float* sums;               // (M_total, layers * N) fp32
    int M_total;
    int G, C, P;
    int tiles_per_layer;       // P / RT
    int splitk;                // CTAs along K; > 1: sums must be zero on entry, results are added atomically
    int kblocks;               // K / 64
    int* error_flag;
};

template <int NBITS, int NB, int NTOK>
struct Cfg {
    static constexpr int PER = codes_per_word(NBITS);
    static constexpr int GS = 16 * NB;                         // group size
    static constexpr int RT = TILE_ROWS / (GS * PER);          // residues per tile
    static_assert(RT * GS * PER == TILE_ROWS && RT >= 1, "tile must hold whole groups");
    static constexpr int RES = RT * PER;                       // scale/zero rows per tile
    static constexpr int A_BYTES = TILE_ROWS * 128;            // 16 KB
    static constexpr int B_BYTES = NTOK * 128;
    static constexpr int SZ_BYTES = RES * BK * 2 * 2;          // s and -z*s, bf16
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + ((SZ_BYTES + 1023) / 1024) * 1024;
    static constexpr int STAGES = (NTOK <= 64) ? 6 : (NTOK <= 128 ? 5 : 4);
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int NBITS, int NB, int NTOK>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(Params prm) {
    using CF = Cfg<NBITS, NB, NTOK>;
    constexpr int PER = CF::PER, GS = CF::GS, RT = CF::RT, RES = CF::RES, STAGES = CF::STAGES;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    unsigned char* tiles = smem_raw + ((1024u - (raw & 1023u)) & 1023u);         // 1024-byte aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)STAGES * CF::STAGE_BYTES);
    uint64_t* full = bars;                 // [STAGES] producers -> MMA
    uint64_t* empty = bars + STAGES;       // [STAGES] MMA -> producers
    uint64_t* accum = bars + 2 * STAGES;   // MMA -> epilogue
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = threadIdx.x / PRODUCERS;       // GROUPS = the MMA warp
    const int tid = threadIdx.x % PRODUCERS;         // thread inside its producer group
    const int tile = blockIdx.x / prm.splitk, ks = blockIdx.x % prm.splitk;
    const int layer = tile / prm.tiles_per_layer;
    const int rho0 = (tile % prm.tiles_per_layer) * RT;
    const hqm_weight& w = prm.w[layer];
    const int K = w.K, N = w.N, G = prm.G, P = prm.P;
    const int kb_per = (prm.kblocks + prm.splitk - 1) / prm.splitk;
    const int kb_begin = ks * kb_per, kb_end = min(prm.kblocks, kb_begin + kb_per);
    const int nkb = max(0, kb_end - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full + s, PRODUCERS);
            mbar_init(empty + s, 1);
        }
        mbar_init(accum, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (group == GROUPS) {   // TMEM: NTOK fp32 columns x 128 lanes for the accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)(NTOK < 32 ? 32 : NTOK))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;

    if (group < GROUPS) {
        // =========================== producers ===========================
        // group g fills the stages of k-blocks g, g + GROUPS, ...: the global-load latency of one
        // block overlaps the arithmetic of the others
        const int bar_id = 1 + group;
        const uint32_t mask = NBITS == 2 ? 0x00030003u : 0x000F000Fu;
        const uint32_t magic = 0x43004300u;            // 128.0 | code  (bf16)
        const uint8_t* Wq = reinterpret_cast<const uint8_t*>(w.W_q);
        for (int it = group; it < nkb; it += GROUPS) {
            const int s = it % STAGES;
            if (it >= STAGES && !*failed) {
                if (!mbar_wait(empty + s, ((it / STAGES) - 1) & 1)) *failed = 1;
            }
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");      // the whole group sees the same verdict
            if (*failed) break;
            unsigned char* st = tiles + (size_t)s * CF::STAGE_BYTES;
            unsigned char* sA = st;
            unsigned char* sB = st + CF::A_BYTES;
            __nv_bfloat16* sS = reinterpret_cast<__nv_bfloat16*>(st + CF::A_BYTES + CF::B_BYTES);   // [RES][64]  s
            __nv_bfloat16* sT = sS + RES * BK;                                                       // [RES][64] -z*s
            const int k0 = (kb_begin + it) * BK;
            // ---- every global load of the k-block is requested up front (one exposed round trip per k-block):
            // (a) scale / zero bytes and their fp16 meta for 4 consecutive columns of one residue row,
            // (b) the packed words of this thread's dequantisation tasks, (c) its chunks of the x tile
            constexpr int META_TASKS = RES * (BK / 4);
            constexpr int NTASK = RT * GS * 4 / PRODUCERS;
            static_assert(RT * GS * 4 % PRODUCERS == 0 && META_TASKS <= PRODUCERS, "task split");
            uint32_t sq4 = 0u, zq4 = 0u;
            uint2 m_ss = make_uint2(0u, 0u), m_zs = m_ss, m_sz = m_ss, m_zz = m_ss;
            const int mri = tid / (BK / 4), mkk = (tid % (BK / 4)) * 4;
            if (tid < META_TASKS) {
                const uint32_t idx = (uint32_t)(PER * rho0 + mri) * (uint32_t)K + (uint32_t)(k0 + mkk);
                const uint32_t col = idx % (uint32_t)prm.C;              // C % 4 == 0: the 4 columns do not wrap
                sq4 = *reinterpret_cast<const uint32_t*>(w.scale_q + idx);
                zq4 = *reinterpret_cast<const uint32_t*>(w.zero_q + idx);
                m_ss = *reinterpret_cast<const uint2*>(w.ms_scale + col);
                m_zs = *reinterpret_cast<const uint2*>(w.mz_scale + col);
                m_sz = *reinterpret_cast<const uint2*>(w.ms_zero + col);
                m_zz = *reinterpret_cast<const uint2*>(w.mz_zero + col);
            }
            constexpr bool X_EARLY = NTOK <= 128;      // the 256-token tile is streamed chunk by chunk after the dequantisation
            uint4 pk[NTASK];
            auto load_w = [&]() {
#pragma unroll
                for (int q = 0; q < NTASK; ++q) {
                    const int task = tid + q * PRODUCERS;
                    const int qq = task >> 2, c = task & 3;
                    const int rr = qq / GS, j = qq % GS;
                    const int64_t R = (int64_t)(rho0 + rr) + (int64_t)j * P;
                    pk[q] = ld_stream_16(Wq + R * K + k0 + 16 * c);
                }
            };
            if constexpr (X_EARLY) load_w();
            // (with 256 tokens the x tile is 16 chunks per thread: too many registers to hold across the
            // dequantisation, so it is fetched afterwards)
            constexpr int XT = X_EARLY ? NTOK * 8 / PRODUCERS : 1;
            uint4 xv[XT];
            auto load_x = [&]() {
#pragma unroll
                for (int q = 0; q < XT; ++q) {
                    const int task = tid + q * PRODUCERS;
                    const int tok = task >> 3, ch = task & 7;
                    xv[q] = make_uint4(0u, 0u, 0u, 0u);
                    if (tok < prm.M) {
                        const int mm = prm.m_base + tok;
                        const int64_t xrow = prm.x_idx ? prm.x_idx[mm] : mm;
                        xv[q] = *reinterpret_cast<const uint4*>(prm.x + xrow * K + k0 + 8 * ch);
                    }
                }
            };
            if constexpr (X_EARLY) load_x();
            // ---- 1. scale / zero of the tile's RES residue rows x 64 columns: s and -z*s as bf16
            if (tid < META_TASKS) {
                const uint32_t ms_s[2] = {m_ss.x, m_ss.y}, mz_s[2] = {m_zs.x, m_zs.y};
                const uint32_t ms_z[2] = {m_sz.x, m_sz.y}, mz_z[2] = {m_zz.x, m_zz.y};
                __nv_bfloat16 so[4], to[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t sh = 16u * (e & 1);
                    const float sc = ((float)((sq4 >> (8 * e)) & 0xffu) - f16_bits_to_float((uint16_t)(mz_s[e >> 1] >> sh))) *
                                     f16_bits_to_float((uint16_t)(ms_s[e >> 1] >> sh));
                    const float zr = ((float)((zq4 >> (8 * e)) & 0xffu) - f16_bits_to_float((uint16_t)(mz_z[e >> 1] >> sh))) *
                                     f16_bits_to_float((uint16_t)(ms_z[e >> 1] >> sh));
                    so[e] = __float2bfloat16_rn(sc);
                    to[e] = __float2bfloat16_rn(-zr * sc);
                }
                *reinterpret_cast<uint2*>(sS + mri * BK + mkk) = *reinterpret_cast<const uint2*>(so);
                *reinterpret_cast<uint2*>(sT + mri * BK + mkk) = *reinterpret_cast<const uint2*>(to);
            }
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
            // ---- 2. dequantise: one task = 16 bytes of one storage row = 16 columns x PER output rows
            if constexpr (!X_EARLY) load_w();
#pragma unroll
            for (int q = 0; q < NTASK; ++q) {
                const int task = tid + q * PRODUCERS;
                const int qq = task >> 2, c = task & 3;
                const int rr = qq / GS, j = qq % GS;
                const uint32_t words[4] = {pk[q].x, pk[q].y, pk[q].z, pk[q].w};
#pragma unroll
                for (int sl = 0; sl < PER; ++sl) {
                    const int ri = rr * PER + sl;
                    const int row = (rr * GS + j) * PER + sl;                 // tile row
                    const uint32_t* S2 = reinterpret_cast<const uint32_t*>(sS + ri * BK + 16 * c);
                    const uint32_t* T2 = reinterpret_cast<const uint32_t*>(sT + ri * BK + 16 * c);
                    uint32_t outw[8];
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        uint32_t lo, hi;
                        slot_pairs<NBITS>(byte_perm(words[wd], 0x3120u), sl, mask, magic, lo, hi);
                        lo = bf2_sub(lo, magic);                              // exact: the code itself
                        hi = bf2_sub(hi, magic);
                        outw[2 * wd] = bf2_fma(lo, S2[2 * wd], T2[2 * wd]);           // (k0, k1)
                        outw[2 * wd + 1] = bf2_fma(hi, S2[2 * wd + 1], T2[2 * wd + 1]);   // (k2, k3)
                    }
                    *reinterpret_cast<uint4*>(sA + sw128(row, 2 * c)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
                    *reinterpret_cast<uint4*>(sA + sw128(row, 2 * c + 1)) =
                        make_uint4(outw[4], outw[5], outw[6], outw[7]);
                }
            }
            // ---- 3. the tokens' 64 columns of x
            if constexpr (X_EARLY) {
#pragma unroll
                for (int q = 0; q < XT; ++q) {
                    const int task = tid + q * PRODUCERS;
                    *reinterpret_cast<uint4*>(sB + sw128(task >> 3, task & 7)) = xv[q];
                }
            } else {
#pragma unroll 4
                for (int task = tid; task < NTOK * 8; task += PRODUCERS) {
                    const int tok = task >> 3, ch = task & 7;
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (tok < prm.M) {
                        const int mm = prm.m_base + tok;
                        const int64_t xrow = prm.x_idx ? prm.x_idx[mm] : mm;
                        v = *reinterpret_cast<const uint4*>(prm.x + xrow * K + k0 + 8 * ch);
                    }
                    *reinterpret_cast<uint4*>(sB + sw128(tok, ch)) = v;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor core
            mbar_arrive(full + s);
        }
        // =========================== epilogue ===========================
        bool ok = !*failed && nkb > 0;
        if (ok && !mbar_wait(accum, 0)) {
            *failed = 1;
            ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);                       // tcgen05.ld below is warp-collective
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int wq = warp & 3;                                           // TMEM lane quarter of this warp
            const int row = 32 * wq + lane;                                    // TMEM lane = tile row
            const int sl = row % PER, j = (row / PER) % GS, rr = row / (PER * GS);
            const int64_t n = (int64_t)layer * N + (int64_t)j * G + PER * (rho0 + rr) + sl;
            const int64_t ncols = (int64_t)N * prm.layers;
#pragma unroll 1
            for (int c0 = 16 * group; c0 < NTOK; c0 += 16 * GROUPS) {      // the groups share the columns
                if (c0 >= prm.M) break;
                uint32_t v[16];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                      "=r"(v[15])
                    : "r"(tmem_d + ((uint32_t)(32 * wq) << 16) + (uint32_t)c0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int tok = c0 + i;
                    if (tok < prm.M) {
                        float* dst = prm.sums + (int64_t)(prm.m_base + tok) * ncols + n;
                        if (prm.splitk > 1) atomicAdd(dst, __uint_as_float(v[i]));
                        else *dst = __uint_as_float(v[i]);
                    }
                }
            }
        }
    } else {
        // =========================== MMA issuer (last warp) ===========================
        if (lane == 0) {
            // instruction descriptor: D fp32, A / B bf16, both K-major, N = NTOK, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) |
                                   ((uint32_t)(TILE_ROWS >> 4) << 24);
            bool ok = true;
            for (int it = 0; it < nkb && ok; ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(full + s, (it / STAGES) & 1)) {
                    *failed = 1;
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = smem_u32(tiles + (size_t)s * CF::STAGE_BYTES);
                const uint64_t da = smem_desc_sw128(a0), db = smem_desc_sw128(a0 + CF::A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)   // +32 bytes (2 descriptor units) per K = 16 step
                    umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty + s);             // the stage is free once these MMAs have read it
            }
            if (ok && nkb > 0) umma_commit(accum);
        }
        __syncwarp();
    }
    // ---- teardown: everyone is done with TMEM before it is freed
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (group == GROUPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                     "r"((uint32_t)(NTOK < 32 ? 32 : NTOK))
                     : "memory");
    }
    if (threadIdx.x == 0 && *failed && prm.error_flag) atomicExch(prm.error_flag, 1);
}

}  // namespace tc

// --------------------------------------------------------------------------- host side
static inline bool tc_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Device-side failure flag of the bounded waits (read by hqm_device_error()).
static __device__ int g_tc_error = 0;
int* tc_error_ptr() {
    static int* ptrs[MAX_DEVICES];                 // the flag of the current device (one copy per device)
    int*& ptr = ptrs[current_device_slot()];
    if (!ptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_tc_error) == cudaSuccess) ptr = (int*)p;
    }
    return ptr;
}

bool gemm_tc_supported(const hqm_weight* w, int G, int C, int64_t M) {
    if ((w->nbits != 2 && w->nbits != 4) || !meta_uniform(w)) return false;
    const int per = codes_per_word(w->nbits);
    const int g = w->group_size;
    if (!((w->nbits == 2 && (g == 16 || g == 32)) || (w->nbits == 4 && (g == 32 || g == 64)))) return false;
    const int rt = 128 / (g * per);
    if (G % per != 0 || (G / per) % rt != 0 || w->K % 64 != 0 || M < 1) return false;
    if ((int64_t)G * w->K >= ((int64_t)1 << 31)) return false;
    if (C % 4 != 0) return false;                  // 4 consecutive scale/zero columns share one meta load
    return tc_aligned16(w->W_q) && tc_aligned16(w->scale_q) && tc_aligned16(w->zero_q) && tc_aligned16(w->ms_scale) &&
           tc_aligned16(w->mz_scale) && tc_aligned16(w->ms_zero) && tc_aligned16(w->mz_zero);
}

int gemm_tc_splitk(const hqm_weight* w, int layers, int G) {
    const int per = codes_per_word(w->nbits);
    const int rt = 128 / (w->group_size * per);
    const int tiles = (G / per) / rt * layers;
    int sk = 1;
    while (tiles * sk < 148 && sk < 8 && (w->K / 64) / (2 * sk) >= 8) sk *= 2;
    return sk;
}

template <int NBITS, int NB, int NTOK>
static int launch_tc(const tc::Params& p, int grid, cudaStream_t st) {
    using CF = tc::Cfg<NBITS, NB, NTOK>;
    auto kern = tc::gemm_tc_kernel<NBITS, NB, NTOK>;
    static bool attr_done[MAX_DEVICES];
    bool& attr_set = attr_done[current_device_slot()];
    if (!attr_set) {
        HQM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CF::SMEM));
        attr_set = true;
    }
    kern<<<grid, tc::THREADS, CF::SMEM, st>>>(p);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

template <int NBITS, int NB>
static int launch_tc_tokens(const tc::Params& p, int grid, int ntok, cudaStream_t st) {
    if (ntok <= 64) return launch_tc<NBITS, NB, 64>(p, grid, st);
    if (ntok <= 128) return launch_tc<NBITS, NB, 128>(p, grid, st);
    return launch_tc<NBITS, NB, 256>(p, grid, st);
}

// sums (M, layers*N) fp32 = x . [w0; w1]^T.  With split K the caller-provided sums are zeroed here first.
int launch_gemm_tc(float* sums, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w0,
                   const hqm_weight* w1, int G, int C, cudaStream_t st) {
    if (!x_idx && gemm_tma_supported(w0, G, C, M)) return launch_gemm_tma(sums, x, M, w0, w1, G, C, st);
    const int layers = w1 ? 2 : 1;
    const int per = codes_per_word(w0->nbits);
    const int nb = w0->group_size / 16;
    const int rt = 128 / (w0->group_size * per);
    tc::Params p{};
    p.w[0] = *w0;
    p.w[1] = w1 ? *w1 : *w0;
    p.layers = layers;
    p.x = x;
    p.x_idx = x_idx;
    p.sums = sums;
    p.M_total = (int)M;
    p.G = G;
    p.C = C;
    p.P = G / per;
    p.tiles_per_layer = p.P / rt;
    p.splitk = gemm_tc_splitk(w0, layers, G);
    p.kblocks = w0->K / 64;
    p.error_flag = tc_error_ptr();
    if (p.splitk > 1) HQM_CUDA(cudaMemsetAsync(sums, 0, (size_t)M * w0->N * layers * sizeof(float), st));
    const int grid = p.tiles_per_layer * layers * p.splitk;
    for (int m0 = 0; m0 < (int)M; m0 += 256) {
        p.m_base = m0;
        p.M = ((int)M - m0 < 256) ? (int)M - m0 : 256;
        int rc;
        if (w0->nbits == 2 && nb == 1) rc = launch_tc_tokens<2, 1>(p, grid, p.M, st);
        else if (w0->nbits == 2 && nb == 2) rc = launch_tc_tokens<2, 2>(p, grid, p.M, st);
        else if (w0->nbits == 4 && nb == 2) rc = launch_tc_tokens<4, 2>(p, grid, p.M, st);
        else if (w0->nbits == 4 && nb == 4) rc = launch_tc_tokens<4, 4>(p, grid, p.M, st);
        else {
            set_error("gemm_tc: no instantiation for nbits=%d group_size=%d", w0->nbits, w0->group_size);
            return HQM_ERR_ARG;
        }
        if (rc != HQM_OK) return rc;
    }
    return HQM_OK;
}

// ---- small epilogue kernels over fp32 sums ---------------------------------------------
__global__ void rows_from_sums_kernel(uint16_t* __restrict__ y, const float* __restrict__ sums,
                                      const uint16_t* __restrict__ bias, int64_t MN, int N) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < MN; i += (int64_t)gridDim.x * blockDim.x) {
        float v = sums[i];
        if (bias) v += bf16_bits_to_float(bias[i % N]);
        y[i] = float_to_bf16_bits(v);
    }
}
// h[m, f] = bf16( bf16(silu(bf16(a))) * bf16(b) ), a = sums[m, f], b = sums[m, F + f]
__global__ void silu_mul_from_sums_kernel(uint16_t* __restrict__ h, const float* __restrict__ sums, int64_t M, int F) {
    const int64_t MF = M * F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < MF; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / F;
        const int f = (int)(i - m * F);
        const float a = round_bf16(sums[m * 2 * F + f]), b = round_bf16(sums[m * 2 * F + F + f]);
        h[i] = float_to_bf16_bits(round_bf16(a / (1.f + __expf(-a))) * b);
    }
}
// out[t] = (accumulate ? out[t] : 0) + bf16(w_i * bf16(sums[i])), t = token_idx[i]
__global__ void scatter_from_sums_kernel(uint16_t* __restrict__ out, const float* __restrict__ sums,
                                         const int32_t* __restrict__ token_idx, const float* __restrict__ route_w,
                                         int64_t M, int H, int accumulate) {
    const int64_t MH = M * H;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < MH; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / H;
        const int n = (int)(i - m * H);
        const int64_t tk = token_idx ? token_idx[m] : m;
        const float v = round_bf16(round_bf16(sums[i]) * (route_w ? route_w[m] : 1.f));
        uint16_t* dst = out + tk * H + n;
        *dst = float_to_bf16_bits(accumulate ? bf16_bits_to_float(*dst) + v : v);
    }
}

static inline int tc_blocks(int64_t n) {
    int64_t b = (n + 255) / 256;
    if (b > 148 * 16) b = 148 * 16;
    return (int)(b < 1 ? 1 : b);
}
int launch_rows_from_sums(uint16_t* y, const float* sums, const uint16_t* bias, int64_t M, int N, cudaStream_t st) {
    rows_from_sums_kernel<<<tc_blocks(M * N), 256, 0, st>>>(y, sums, bias, M * N, N);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}
int launch_silu_mul_from_sums(uint16_t* h, const float* sums, int64_t M, int F, cudaStream_t st) {
    silu_mul_from_sums_kernel<<<tc_blocks(M * F), 256, 0, st>>>(h, sums, M, F);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}
int launch_scatter_from_sums(uint16_t* out, const float* sums, const int32_t* token_idx, const float* route_w,
                             int accumulate, int64_t M, int H, cudaStream_t st) {
    scatter_from_sums_kernel<<<tc_blocks(M * H), 256, 0, st>>>(out, sums, token_idx, route_w, M, H, accumulate);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

}  // namespace hqm

// Reads and clears the device-side failure flag (see the header); synchronises the device.  Not part of
// the per-token path.
extern "C" int hqm_device_error(void) {
    int v = 0;
    int* p = hqm::tc_error_ptr();
    if (!p) return -1;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v != 0 && cudaMemset(p, 0, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
