// 3-bit quantized GEMM on the tcgen05 tensor cores: the path that replaces the reference's
// matmul3_kernel_transpose (triton_kernels.py:414-564) and the two Quantizer.dequantize calls in
// front of it (custom_layers.py:62-66) for five or more rows of x.
//
// Two launches per call.
//   1. meta_tables_kernel decodes the 8-bit scale and zero of the whole layer ONCE into two bf16
//      tables  S[r, k] = s  and  T[r, k] = -z * s  (the reference materialises fp16 scale and zero
//      the same way, per call).  With ten codes per word and G not a multiple of ten, the 64 rows
//      of a quantisation group are spread over 64 different tiles, so decoding inside the GEMM
//      would repeat this work 64 times.
//   2. gemm_tc3_kernel: a CTA owns 12 consecutive storage rows = 120 consecutive output rows (rows
//      120..127 of the MMA tile are unused).  Per 64-column k-block a producer thread takes one storage
//      row x 8 columns: eight int32 words, ten 3-bit fields each; two words are merged with PRMT so
//      that one LOP3 yields the bf16 pair 128 + code of two adjacent columns, an exact subtract
//      and one fused multiply-add with the row's (S, T) pairs give the dequantised weights, stored
//      as one 16-byte chunk of the K-major, 128-byte-swizzled A tile.  The tokens are the MMA's N
//      dimension (64 or 128), the accumulator lives in TMEM; ring of stages, full / empty
//      mbarriers with bounded waits, exactly as in gemm_tc.cu.
#include "common.cuh"
#include "kernels.cuh"
#include "tc_common.cuh"

namespace hqm {
namespace tc3 {

using namespace tc;

constexpr int WORDS_PER_TILE = 12;                   // storage rows per CTA
constexpr int ROWS_PER_TILE = 10 * WORDS_PER_TILE;   // 120 output rows
constexpr int STAGES = 6;

// S = s, T = -z * s for every (residue, column), bf16
__global__ void meta_tables_kernel(uint16_t* __restrict__ S, uint16_t* __restrict__ T, hqm_weight w, uint32_t GK,
                                   uint32_t C) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < GK; i += gridDim.x * blockDim.x) {
        const uint32_t col = i % C;
        const float sc = ((float)w.scale_q[i] - f16_bits_to_float(w.mz_scale[col])) * f16_bits_to_float(w.ms_scale[col]);
        const float zr = ((float)w.zero_q[i] - f16_bits_to_float(w.mz_zero[col])) * f16_bits_to_float(w.ms_zero[col]);
        S[i] = float_to_bf16_bits(sc);
        T[i] = float_to_bf16_bits(-zr * sc);
    }
}

struct Params {
    hqm_weight w;
    const uint16_t* S;         // (G, K) bf16
    const uint16_t* T;
    const uint16_t* x;         // (rows, K) bf16
    const int32_t* x_idx;      // optional gather
    int M;                     // rows of x in this launch (<= NTOK)
    int m_base;
    float* sums;               // (M_total, N) fp32
    int G;
    int rows;                  // storage rows, ceil(N / 10)
    int kblocks;               // K / 64
    int* error_flag;
};

template <int NTOK>
struct Cfg {
    static constexpr int A_BYTES = TILE_ROWS * 128;
    static constexpr int B_BYTES = NTOK * 128;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int NTOK>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc3_kernel(Params prm) {
    using CF = Cfg<NTOK>;
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
    const int tid = threadIdx.x % PRODUCERS;
    const hqm_weight& w = prm.w;
    const int K = w.K, N = w.N, G = prm.G;
    const int s0 = blockIdx.x * WORDS_PER_TILE;      // first storage row of the tile
    const int nkb = prm.kblocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full + s, PRODUCERS);
            mbar_init(empty + s, 1);
        }
        mbar_init(accum, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (group == GROUPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)NTOK)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;

    if (group < GROUPS) {
        // =========================== producers ===========================
        const int bar_id = 1 + group;
        const uint32_t mask = 0x00070007u, magic = 0x43004300u;       // 128.0 | code (bf16)
        const uint32_t* Wq = reinterpret_cast<const uint32_t*>(w.W_q);
        // this thread's dequantisation task: storage row i of the tile, 8-column chunk c
        const int i = tid >> 3, c = tid & 7;
        const int R = s0 + i;
        const bool has_task = (i < WORDS_PER_TILE) && (R < prm.rows);
        const int n_first = 10 * R;
        const uint32_t r_first = has_task ? (uint32_t)n_first % (uint32_t)G : 0u;
        for (int it = group; it < nkb; it += GROUPS) {
            const int s = it % STAGES;
            if (it >= STAGES && !*failed) {
                if (!mbar_wait(empty + s, ((it / STAGES) - 1) & 1)) *failed = 1;
            }
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");      // the whole group sees the same verdict
            if (*failed) break;
            unsigned char* sA = tiles + (size_t)s * CF::STAGE_BYTES;
            unsigned char* sB = sA + CF::A_BYTES;
            const int k0 = it * BK;
            // ---- every load a thread can hold is requested before anything is computed: the packed words, the
            // (S, T) rows of five slots at a time, and (64-token tile only) the x chunks
            constexpr bool X_EARLY = NTOK <= 64;
            constexpr int XT = X_EARLY ? NTOK * 8 / PRODUCERS : 1;
            uint4 xv[XT];
            if constexpr (X_EARLY) {
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
            }
            // ---- dequantise 10 rows x 8 columns
            if (has_task) {
                const uint32_t* src = Wq + (int64_t)R * K + k0 + 8 * c;
                const uint4 pa = ld_stream_16(src), pb = ld_stream_16(src + 4);
                // two adjacent columns per register: lo = low halves of both words (slots 9..5 at bits 0, 3, .., 12 of
                // each half), hi = the same of the words >> 15 (slots 4..0)
                const uint32_t w[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int cp = 0; cp < 4; ++cp) {
                    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(lo[cp]) : "r"(w[2 * cp]), "r"(w[2 * cp + 1]));
                    asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(hi[cp]) : "r"(w[2 * cp] >> 15), "r"(w[2 * cp + 1] >> 15));
                }
#pragma unroll
                for (int half = 0; half < 2; ++half) {                  // slots 0..4 (from hi), then 5..9 (from lo)
                    uint4 sv[5], tv[5];
#pragma unroll
                    for (int q = 0; q < 5; ++q) {
                        const int sl = 5 * half + q;
                        uint32_t r = r_first + (uint32_t)sl;
                        r = r >= (uint32_t)G ? r - (uint32_t)G : r;
                        if (r >= (uint32_t)G) r %= (uint32_t)G;         // only layers with fewer than ten groups
                        const size_t off = (size_t)r * K + k0 + 8 * c;
                        const bool ok = n_first + sl < N;
                        sv[q] = ok ? *reinterpret_cast<const uint4*>(prm.S + off) : make_uint4(0u, 0u, 0u, 0u);
                        tv[q] = ok ? *reinterpret_cast<const uint4*>(prm.T + off) : make_uint4(0u, 0u, 0u, 0u);
                    }
#pragma unroll
                    for (int q = 0; q < 5; ++q) {
                        const int sl = 5 * half + q;
                        const int sh = 3 * ((half ? 9 : 4) - sl);       // slot 4 / 9 sits at bit 0 of its half
                        const uint32_t* from = half ? lo : hi;
                        uint4 o;
                        o.x = bf2_fma(bf2_sub(lop_and_or(from[0] >> sh, mask, magic), magic), sv[q].x, tv[q].x);
                        o.y = bf2_fma(bf2_sub(lop_and_or(from[1] >> sh, mask, magic), magic), sv[q].y, tv[q].y);
                        o.z = bf2_fma(bf2_sub(lop_and_or(from[2] >> sh, mask, magic), magic), sv[q].z, tv[q].z);
                        o.w = bf2_fma(bf2_sub(lop_and_or(from[3] >> sh, mask, magic), magic), sv[q].w, tv[q].w);
                        if (n_first + sl < N) *reinterpret_cast<uint4*>(sA + sw128(10 * i + sl, c)) = o;
                    }
                }
            }
            // ---- the tokens' 64 columns of x
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
            const int64_t n = (int64_t)10 * s0 + row;
            const bool row_ok = row < ROWS_PER_TILE && n < N;
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
                if (row_ok) {
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        const int tok = c0 + q;
                        if (tok < prm.M) prm.sums[(int64_t)(prm.m_base + tok) * N + n] = __uint_as_float(v[q]);
                    }
                }
            }
        }
    } else {
        // =========================== MMA issuer (last warp) ===========================
        if (lane == 0) {
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
                for (int k = 0; k < BK / 16; ++k)
                    umma_bf16(tmem_d, da + 2 * k, db + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty + s);
            }
            if (ok && nkb > 0) umma_commit(accum);
        }
        __syncwarp();
    }
    // ---- teardown: everyone is done with TMEM before it is freed
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (group == GROUPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)NTOK)
                     : "memory");
    }
    if (threadIdx.x == 0 && *failed && prm.error_flag) atomicExch(prm.error_flag, 1);
}

}  // namespace tc3

// --------------------------------------------------------------------------- host side
static inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

bool gemm_tc3_supported(const hqm_weight* w, int G, int C, int64_t M) {
    (void)C;
    // up to 4 rows the streaming kernel (one launch per row) is faster than decoding the tables and
    // dequantising whole tiles
    if (w->nbits != 3 || M < 5 || w->K % 64 != 0 || !meta_uniform(w)) return false;
    if ((int64_t)G * w->K >= ((int64_t)1 << 31)) return false;
    return (reinterpret_cast<uintptr_t>(w->W_q) & 15u) == 0;
}

// [ fp32 sums (M, N) | S (G, K) bf16 | T (G, K) bf16 ]
size_t gemm_tc3_scratch_bytes(const hqm_weight* w, int G, int64_t M) {
    return up256((size_t)M * w->N * sizeof(float)) + 2 * up256((size_t)G * w->K * 2);
}

template <int NTOK>
static int launch_tc3(const tc3::Params& p, int grid, cudaStream_t st) {
    using CF = tc3::Cfg<NTOK>;
    auto kern = tc3::gemm_tc3_kernel<NTOK>;
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

int launch_gemm_tc3(uint16_t* y, void* scratch, const uint16_t* x, const int32_t* x_idx, int64_t M,
                    const hqm_weight* w, const uint16_t* bias, int G, int C, cudaStream_t st) {
    const size_t table = up256((size_t)G * w->K * 2);
    float* sums = (float*)scratch;
    uint16_t* S = (uint16_t*)((uint8_t*)scratch + up256((size_t)M * w->N * sizeof(float)));
    uint16_t* T = (uint16_t*)((uint8_t*)S + table);
    const uint32_t GK = (uint32_t)((int64_t)G * w->K);
    tc3::meta_tables_kernel<<<(int)((GK + 255) / 256 > 148 * 16 ? 148 * 16 : (GK + 255) / 256), 256, 0, st>>>(
        S, T, *w, GK, (uint32_t)C);
    HQM_LAUNCH_CHECK();
    tc3::Params p{};
    p.w = *w;
    p.S = S;
    p.T = T;
    p.x = x;
    p.x_idx = x_idx;
    p.sums = sums;
    p.G = G;
    p.rows = (w->N + 9) / 10;
    p.kblocks = w->K / 64;
    p.error_flag = tc_error_ptr();
    const int grid = (p.rows + tc3::WORDS_PER_TILE - 1) / tc3::WORDS_PER_TILE;
    for (int m0 = 0; m0 < (int)M; m0 += 128) {
        p.m_base = m0;
        p.M = ((int)M - m0 < 128) ? (int)M - m0 : 128;
        const int rc = (p.M <= 64) ? launch_tc3<64>(p, grid, st) : launch_tc3<128>(p, grid, st);
        if (rc != HQM_OK) return rc;
    }
    return launch_rows_from_sums(y, sums, bias, M, w->N, st);
}

}  // namespace hqm
