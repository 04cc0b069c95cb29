// Many-row quantized GEMM on the 5th-generation tensor cores, second generation of gemm_tc.cu: the same
// arithmetic (weights as the MMA's A operand, 128 output rows per tile, tokens as its N dimension, fp32
// accumulators in TMEM), but nothing a thread computes with comes straight from global memory any more.
//
//   sums[m, n] = sum_k x[m, k] * W_est[n, k]          fp32
//
// Replaces the reference's Triton kernels (triton_kernels.py:37-131, 225-319) for 17 or more rows of x.
//
// A unit of work is one 64-column k-block of one tile (128 output rows x one chunk of NTOK tokens).  Three rings
// of shared-memory buffers decouple what has different sizes and latencies:
//   raw ring (2 PG deep, 3-5 KB)    the packed codes of the tile's storage rows and its scale and zero bytes, as
//                               they lie in HBM
//   B ring (PG or 2 PG deep)     the x tile (NTOK rows x 64 bf16, 128-byte swizzle): it IS the MMA's B operand
//   A ring (5 to 8 deep, 16 KB)   the dequantised weights, K-major, 128-byte swizzle, plus the decoded scales
// Roles of the warps of a CTA (one CTA per SM, persistent; PG = 4 producer groups, 3 with 128- and 256-token tiles):
//   producers    PG groups of 128 threads; group g takes the units g, g+PG, ...: decodes scale / zero (8 bit -> s
//                and -z*s as bf16; the fp16 meta values are the only thing read with plain loads, requested
//                before the group waits for its buffers), dequantises 128 x 64 weights into an A slot (one LOP3,
//                one exact subtract, one fused multiply-add per two weights), hands the raw slot back
//   issue warps  PG warps; warp w issues the tiled TMA copies of the units w, w+PG, ...: three lanes the raw
//                copies, a fourth the x tile; mbarriers count the bytes.  (One thread issuing every copy of
//                every unit was the bottleneck: a tiled copy costs its issuing thread some hundred cycles.)
//   MMA warp     one lane issues the four tcgen05.mma (K = 16 each) of a unit and the commits that release its A
//                and B slots; at the end of a tile it commits the accumulator to the epilogue warps
//   epilogue     four warps read a finished accumulator with tcgen05.ld (each its quarter of the TMEM lanes), turn
//                it round in shared memory and write PER consecutive output rows of a token at a time.  Two
//                accumulators (2 x NTOK columns) alternate, so the next tile's MMAs run meanwhile.
//
// Work split: every CTA takes items / grid whole tiles (their sums are stored) and an equal contiguous slice of
// the k-blocks of the tiles left over (those are completed by vector reductions into zeroed sums), so no SM idles
// while another finishes a tile.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the error flag, all roles leave their loops,
// TMEM is freed and the kernel returns.
#include <cuda.h>
#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "kernels.cuh"
#include "tc_common.cuh"

namespace hqm {

namespace tc2 {
using namespace tc;

constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int EPI_PITCH = 36;                    // floats per token row of an epilogue warp's transpose buffer (32 + pad)
constexpr int EPI_BYTES = 4 * 16 * EPI_PITCH * 4;

struct Params {
    CUtensorMap x_map;                           // (K, rows) bf16, box (64, NTOK), 128-byte swizzle
    CUtensorMap w0_map[3], w1_map[3];            // per layer: codes (K, P, group) box (64, RT, group); scale_q and zero_q (K, G) box (64, RES)
    const uint16_t* meta0[4];                    // ms_scale, mz_scale, ms_zero, mz_zero (fp16) of layer 0
    const uint16_t* meta1[4];
    int layers, N, K, C, P;
    int tiles_per_layer, chunks, kblocks, items; // items = layers * tiles_per_layer * chunks
    int M_total;
    float* sums;                                 // (M_total, layers * N); zero on entry when tiles are split
    int* error_flag;
};

template <int NBITS, int NB, int NTOK>
struct Cfg {
    static constexpr int PER = codes_per_word(NBITS);
    static constexpr int GS = 16 * NB;
    static constexpr int RT = TILE_ROWS / (GS * PER);
    static_assert(RT * GS * PER == TILE_ROWS && RT >= 1, "tile must hold whole groups");
    static constexpr int RES = RT * PER;
    // PG producer groups of 128 threads, PG warps that issue the copies, the MMA warp, 4 epilogue warps (four
    // consecutive warps: each TMEM lane quarter once)
    static constexpr int PG = NTOK >= 128 ? 3 : 4;
    static constexpr int WARP_ISSUE = 4 * PG, WARP_MMA = 5 * PG, WARP_EPI = 5 * PG + 1;
    static constexpr int NTHREADS = (WARP_EPI + 4) * 32;
    // Ring depths.  A wait by phase parity is only sound while the waiter is at most one phase behind the
    // barrier.  Raw and B slots are refilled by one issue warp each (depths are multiples of PG), which waited for
    // the slot's previous release itself.  A slots rotate over the groups: group g's previous unit is PG back, which
    // proves that the unit PG + N_A back has been consumed; N_A >= PG makes that cover the slot's last-but-one
    // release.  The A ring takes what shared memory the B ring (x tiles in flight against the copy latency) leaves.
    static constexpr int N_RAW = 2 * PG;
    static constexpr int N_B = NTOK > 128 ? PG : (NTOK > 64 ? 2 * PG : 2 * PG);
    static constexpr int B_BYTES = NTOK * 128;
    static constexpr int W_BYTES = GS * RT * BK;              // staged packed bytes: [member][residue][64]
    static constexpr int Q_BYTES = RES * BK;                  // staged scale (and zero) bytes: [row][64]
    static constexpr int D_BYTES = RES * BK * 2;              // decoded s (and -z*s) as bf16
    // raw slot
    static constexpr int SQ_OFF = W_BYTES, ZQ_OFF = SQ_OFF + Q_BYTES;
    static constexpr int RAW_BYTES = (ZQ_OFF + Q_BYTES + 127) / 128 * 128;
    static constexpr uint32_t RAW_TX = W_BYTES + 2 * Q_BYTES;
    // A slot: the tile, then s and -z*s
    static constexpr int S_OFF = TILE_ROWS * 128, T_OFF = S_OFF + D_BYTES;
    static constexpr int A_BYTES = (T_OFF + D_BYTES + 1023) / 1024 * 1024;
    static constexpr int FIXED = 1024 /*alignment slack*/ + 1024 /*barriers*/ + EPI_BYTES + N_RAW * RAW_BYTES + N_B * B_BYTES;
    static constexpr int NA_FIT = (SMEM_LIMIT - FIXED) / A_BYTES;
    static constexpr int N_A = NA_FIT > 8 ? 8 : NA_FIT;
    static_assert(N_A >= PG, "A ring too shallow for the producer groups");
    static constexpr int B_OFF = 0, A_OFF = N_B * B_BYTES, RAW_OFF = A_OFF + N_A * A_BYTES, EPI_OFF = RAW_OFF + N_RAW * RAW_BYTES,
                         BAR_OFF = EPI_OFF + EPI_BYTES;
    static constexpr size_t SMEM = (size_t)BAR_OFF + 1024 + 1024;
    static constexpr uint32_t TMEM_COLS = 2 * NTOK;           // 128 / 256 / 512: a power of two >= 32
};

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the roles that can afford a late wake-up: sleeps after every look, so that the waiting warps
// leave the issue slots of their scheduler to the warps that have work (the MMA-issuing lane above all).
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        __nanosleep(i < 16 ? 32 : 128);
    }
    return false;
}
// Tiled copies global -> shared memory of this CTA, completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
// Named barrier over 128 threads that also ORs a flag: every thread gets the same answer.
__device__ __forceinline__ bool group_any(int bar_id, bool flag) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "barrier.cta.red.or.pred p, %2, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)flag), "r"(bar_id)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ uint4 lds128(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}
// byte `i` of `v` as a float: 2^23 + b is exact, the subtraction gives b
__device__ __forceinline__ float byte_to_float(uint32_t v, int i) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(v), "r"(0x4B000000u), "r"(0x7650u + (uint32_t)i));
    return __uint_as_float(r) - 8388608.f;
}

// The share of one CTA: `whole` complete tiles (tile i * grid + block: nobody else touches their sums, so they
// are stored, not added), then an equal slice [r0, r0 + rn) of the k-block units of the tiles left over.
struct Work {
    int whole, r0, rn, n_units;
};
__device__ __forceinline__ Work work_of(const Params& prm) {
    Work w;
    const int grid = (int)gridDim.x, b = (int)blockIdx.x;
    w.whole = prm.items / grid;
    const int64_t rem_units = (int64_t)(prm.items - w.whole * grid) * prm.kblocks;
    w.r0 = (int)(rem_units * b / grid);
    w.rn = (int)(rem_units * (b + 1) / grid) - w.r0;
    w.n_units = w.whole * prm.kblocks + w.rn;
    return w;
}
// Walks the CTA's units; the divisions happen once per tile, not per k-block.
template <int RT>
struct Cursor {
    int it, seg_begin, seg_end;      // seg: the run of this CTA's units inside one tile
    int kb, layer, rho0, chunk;
    __device__ __forceinline__ void locate(int at, const Work& w, const Params& prm) {
        it = at;
        if (at >= w.n_units) return;
        const int nw = w.whole * prm.kblocks;
        int item;
        if (at < nw) {
            const int i = at / prm.kblocks;
            kb = at - i * prm.kblocks;
            item = i * (int)gridDim.x + (int)blockIdx.x;
            seg_begin = at - kb;
            seg_end = seg_begin + prm.kblocks;
        } else {
            const int u = w.r0 + (at - nw);
            const int i = u / prm.kblocks;
            kb = u - i * prm.kblocks;
            item = w.whole * (int)gridDim.x + i;
            const int kb0 = max(0, kb - (at - nw));              // first k-block of the tile that is ours
            seg_begin = at - (kb - kb0);
            seg_end = min(at + (prm.kblocks - kb), w.n_units);
        }
        const int t = item / prm.chunks;
        chunk = item - t * prm.chunks;
        layer = t / prm.tiles_per_layer;
        rho0 = (t - layer * prm.tiles_per_layer) * RT;
    }
    __device__ __forceinline__ void advance(int step, const Work& w, const Params& prm) {
        if (it + step < seg_end) {
            it += step;
            kb += step;
        } else {
            locate(it + step, w, prm);
        }
    }
};


template <int NBITS, int NB, int NTOK>
__global__ void __launch_bounds__((Cfg<NBITS, NB, NTOK>::NTHREADS), 1)
gemm_tma_kernel(const __grid_constant__ Params prm) {
    using CF = Cfg<NBITS, NB, NTOK>;
    constexpr int PER = CF::PER, GS = CF::GS, RT = CF::RT, RES = CF::RES, N_B = CF::N_B, N_A = CF::N_A, N_RAW = CF::N_RAW;
    constexpr int PGROUPS = CF::PG, WARP_ISSUE = CF::WARP_ISSUE, WARP_MMA = CF::WARP_MMA, WARP_EPI = CF::WARP_EPI;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    unsigned char* base = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
    unsigned char* b_ring = base + CF::B_OFF;
    unsigned char* a_ring = base + CF::A_OFF;
    unsigned char* raw_ring = base + CF::RAW_OFF;
    float* epi_buf = reinterpret_cast<float*>(base + CF::EPI_OFF);
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + CF::BAR_OFF);
    uint64_t* raw_full = bars;                     // [N_RAW] copies landed
    uint64_t* raw_empty = raw_full + N_RAW;        // [N_RAW] a producer group has read the slot
    uint64_t* a_full = raw_empty + N_RAW;          // [N_A] A tile written
    uint64_t* a_empty = a_full + N_A;              // [N_A] the MMAs have read the A slot
    uint64_t* b_full = a_empty + N_A;              // [N_B] x tile landed
    uint64_t* done = b_full + N_B;                 // [N_B] the MMAs have read the B slot
    uint64_t* acc_full = done + N_B;               // [2] MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;            // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);
    static_assert((2 * N_RAW + 2 * N_A + 2 * N_B + 4) * 8 + 8 <= 1024, "barrier area");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Work work = work_of(prm);
    const int n_units = work.n_units;

    if (threadIdx.x == 0) {
        for (int s = 0; s < N_RAW; ++s) {
            mbar_init(raw_full + s, 1);
            mbar_init(raw_empty + s, PRODUCERS);
        }
        for (int s = 0; s < N_A; ++s) {
            mbar_init(a_full + s, PRODUCERS);
            mbar_init(a_empty + s, 1);
        }
        for (int s = 0; s < N_B; ++s) {
            mbar_init(b_full + s, 1);
            mbar_init(done + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full + b, 1);
            mbar_init(acc_empty + b, 4);
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(CF::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;

    if (warp < WARP_ISSUE) {
        // =========================== producers ===========================
        const int group = warp >> 2, tid = threadIdx.x & (PRODUCERS - 1);
        const int bar_id = 1 + group;
        const uint32_t mask = NBITS == 2 ? 0x00030003u : 0x000F000Fu;
        const uint32_t magic = 0x43004300u;            // 128.0 | code  (bf16)
        constexpr int META_TASKS = RES * (BK / 4);
        constexpr int NTASK = RT * GS * 4 / PRODUCERS;
        static_assert(RT * GS * 4 % PRODUCERS == 0 && META_TASKS <= PRODUCERS, "task split");
        const int mri = tid / (BK / 4), mkk = (tid % (BK / 4)) * 4;
        Cursor<RT> cur;
        cur.locate(group, work, prm);
        int base_seg = -1;
        uint32_t base_col = 0;
        for (int it = group; it < n_units; it += PGROUPS) {
            const int r = it % N_RAW, a = it % N_A;
            // the fp16 meta values of the 4 scale / zero columns this thread decodes: requested before the waits, used
            // right after them (no load of this thread is in flight when it fences its shared-memory writes below)
            uint2 m_ss = make_uint2(0u, 0u), m_zs = m_ss, m_sz = m_ss, m_zz = m_ss;
            if (tid < META_TASKS) {
                if (cur.seg_begin != base_seg) {     // the row start's flat scale index modulo the meta columns: per tile
                    base_seg = cur.seg_begin;
                    base_col = (uint32_t)(((uint64_t)(PER * cur.rho0 + mri) * (uint64_t)prm.K) % (uint32_t)prm.C);
                }
                uint32_t col = base_col + (uint32_t)(cur.kb * BK + mkk);    // C % 64 == 0: a k-block's columns do not wrap
                if (col >= (uint32_t)prm.C) col %= (uint32_t)prm.C;
                const uint16_t* const* mt = cur.layer ? prm.meta1 : prm.meta0;
                m_ss = *reinterpret_cast<const uint2*>(mt[0] + col);
                m_zs = *reinterpret_cast<const uint2*>(mt[1] + col);
                m_sz = *reinterpret_cast<const uint2*>(mt[2] + col);
                m_zz = *reinterpret_cast<const uint2*>(mt[3] + col);
            }
            cur.advance(PGROUPS, work, prm);
            bool bad = *failed != 0;
            if (!bad && !mbar_wait_relaxed(raw_full + r, (it / N_RAW) & 1)) bad = true;
            // the A slot's previous tile (unit it - N_A) has been read by its MMAs
            if (!bad && it >= N_A && !mbar_wait_relaxed(a_empty + a, ((it / N_A) - 1) & 1)) bad = true;
            bad = group_any(bar_id, bad);                                    // the whole group takes the same decision
            if (bad) {
                *failed = 1;
                break;
            }
            const unsigned char* rw = raw_ring + (size_t)r * CF::RAW_BYTES;
            unsigned char* sA = a_ring + (size_t)a * CF::A_BYTES;
            __nv_bfloat16* sS = reinterpret_cast<__nv_bfloat16*>(sA + CF::S_OFF);   // [RES][64]  s
            __nv_bfloat16* sT = reinterpret_cast<__nv_bfloat16*>(sA + CF::T_OFF);   // [RES][64] -z*s
            // ---- 1. scale / zero of the tile's RES residue rows x 64 columns: s and -z*s as bf16
            if (tid < META_TASKS) {
                const uint32_t sq4 = *reinterpret_cast<const uint32_t*>(rw + CF::SQ_OFF + mri * BK + mkk);
                const uint32_t zq4 = *reinterpret_cast<const uint32_t*>(rw + CF::ZQ_OFF + mri * BK + mkk);
                const uint32_t ms_s[2] = {m_ss.x, m_ss.y}, mz_s[2] = {m_zs.x, m_zs.y};
                const uint32_t ms_z[2] = {m_sz.x, m_sz.y}, mz_z[2] = {m_zz.x, m_zz.y};
                float sc[4], tt[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t sh = 16u * (e & 1);
                    sc[e] = (byte_to_float(sq4, e) - f16_bits_to_float((uint16_t)(mz_s[e >> 1] >> sh))) *
                            f16_bits_to_float((uint16_t)(ms_s[e >> 1] >> sh));
                    const float zr = (byte_to_float(zq4, e) - f16_bits_to_float((uint16_t)(mz_z[e >> 1] >> sh))) *
                                     f16_bits_to_float((uint16_t)(ms_z[e >> 1] >> sh));
                    tt[e] = -zr * sc[e];
                }
                __nv_bfloat162 s01 = __floats2bfloat162_rn(sc[0], sc[1]), s23 = __floats2bfloat162_rn(sc[2], sc[3]);
                __nv_bfloat162 t01 = __floats2bfloat162_rn(tt[0], tt[1]), t23 = __floats2bfloat162_rn(tt[2], tt[3]);
                *reinterpret_cast<uint2*>(sS + mri * BK + mkk) =
                    make_uint2(*reinterpret_cast<uint32_t*>(&s01), *reinterpret_cast<uint32_t*>(&s23));
                *reinterpret_cast<uint2*>(sT + mri * BK + mkk) =
                    make_uint2(*reinterpret_cast<uint32_t*>(&t01), *reinterpret_cast<uint32_t*>(&t23));
            }
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
            // ---- 2. dequantise: one task = 16 staged bytes of one storage row = 16 columns x PER output rows
#pragma unroll
            for (int q = 0; q < NTASK; ++q) {
                const int task = tid + q * PRODUCERS;
                const int qq = task >> 2, c = task & 3;
                const int rr = qq / GS, j = qq % GS;
                const uint4 pk = lds128(rw + (j * RT + rr) * BK + 16 * c);
                // bytes B0,B2,B1,B3: the low byte of each half holds columns k0 / k1, the high byte k2 / k3
                const uint32_t words[4] = {byte_perm(pk.x, 0x3120u), byte_perm(pk.y, 0x3120u), byte_perm(pk.z, 0x3120u),
                                           byte_perm(pk.w, 0x3120u)};
#pragma unroll
                for (int sl = 0; sl < PER; ++sl) {
                    const int ri = rr * PER + sl;
                    const int row = (rr * GS + j) * PER + sl;                 // tile row
                    const uint4 s_lo = lds128(sS + ri * BK + 16 * c), s_hi = lds128(sS + ri * BK + 16 * c + 8);
                    const uint4 t_lo = lds128(sT + ri * BK + 16 * c), t_hi = lds128(sT + ri * BK + 16 * c + 8);
                    const uint32_t S2[8] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w, s_hi.x, s_hi.y, s_hi.z, s_hi.w};
                    const uint32_t T2[8] = {t_lo.x, t_lo.y, t_lo.z, t_lo.w, t_hi.x, t_hi.y, t_hi.z, t_hi.w};
                    uint32_t outw[8];
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        const int sh = NBITS * (PER - 1 - sl);
                        uint32_t lo = lop_and_or(words[wd] >> sh, mask, magic);
                        uint32_t hi = lop_and_or(words[wd] >> (sh + 8), mask, magic);
                        lo = bf2_sub(lo, magic);                              // exact: the code itself
                        hi = bf2_sub(hi, magic);
                        outw[2 * wd] = bf2_fma(lo, S2[2 * wd], T2[2 * wd]);               // (k0, k1)
                        outw[2 * wd + 1] = bf2_fma(hi, S2[2 * wd + 1], T2[2 * wd + 1]);   // (k2, k3)
                    }
                    *reinterpret_cast<uint4*>(sA + sw128(row, 2 * c)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
                    *reinterpret_cast<uint4*>(sA + sw128(row, 2 * c + 1)) =
                        make_uint4(outw[4], outw[5], outw[6], outw[7]);
                }
            }
            mbar_arrive(raw_empty + r);                                    // the staged bytes have been read
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor core
            mbar_arrive(a_full + a);
        }
    } else if (warp < WARP_MMA) {
        // =========================== copy issue ===========================
        // issue warp w serves the units w, w + PG, ...: lanes 0-2 the three raw copies, lane 3 the x tile
        const int w = warp - WARP_ISSUE;
        Cursor<RT> cur;
        cur.locate(w, work, prm);
        for (int it = w; it < n_units; it += PGROUPS) {
            const int r = it % N_RAW, b = it % N_B;
            int ok = 1;
            if (lane == 0) {
                if (it >= N_RAW && !mbar_wait_relaxed(raw_empty + r, ((it / N_RAW) - 1) & 1)) *failed = 1;
                if (!*failed && it >= N_B && !mbar_wait_relaxed(done + b, ((it / N_B) - 1) & 1)) *failed = 1;
                ok = *failed ? 0 : 1;
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            const uint32_t dst = smem_u32(raw_ring + (size_t)r * CF::RAW_BYTES);
            const uint32_t bar = smem_u32(raw_full + r);
            const CUtensorMap* wm = cur.layer ? prm.w1_map : prm.w0_map;
            const int k0 = cur.kb * BK;
            if (lane == 0) {
                mbar_expect_tx(bar, CF::RAW_TX);
                tma_load_3d(dst, wm + 0, k0, cur.rho0, 0, bar);
            } else if (lane < 3) {
                tma_load_2d(dst + (lane == 1 ? CF::SQ_OFF : CF::ZQ_OFF), wm + lane, k0, PER * cur.rho0, bar);
            } else if (lane == 3) {
                const uint32_t bbar = smem_u32(b_full + b);
                mbar_expect_tx(bbar, CF::B_BYTES);
                tma_load_2d(smem_u32(b_ring + (size_t)b * CF::B_BYTES), &prm.x_map, k0, cur.chunk * NTOK, bbar);
            }
            __syncwarp();
            cur.advance(PGROUPS, work, prm);
        }
    } else if (warp == WARP_MMA) {
        // =========================== MMA issue ===========================
        if (lane == 0) {
            // instruction descriptor: D fp32, A / B bf16, both K-major, N = NTOK, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NTOK >> 3) << 17) |
                                   ((uint32_t)(TILE_ROWS >> 4) << 24);
            // This lane's instruction stream is the floor of the whole pipeline (a unit's four MMAs take 128 to 512
            // tensor cycles), so everything per unit is kept incremental: slot indices, phases and the descriptors'
            // address fields advance by constants, the tile boundaries come from a countdown.
            Cursor<RT> cur;
            cur.locate(0, work, prm);
            int left = cur.seg_end - cur.seg_begin;                  // units of the current tile still to issue
            bool first = true;
            int seg = 0;
            constexpr uint64_t DESC_HI = (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
            const uint32_t a_enc0 = (smem_u32(a_ring) & 0x3FFFFu) >> 4, b_enc0 = (smem_u32(b_ring) & 0x3FFFFu) >> 4;
            uint32_t a_enc = a_enc0, b_enc = b_enc0;                 // start-address fields of the slots in use
            int a = 0, b = 0;
            uint32_t a_par = 0, b_par = 0;
            for (int it = 0; it < n_units; ++it) {
                const int buf = seg & 1;
                if (first && seg >= 2) {            // the epilogue has drained this accumulator
                    if (!mbar_wait(acc_empty + buf, ((seg >> 1) - 1) & 1)) {
                        *failed = 1;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                if (!mbar_wait(b_full + b, b_par) || !mbar_wait(a_full + a, a_par)) {
                    *failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = DESC_HI | a_enc, db = DESC_HI | b_enc;
                const uint32_t d = tmem_d + (uint32_t)(buf * NTOK);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)   // +32 bytes (2 descriptor units) per K = 16 step
                    umma_bf16(d, da + 2 * k, db + 2 * k, idesc, (!first || k > 0) ? 1u : 0u);
                umma_commit(a_empty + a);           // the slots are free once these MMAs have read them
                umma_commit(done + b);
                first = false;
                if (--left == 0) {                  // the tile's (or this CTA's share of its) k-blocks are issued
                    umma_commit(acc_full + buf);
                    ++seg;
                    cur.locate(cur.seg_end, work, prm);
                    left = cur.seg_end - cur.seg_begin;
                    first = true;
                }
                if (++a == N_A) {
                    a = 0;
                    a_par ^= 1u;
                    a_enc = a_enc0;
                } else {
                    a_enc += CF::A_BYTES >> 4;
                }
                if (++b == N_B) {
                    b = 0;
                    b_par ^= 1u;
                    b_enc = b_enc0;
                } else {
                    b_enc += CF::B_BYTES >> 4;
                }
            }
        }
        __syncwarp();
    } else {
        // =========================== epilogue ===========================
        // A warp reads its 32 TMEM lanes (tile rows) x 16 tokens, turns the block round in shared memory and
        // writes PER consecutive output rows of one token at a time (the rows of a packed byte are neighbours in
        // n): one vector store, or one vector reduction where another CTA adds to the same tile.
        const int wq = warp & 3;                                           // TMEM lane quarter of this warp
        constexpr int VG = 32 / PER;                                       // row groups of a warp
        const int vg = lane % VG, vt = lane / VG;                          // this lane writes group vg, tokens vt, vt + 32 / VG, ...
        const int row0 = 32 * wq + PER * vg;                               // first tile row of the group (slot 0)
        const int j = (row0 / PER) % GS, rr = row0 / (PER * GS);
        const int64_t ncols = (int64_t)prm.N * prm.layers;
        const int G = prm.P * PER;
        float* tb = epi_buf + (warp - WARP_EPI) * 16 * EPI_PITCH;
        Cursor<RT> cur;
        cur.locate(0, work, prm);
        int seg = 0;
        while (cur.it < n_units) {
            const int buf = seg & 1;
            bool ok = !*failed && mbar_wait_relaxed(acc_full + buf, (seg >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);                       // tcgen05.ld below is warp-collective
            if (!ok) {
                *failed = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t n0 = (int64_t)cur.layer * prm.N + (int64_t)j * G + PER * (cur.rho0 + rr);
            const int m_base = cur.chunk * NTOK;
            const bool whole = cur.seg_end - cur.seg_begin == prm.kblocks;       // nobody else adds to this tile
#pragma unroll 1
            for (int c0 = 0; c0 < NTOK; c0 += 16) {
                if (m_base + c0 >= prm.M_total) break;
                uint32_t v[16];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                      "=r"(v[15])
                    : "r"(tmem_d + ((uint32_t)(32 * wq) << 16) + (uint32_t)(buf * NTOK + c0)));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) tb[i * EPI_PITCH + lane] = __uint_as_float(v[i]);
                __syncwarp();
#pragma unroll
                for (int t = vt; t < 16; t += 32 / VG) {
                    const int tok = m_base + c0 + t;
                    if (tok < prm.M_total) {
                        float* dst = prm.sums + (int64_t)tok * ncols + n0;
                        if constexpr (PER == 4) {
                            const float4 o = *reinterpret_cast<const float4*>(tb + t * EPI_PITCH + PER * vg);
                            if (whole) *reinterpret_cast<float4*>(dst) = o;
                            else
                                asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "f"(o.x), "f"(o.y),
                                             "f"(o.z), "f"(o.w)
                                             : "memory");
                        } else {
                            const float2 o = *reinterpret_cast<const float2*>(tb + t * EPI_PITCH + PER * vg);
                            if (whole) *reinterpret_cast<float2*>(dst) = o;
                            else asm volatile("red.global.add.v2.f32 [%0], {%1,%2};" ::"l"(dst), "f"(o.x), "f"(o.y) : "memory");
                        }
                    }
                }
                __syncwarp();
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + buf);
            cur.locate(cur.seg_end, work, prm);
            ++seg;
        }
    }
    // ---- teardown: everyone is done with TMEM before it is freed
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(CF::TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *failed && prm.error_flag) atomicExch(prm.error_flag, 1);
}

// x rows picked by an index list, made contiguous for the tiled copies of the kernel above.
__global__ void gather_rows_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ x,
                                   const int32_t* __restrict__ idx, int64_t M, int K8) {
    const int64_t total = M * K8;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / K8;
        const int c = (int)(i - m * K8);
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(x)[(int64_t)idx[m] * K8 + c];
    }
}

}  // namespace tc2

// --------------------------------------------------------------------------- host side
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool gemm_tma_disabled() {
    static const bool off = [] {
        const char* v = getenv("HQM_GEMM_TMA");
        return v && v[0] == '0';
    }();
    return off;
}

struct WKey {
    const void* q;
    const void* s;
    const void* z;
    int N, K, nbits, group;
    bool operator==(const WKey& o) const {
        return q == o.q && s == o.s && z == o.z && N == o.N && K == o.K && nbits == o.nbits && group == o.group;
    }
};
struct WKeyHash {
    size_t operator()(const WKey& k) const {
        size_t h = reinterpret_cast<uintptr_t>(k.q) * 0x9E3779B97F4A7C15ull;
        h ^= reinterpret_cast<uintptr_t>(k.s) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        h ^= (size_t)k.N * 1315423911u + (size_t)k.K * 2654435761u + (size_t)k.nbits * 97u + (size_t)k.group;
        return h;
    }
};
struct WMaps {
    CUtensorMap m[3];
};

// codes as (K, P, group_size) bytes with box (64, RT, group_size); scale_q / zero_q as (K, G) bytes with box (64, RES)
bool encode_weight_maps(const hqm_weight* w, int G, CUtensorMap* out) {
    EncodeTiledFn enc = (EncodeTiledFn)tma_encode_entry();
    if (!enc) return false;
    const int per = codes_per_word(w->nbits);
    const int rt = 128 / (w->group_size * per);
    const cuuint64_t K = (cuuint64_t)w->K, P = (cuuint64_t)(G / per);
    const cuuint32_t ones[3] = {1, 1, 1};
    {
        const cuuint64_t dims[3] = {K, P, (cuuint64_t)w->group_size};
        const cuuint64_t strides[2] = {K, P * K};
        const cuuint32_t box[3] = {64, (cuuint32_t)rt, (cuuint32_t)w->group_size};
        if (enc(&out[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(w->W_q), dims, strides, box, ones,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    const void* bytes[2] = {w->scale_q, w->zero_q};
    for (int i = 0; i < 2; ++i) {
        const cuuint64_t dims[2] = {K, (cuuint64_t)G};
        const cuuint64_t strides[1] = {K};
        const cuuint32_t box[2] = {64, (cuuint32_t)(rt * per)};
        if (enc(&out[1 + i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(bytes[i]), dims, strides, box, ones,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}

bool cached_weight_maps(const hqm_weight* w, int G, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<WKey, WMaps, WKeyHash> cache;
    const WKey key{w->W_q, w->scale_q, w->zero_q, w->N, w->K, w->nbits, w->group_size};
    std::lock_guard<std::mutex> lock(mu);
    auto itr = cache.find(key);
    if (itr == cache.end()) {
        WMaps tr;
        if (!encode_weight_maps(w, G, tr.m)) return false;
        if (cache.size() > 16384) cache.clear();
        itr = cache.emplace(key, tr).first;
    }
    for (int i = 0; i < 3; ++i) out[i] = itr->second.m[i];
    return true;
}

bool encode_x_map(const uint16_t* x, int64_t rows, int K, int ntok, CUtensorMap* out) {
    EncodeTiledFn enc = (EncodeTiledFn)tma_encode_entry();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)ntok};
    const cuuint32_t ones[2] = {1, 1};
    return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(x), dims, strides, box, ones,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
    static int counts[MAX_DEVICES];
    int& c = counts[current_device_slot()];
    if (c == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
        c = sms;
    }
    return c;
}

template <int NBITS, int NB, int NTOK>
int launch_one(const tc2::Params& p, int grid, cudaStream_t st) {
    using CF = tc2::Cfg<NBITS, NB, NTOK>;
    auto kern = tc2::gemm_tma_kernel<NBITS, NB, NTOK>;
    static bool attr_done[MAX_DEVICES];
    bool& attr_set = attr_done[current_device_slot()];
    if (!attr_set) {
        HQM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CF::SMEM));
        attr_set = true;
    }
    kern<<<grid, CF::NTHREADS, CF::SMEM, st>>>(p);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

template <int NBITS, int NB>
int launch_tokens(const tc2::Params& p, int grid, int ntok, cudaStream_t st) {
    if (ntok == 64) return launch_one<NBITS, NB, 64>(p, grid, st);
    if (ntok == 128) return launch_one<NBITS, NB, 128>(p, grid, st);
    return launch_one<NBITS, NB, 256>(p, grid, st);
}

}  // namespace

bool gemm_tma_supported(const hqm_weight* w, int G, int C, int64_t M) {
    if (gemm_tma_disabled() || tma_encode_entry() == nullptr) return false;
    if (!gemm_tc_supported(w, G, C, M)) return false;
    return C % 64 == 0 && M <= INT32_MAX / 2;
}

int gemm_tma_ntok(int64_t M) { return M <= 64 ? 64 : (M <= 128 ? 128 : 256); }

int launch_gather_rows(uint16_t* dst, const uint16_t* x, const int32_t* idx, int64_t M, int K, cudaStream_t st) {
    const int64_t total = M * (K / 8);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    tc2::gather_rows_kernel<<<(int)(blocks < 1 ? 1 : blocks), 256, 0, st>>>(dst, x, idx, M, K / 8);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

// sums (M, layers*N) fp32 = x . [w0; w1]^T for contiguous rows of x.  The sums are zeroed here first.
int launch_gemm_tma(float* sums, const uint16_t* x, int64_t M, const hqm_weight* w0, const hqm_weight* w1, int G, int C,
                    cudaStream_t st) {
    const int layers = w1 ? 2 : 1;
    const int per = codes_per_word(w0->nbits);
    const int nb = w0->group_size / 16;
    const int rt = 128 / (w0->group_size * per);
    const int ntok = gemm_tma_ntok(M);
    tc2::Params p{};
    if (!encode_x_map(x, M, w0->K, ntok, &p.x_map) || !cached_weight_maps(w0, G, p.w0_map) ||
        !cached_weight_maps(w1 ? w1 : w0, G, p.w1_map)) {
        set_error("gemm_tma: cuTensorMapEncodeTiled failed for a %dx%d %d-bit layer, %lld rows", w0->N, w0->K, w0->nbits,
                  (long long)M);
        return HQM_ERR_CUDA;
    }
    const hqm_weight* ws[2] = {w0, w1 ? w1 : w0};
    for (int l = 0; l < 2; ++l) {
        const uint16_t** mt = l ? p.meta1 : p.meta0;
        mt[0] = ws[l]->ms_scale;
        mt[1] = ws[l]->mz_scale;
        mt[2] = ws[l]->ms_zero;
        mt[3] = ws[l]->mz_zero;
    }
    p.layers = layers;
    p.N = w0->N;
    p.K = w0->K;
    p.C = C;
    p.P = G / per;
    p.tiles_per_layer = p.P / rt;
    p.chunks = (int)((M + ntok - 1) / ntok);
    p.kblocks = w0->K / 64;
    p.items = layers * p.tiles_per_layer * p.chunks;
    p.M_total = (int)M;
    p.sums = sums;
    p.error_flag = tc_error_ptr();
    const int64_t total = (int64_t)p.items * p.kblocks;
    int64_t grid = sm_count();
    if (grid > total / 8) grid = total / 8 < 1 ? 1 : total / 8;
    // tiles that are split between CTAs are completed by additions into zeroed sums
    if (p.items % grid != 0) HQM_CUDA(cudaMemsetAsync(sums, 0, (size_t)M * w0->N * layers * sizeof(float), st));
    if (w0->nbits == 2 && nb == 1) return launch_tokens<2, 1>(p, (int)grid, ntok, st);
    if (w0->nbits == 2 && nb == 2) return launch_tokens<2, 2>(p, (int)grid, ntok, st);
    if (w0->nbits == 4 && nb == 2) return launch_tokens<4, 2>(p, (int)grid, ntok, st);
    if (w0->nbits == 4 && nb == 4) return launch_tokens<4, 4>(p, (int)grid, ntok, st);
    set_error("gemm_tma: no instantiation for nbits=%d group_size=%d", w0->nbits, w0->group_size);
    return HQM_ERR_ARG;
}

}  // namespace hqm

