// Weight-streaming quantized linear for ONE row of x (decode at batch 1), packed tiles staged by TMA:
// the kernel that replaces triton_matmul4_transpose / triton_matmul2_transpose of the reference
// (triton_kernels.py:133-191, 321-380) and the two per-call Quantizer.dequantize launches in front of
// them (custom_layers.py:62-66) where the time goes at decode.
//
// Algebra (as in gemv_stream.cu).  With r = n % G the residue of output row n and j = n / G its position
// inside the quantisation group,
//     y[jG + r] = sum_k (x[k] s[r,k]) q[jG + r, k]  -  sum_k (x[k] s[r,k]) z[r,k],
// so scale and zero are decoded (8 bit -> fp16) once per (r, k) and folded into the activation; per
// weight only the bit-field extraction remains, and mma.sync.m16n8k16 serves as the reduction over k:
// A = 16 group members x 16 columns of one slot (bit field) of the packed bytes, B column s = x*s of slot s.
//
// Mapping.  A pass = 16 members of one storage-row residue (16 storage rows, P*K bytes apart) x 128
// columns: 2 KB of packed codes plus the PER x 128 scale bytes and PER x 128 zero bytes of those columns,
// brought into shared memory by three tiled TMA copies (cp.async.bulk.tensor into this CTA only) that one
// lane each issues and an mbarrier completes.  The codes tile uses the 128-byte swizzle, so that the
// fragment loads (row g, 16-byte chunk 2t+u) touch every bank once.  Passes are numbered
// (residue, member block)-major and cut into equal contiguous ranges, one per CTA of a one-CTA-per-SM
// grid; inside a CTA pass i belongs to warp i % 8, and every warp keeps its next DEPTH passes in flight
// in its own ring of stages (8 warps x 6 stages x 3 KB = 144 KB of copies outstanding per SM).  A warp
// needs no barrier with the other warps until a residue ends: then the 8 warps' fp32 sums are added in
// a fixed order in shared memory and ONE partial row-set per CTA and residue goes to the scratch buffer
// (two or three per output instead of one per warp), which the consumer kernels add up.
//
// In a pass a lane pair-role is fixed by its MMA position (g = lane / 4, t = lane % 4): lanes with g < PER
// decode x*s of slot g for their 16 columns straight into their B fragment, lanes with 4 <= g < 4 + PER
// decode z of slot g - 4 with the same instruction stream into rows 4.. of the correction tile
// (A = [.; z; OFFSET], one extra MMA per 16 columns gives sum xs*z and OFFSET*sum xs).  Nothing is
// exchanged through shared memory inside a pass.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "kernels.cuh"
#include "stream_split.cuh"

namespace hqm {

namespace {

constexpr int WARPS = 8;
constexpr int KC = 128;                    // columns per pass
constexpr int STAGE_BYTES = 3072;          // 2048 codes + 512 scale bytes + 512 zero bytes
constexpr int S_OFF = 2048, Z_OFF = 2560;
constexpr uint32_t WAIT_POLLS = 1u << 20;  // bounded mbarrier wait (each poll may itself block for a while)
constexpr int RED_FLOATS = 64;             // 16 members x up to 4 slots

struct TmaLayerParams {
    const uint16_t* meta[4];               // ms_scale, mz_scale, ms_zero, mz_zero (fp16)
    CUtensorMap maps[3];                   // codes (swizzle 128B), scale_q, zero_q
};

struct TmaParams {
    TmaLayerParams ly[STREAM_MAX_LAYERS];
    int count, nb_log2, K, PT;
    int pr0[STREAM_MAX_LAYERS + 1];        // first (residue, block) unit of each layer
    int col0[STREAM_MAX_LAYERS + 1];
    int G[STREAM_MAX_LAYERS], C[STREAM_MAX_LAYERS];
    int k_mod_c[STREAM_MAX_LAYERS];        // K % C: what the flat scale/zero index of a row advances the meta column by
    int step_mod_c[STREAM_MAX_LAYERS];     // (WARPS * KC) % C: a warp's step from one of its passes to the next
    int xrow[STREAM_MAX_LAYERS], xslot[STREAM_MAX_LAYERS];
    int nx;                                // distinct rows of x
    const StreamEntry* table;
    const int32_t* sel[STREAM_MAX_LAYERS];
    int which[STREAM_MAX_LAYERS];
    int sel_settled;
    uint32_t mask[4], magic[4];            // bit-field extraction constants per slot
    // finishing: units split over several CTAs keep their parts in `inter` ([unit][maxc][64] floats) and count
    // arrivals in `counters` (zero before and after the launch); the last CTA adds the parts in order
    float* inter;
    uint32_t* counters;
    int maxc;
    uint16_t* y_out;                       // when set: the finished row as bf16 (+ bias) instead of fp32 sums
    const uint16_t* bias;
};

struct LayerConst {                        // per layer, in shared memory
    const uint16_t* meta[4];
    const CUtensorMap* maps;
    int C, units, k_mod_c, step_mod_c, xslot, pad;      // units: (residue, block) units of the layer
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t lop_and_or(uint32_t v, uint32_t mask, uint32_t magic) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(v), "r"(mask), "r"(magic));
    return d;
}
__device__ __forceinline__ uint32_t prmt2(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 ldg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) {
    __half2 r = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t h2mul(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_POLLS; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// Tiled 3-D copy global -> shared (this CTA), completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}

// Position of a pass in the launch: layer, unit = (residue, block of 16 members) inside the layer, 128-column chunk.
// A cursor that has run past the end of the launch keeps counting inside the last layer and is never dereferenced.
struct Cursor {
    int layer, unit, p;
    __device__ __forceinline__ void set(uint32_t L, const TmaParams& prm) {
        const int pr = (int)(L / (uint32_t)prm.PT);
        p = (int)(L - (uint32_t)pr * (uint32_t)prm.PT);
        layer = 0;
#pragma unroll
        for (int l = 1; l < STREAM_MAX_LAYERS; ++l) layer += (l < prm.count && pr >= prm.pr0[l]) ? 1 : 0;
        unit = pr - prm.pr0[layer];
    }
    // the next pass; true when it starts another unit
    __device__ __forceinline__ bool next(int PT, const LayerConst* ly, int count) {
        if (++p < PT) return false;
        p = 0;
        if (++unit >= ly[layer].units && layer + 1 < count) {
            unit = 0;
            ++layer;
        }
        return true;
    }
};

constexpr int SEG_SLOTS = 3;               // units a warp's range may touch


template <int NBITS, int DEPTH>
__global__ void __launch_bounds__(WARPS * 32, 2)
gemv_tma_kernel(float* __restrict__ partial, const uint16_t* __restrict__ x, const int32_t* __restrict__ x_idx,
                int m_base, int M_total, const __grid_constant__ TmaParams prm, const Split sp, int* error_flag) {
    constexpr int PER = NBITS == 2 ? 4 : 2;
    constexpr uint32_t TX_BYTES = 2048 + 2 * PER * KC;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ LayerConst s_ly[STREAM_MAX_LAYERS];
    __shared__ int s_first_pr[WARPS + 1];              // unit of each warp's first pass ([WARPS]: unit after the CTA's last)

    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int K = prm.K, PT = prm.PT, NBL = prm.nb_log2;
    const int N_total = prm.col0[prm.count];

    const uint32_t ring = smem_addr(smem + (size_t)wi * DEPTH * STAGE_BYTES);
    __half* x_s = reinterpret_cast<__half*>(smem + (size_t)WARPS * DEPTH * STAGE_BYTES);          // [nx][K]
    __half* ones_s = x_s + (size_t)prm.nx * K;                                                    // 16 halves
    float* red = reinterpret_cast<float*>(ones_s + 16);                                           // [WARPS][SEG_SLOTS][64]
    uint64_t* bars_g = reinterpret_cast<uint64_t*>(red + WARPS * SEG_SLOTS * RED_FLOATS);         // [WARPS][DEPTH]
    const uint32_t bars = smem_addr(bars_g + wi * DEPTH);

    // The kernel behind this one may be made resident right away; this one overlaps the tail of its
    // predecessor until `synced`: weights (and their fp16 meta) are never written inside a chain of
    // launches, so the first copies are requested before the wait; x, the row index, the expert choice
    // and the partial buffer are touched only after it.
    grid_launch_dependents();
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < DEPTH; ++s) mbar_init(bars + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // this warp's contiguous share of the CTA's range
    const uint32_t L0 = sp.begin(blockIdx.x), L1 = sp.begin(blockIdx.x + 1);
    const int n_cta = (int)(L1 - L0);
    const int share = n_cta / WARPS, extra = n_cta - share * WARPS;
    const int my0 = wi * share + (wi < extra ? wi : extra);
    const int n_mine = share + (wi < extra ? 1 : 0);
    Cursor iss;
    iss.set(L0 + (uint32_t)my0, prm);
    int n_issued = 0;
    __syncwarp();
    // ---- copy issue: lanes 0..2 request the codes / scale / zero tile of a pass into stage `st`
    auto issue_at = [&](int st, const CUtensorMap* maps, int unit, int p) {
        if (lane < 3) {
            const int rho = unit >> NBL, b = unit - (rho << NBL);
            const uint32_t stage = ring + (uint32_t)st * STAGE_BYTES;
            const uint32_t bar = bars + 8 * st;
            if (lane == 0) mbar_expect_tx(bar, TX_BYTES);
            const int c1 = lane == 0 ? rho : PER * rho;
            const int c2 = lane == 0 ? 16 * b : 0;
            const uint32_t dst = stage + (lane == 0 ? 0u : (lane == 1 ? (uint32_t)S_OFF : (uint32_t)Z_OFF));
            tma_load_3d(dst, maps + lane, p * KC, c1, c2, bar);
        }
    };
    if (!prm.table) {
        // the tensor maps are kernel parameters: the first copies leave before anything else is set up
        const int n_pro = n_mine < DEPTH ? n_mine : DEPTH;
        for (; n_issued < n_pro; ++n_issued) {
            issue_at(n_issued, prm.ly[iss.layer].maps, iss.unit, iss.p);
            if (++iss.p == PT) {
                iss.p = 0;
                if (++iss.unit >= prm.pr0[iss.layer + 1] - prm.pr0[iss.layer] && iss.layer + 1 < prm.count) {
                    iss.unit = 0;
                    ++iss.layer;
                }
            }
        }
    }
    bool synced = false;
    if (prm.table && !prm.sel_settled) {
        grid_dependency_wait();
        synced = true;
    }
    if ((int)threadIdx.x < prm.count) {
        const int l = threadIdx.x;
        LayerConst c;
        if (prm.table) {
            const StreamEntry* e = prm.table + 3 * __ldcg(prm.sel[l]) + prm.which[l];
            c.meta[0] = e->w.ms_scale;
            c.meta[1] = e->w.mz_scale;
            c.meta[2] = e->w.ms_zero;
            c.meta[3] = e->w.mz_zero;
            c.maps = reinterpret_cast<const CUtensorMap*>(e->maps);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) c.meta[i] = prm.ly[l].meta[i];
            c.maps = prm.ly[l].maps;
        }
        c.C = prm.C[l];
        c.units = prm.pr0[l + 1] - prm.pr0[l];
        c.k_mod_c = prm.k_mod_c[l];
        c.step_mod_c = 0;
        c.xslot = prm.xslot[l];
        c.pad = 0;
        s_ly[l] = c;
    }
    if (threadIdx.x < 16) ones_s[threadIdx.x] = __float2half(1.f);
    if (lane == 0) {
        s_first_pr[wi] = (int)((L0 + (uint32_t)my0) / (uint32_t)PT);
        if (wi == 0) s_first_pr[WARPS] = (int)((L1 + (uint32_t)PT - 1) / (uint32_t)PT);
    }
    __syncthreads();
    auto issue = [&](int st) {
        issue_at(st, s_ly[iss.layer].maps, iss.unit, iss.p);
        iss.next(PT, s_ly, prm.count);
    };
    if (prm.table) {
        if (lane < 3) {
            // tensor maps that live in global memory: make them visible to the copy engine's proxy
            for (int l = 0; l < prm.count; ++l) {
                const void* m = s_ly[l].maps + lane;
                asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(m) : "memory");
            }
        }
        const int n_pro = n_mine < DEPTH ? n_mine : DEPTH;
        for (; n_issued < n_pro; ++n_issued) issue(n_issued);
    }

    // ---- roles
    const bool isz = g >= 4;
    const int slot = ((g & 3) < PER) ? (g & 3) : 0;
    // fp16 pair holding the OFFSET of slot g & 3 (the constant the bit field of that slot is OR-ed into)
    uint32_t off_h2;
    if (NBITS == 2) {
        const int s4 = g & 3;
        off_h2 = s4 == 0 ? 0x4C004C00u : (s4 == 1 ? 0x54005400u : (s4 == 2 ? 0x5C005C00u : 0x64006400u));
    } else {
        off_h2 = (g & 1) == 0 ? 0x54005400u : 0x64006400u;
    }
    const uint32_t cdoff = (uint32_t)(g * 128);                      // row g of the codes tile (row g + 8: + 1024)
    const uint32_t bytes_off = (uint32_t)((isz ? Z_OFF : S_OFF) + slot * KC + 32 * t);
    const uint32_t ch0 = cdoff + (uint32_t)(((2 * t) ^ g) << 4), ch1 = cdoff + (uint32_t)(((2 * t + 1) ^ g) << 4);

    // ---- meta (fp16 scale / zero of the 8-bit scale and zero bytes; L2 resident) goes through registers, requested a
    // whole pass ahead: a half's registers are reloaded for the next pass as soon as that half has been consumed.
    // The meta column of (row r, column k) is (r * K + k) % C; tracked incrementally.
    Cursor cur;
    cur.set(L0 + (uint32_t)my0, prm);
    const uint16_t* ms_p = nullptr;
    const uint16_t* mz_p = nullptr;
    uint32_t mcol = 0;                     // meta column of this lane's row at the first column of the pass `cur`
    int curC = 1, kmodC = 0;
    auto bind = [&](const Cursor& c) {     // from scratch (launch start, or after crossing into another layer)
        const LayerConst& lc = s_ly[c.layer];
        ms_p = lc.meta[isz ? 2 : 0] + 32 * t;
        mz_p = lc.meta[isz ? 3 : 1] + 32 * t;
        curC = lc.C;
        kmodC = lc.k_mod_c;
        const int rho = c.unit >> NBL;
        const uint64_t flat = (uint64_t)(PER * rho + slot) * (uint64_t)K + (uint64_t)(c.p * KC);
        mcol = (uint32_t)(flat % (uint64_t)curC);
    };
    uint4 ms0[2], mz0[2], ms1[2], mz1[2];  // halves 0 / 1 of a pass
    if (n_mine > 0) {
        bind(cur);
        ms0[0] = ldg128(ms_p + mcol);
        ms0[1] = ldg128(ms_p + mcol + 8);
        mz0[0] = ldg128(mz_p + mcol);
        mz0[1] = ldg128(mz_p + mcol + 8);
        ms1[0] = ldg128(ms_p + mcol + 16);
        ms1[1] = ldg128(ms_p + mcol + 24);
        mz1[0] = ldg128(mz_p + mcol + 16);
        mz1[1] = ldg128(mz_p + mcol + 24);
    }

    if (!synced) grid_dependency_wait();
    // ---- x as fp16 in shared memory
    {
        const int row0 = x_idx ? x_idx[m_base] : m_base;
        for (int s = 0; s < prm.nx; ++s) {
            int xr = 0;
#pragma unroll
            for (int l = 0; l < STREAM_MAX_LAYERS; ++l)
                if (l < prm.count && prm.xslot[l] == s) xr = prm.xrow[l];
            const uint16_t* src = x + (int64_t)(row0 + xr) * K;
            for (int i = threadIdx.x * 8; i < K; i += WARPS * 32 * 8) {
                const uint4 v = *reinterpret_cast<const uint4*>(src + i);
                const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 h = __floats2half2_rn(__uint_as_float(w4[j] << 16), __uint_as_float(w4[j] & 0xffff0000u));
                    o[j] = *reinterpret_cast<const uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(x_s + (size_t)s * K + i) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
    __syncthreads();

    const uint32_t m0 = prm.mask[0], m1 = prm.mask[1], m2 = prm.mask[2], m3 = prm.mask[3];
    const uint32_t k0c = prm.magic[0], k1c = prm.magic[1], k2c = prm.magic[2], k3c = prm.magic[3];
    const uint32_t ones_a = smem_addr(ones_s);
    const uint32_t xs_a = smem_addr(x_s) + (uint32_t)(64 * t);       // this lane's 32 columns (2 x 16) of a pass: + 32 * u

    float acc[PER][4];
    float accc[4];
#pragma unroll
    for (int s = 0; s < PER; ++s)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[s][v] = 0.f;
#pragma unroll
    for (int v = 0; v < 4; ++v) accc[v] = 0.f;

    // one 64-column half of a pass: decode this lane's 16 scale (or zero) values, 4 k-steps of MMAs
    auto half_pass = [&](const uint4& q0, const uint4& q1, const uint4& bq, const uint4& xa, const uint4& xb,
                         const uint4 (&ms)[2], const uint4 (&mz)[2]) {
        const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w};
        const uint32_t msr[8] = {ms[0].x, ms[0].y, ms[0].z, ms[0].w, ms[1].x, ms[1].y, ms[1].z, ms[1].w};
        const uint32_t mzr[8] = {mz[0].x, mz[0].y, mz[0].z, mz[0].w, mz[1].x, mz[1].y, mz[1].z, mz[1].w};
        const uint32_t xr[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w};
        const uint32_t w1[4] = {q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
            // (q - mz) * ms (* x): columns 4wd .. 4wd+3 of this lane's 16
            uint32_t n0 = h2sub(prmt2(bw[wd], 0x64646464u, 0x4140u), 0x64006400u);
            uint32_t n1 = h2sub(prmt2(bw[wd], 0x64646464u, 0x4342u), 0x64006400u);
            n0 = h2mul(h2mul(h2sub(n0, mzr[2 * wd]), msr[2 * wd]), xr[2 * wd]);
            n1 = h2mul(h2mul(h2sub(n1, mzr[2 * wd + 1]), msr[2 * wd + 1]), xr[2 * wd + 1]);
            const uint32_t r0 = prmt2(n0, n1, 0x5410u);      // columns (0, 2)
            const uint32_t r1 = prmt2(n0, n1, 0x7632u);      // columns (1, 3)
            const uint32_t u0 = w0[wd], u1 = w1[wd], u0s = u0 >> 8, u1s = u1 >> 8;
            mma16816(acc[0], lop_and_or(u0, m0, k0c), lop_and_or(u1, m0, k0c), lop_and_or(u0s, m0, k0c),
                     lop_and_or(u1s, m0, k0c), r0, r1);
            mma16816(acc[1], lop_and_or(u0, m1, k1c), lop_and_or(u1, m1, k1c), lop_and_or(u0s, m1, k1c),
                     lop_and_or(u1s, m1, k1c), r0, r1);
            if constexpr (PER == 4) {
                mma16816(acc[PER - 2], lop_and_or(u0, m2, k2c), lop_and_or(u1, m2, k2c), lop_and_or(u0s, m2, k2c),
                         lop_and_or(u1s, m2, k2c), r0, r1);
                mma16816(acc[PER - 1], lop_and_or(u0, m3, k3c), lop_and_or(u1, m3, k3c), lop_and_or(u0s, m3, k3c),
                         lop_and_or(u1s, m3, k3c), r0, r1);
            }
            mma16816(accc, r0, off_h2, r1, off_h2, r0, r1);
        }
    };

    // the sums of the unit this warp has been working on -> its next slot of the reduction buffer
    int n_flushed = 0;
    auto flush = [&]() {
        const float mine_z = (g & 1) ? accc[1] : accc[0];        // valid in lane (4 + s, s / 2): sum xs*z of slot s
        const float mine_o = (g & 1) ? accc[3] : accc[2];        // valid in lane (s, s / 2): OFFSET_s * sum xs
        const int sa = (2 * t) % PER;
        const float ca = __shfl_sync(0xffffffffu, mine_z, (4 + sa) * 4 + t) + __shfl_sync(0xffffffffu, mine_o, sa * 4 + t);
        const float cb = __shfl_sync(0xffffffffu, mine_z, (5 + sa) * 4 + t) + __shfl_sync(0xffffffffu, mine_o, (sa + 1) * 4 + t);
        float* mine = red + (wi * SEG_SLOTS + n_flushed) * RED_FLOATS;
        if (t < PER / 2) {
            float va0, va1, vb0, vb1;
            if (PER == 4 && t == 1) {
                va0 = acc[PER - 2][0]; vb0 = acc[PER - 1][1]; va1 = acc[PER - 2][2]; vb1 = acc[PER - 1][3];
            } else {
                va0 = acc[0][0]; vb0 = acc[1][1]; va1 = acc[0][2]; vb1 = acc[1][3];
            }
            *reinterpret_cast<float2*>(mine + g * PER + sa) = make_float2(va0 - ca, vb0 - cb);
            *reinterpret_cast<float2*>(mine + (g + 8) * PER + sa) = make_float2(va1 - ca, vb1 - cb);
        }
        ++n_flushed;
#pragma unroll
        for (int s = 0; s < PER; ++s)
#pragma unroll
            for (int v = 0; v < 4; ++v) acc[s][v] = 0.f;
#pragma unroll
        for (int v = 0; v < 4; ++v) accc[v] = 0.f;
    };

    // ---- this warp's passes
    int st = 0;                            // stage of the pass being computed
    uint32_t parity = 0;                   // bit s: phase parity the next wait on stage s expects
    bool dead = false;
    for (int it = 0; it < n_mine; ++it) {
        const uint32_t stage = ring + (uint32_t)st * STAGE_BYTES;
        const uint32_t xs_base = isz ? ones_a : xs_a + (uint32_t)((s_ly[cur.layer].xslot * K + cur.p * KC) * 2);
        const uint32_t xstep = isz ? 0u : 32u, xhalf = isz ? 0u : 16u;
        {
            const bool ok = mbar_wait(bars + 8 * st, (parity >> st) & 1u);
            if (!__all_sync(0xffffffffu, ok)) {      // give up as a warp: the rest of the range is skipped
                dead = true;
                if (lane == 0 && error_flag) atomicExch(error_flag, 1);
                break;
            }
        }
        parity ^= 1u << st;
        // where the next pass is, and the meta column of this lane's row there
        const bool last = it + 1 == n_mine;
        const int old_layer = cur.layer, old_rho = cur.unit >> NBL;
        const bool new_unit = cur.next(PT, s_ly, prm.count);
        uint32_t ncol = mcol + (uint32_t)KC;
        if (new_unit && !last) {
            if (cur.layer != old_layer) {
                bind(cur);
                ncol = mcol;
            } else {
                // wrapped around K (flat index - K), possibly into the next residue (flat index + PER * K)
                const uint32_t kc = (uint32_t)kmodC;
                ncol += ((uint32_t)curC - kc) + (((cur.unit >> NBL) != old_rho) ? PER * kc : 0u);
            }
        }
        if (ncol >= (uint32_t)curC) {
            ncol -= (uint32_t)curC;
            while (ncol >= (uint32_t)curC) ncol -= (uint32_t)curC;
        }
        mcol = ncol;

        uint4 q0 = lds128(stage + ch0), q1 = lds128(stage + 1024 + ch0);
        uint4 bq = lds128(stage + bytes_off);
        uint4 xa = lds128(xs_base), xb = lds128(xs_base + xhalf);
        half_pass(q0, q1, bq, xa, xb, ms0, mz0);
        if (!last) {                                 // this half's registers: the next pass's first half
            ms0[0] = ldg128(ms_p + mcol);
            ms0[1] = ldg128(ms_p + mcol + 8);
            mz0[0] = ldg128(mz_p + mcol);
            mz0[1] = ldg128(mz_p + mcol + 8);
        }
        q0 = lds128(stage + ch1);
        q1 = lds128(stage + 1024 + ch1);
        bq = lds128(stage + bytes_off + 16);
        xa = lds128(xs_base + xstep);
        xb = lds128(xs_base + xstep + xhalf);
        __syncwarp();
        // the stage is free again: request the pass DEPTH ahead into it
        if (n_issued < n_mine) {
            issue(st);
            ++n_issued;
        }
        half_pass(q0, q1, bq, xa, xb, ms1, mz1);
        if (!last) {
            ms1[0] = ldg128(ms_p + mcol + 16);
            ms1[1] = ldg128(ms_p + mcol + 24);
            mz1[0] = ldg128(mz_p + mcol + 16);
            mz1[1] = ldg128(mz_p + mcol + 24);
        }
        st = (st + 1 == DEPTH) ? 0 : st + 1;
        if (new_unit || last) flush();
    }
    if (dead) {
        // copies may still be in flight towards this CTA's shared memory: give them time before leaving;
        // the unit being worked on is flushed as it is so that the reduction below reads defined values
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        while (n_flushed < SEG_SLOTS) flush();
    }
    __syncthreads();

    // ---- the CTA's units: each is summed over the warps that touched it, in warp order, by one warp.  A unit
    // that other CTAs share is finished by whichever of them arrives last: it adds the CTAs' parts in CTA order.
    {
        const int pr_first = s_first_pr[0], pr_end = s_first_pr[WARPS];
        for (int pr = pr_first + wi; pr < pr_end; pr += WARPS) {
            const bool active = lane < 16 * PER / 2;
            float2 v = make_float2(0.f, 0.f);
            if (active) {
                for (int w = 0; w < WARPS; ++w) {
                    const int k = pr - s_first_pr[w];                       // slot of this unit in warp w's buffer
                    const int n_w = share + (w < extra ? 1 : 0);
                    if (k < 0 || n_w == 0) continue;
                    const int w0p = w * share + (w < extra ? w : extra);
                    const int last_pr = (int)((L0 + (uint32_t)(w0p + n_w - 1)) / (uint32_t)PT);
                    if (pr > last_pr) continue;
                    const float2 a = *reinterpret_cast<const float2*>(red + (w * SEG_SLOTS + k) * RED_FLOATS + 2 * lane);
                    v.x += a.x;
                    v.y += a.y;
                }
            }
            const int c_first = sp.owner((uint32_t)pr * (uint32_t)PT);
            const int c_last = sp.owner((uint32_t)pr * (uint32_t)PT + (uint32_t)PT - 1u);
            const int n_parts = c_last - c_first + 1;
            bool finish = true;
            if (n_parts > 1) {
                float* parts = prm.inter + ((size_t)pr * prm.maxc) * RED_FLOATS + 2 * lane;
                if (active) __stcg(reinterpret_cast<float2*>(parts + ((int)blockIdx.x - c_first) * RED_FLOATS), v);
                __threadfence();
                __syncwarp();
                unsigned int arrived = 0;
                if (lane == 0) arrived = atomicAdd(prm.counters + pr, 1u);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                finish = arrived == (unsigned int)(n_parts - 1);
                // a count that cannot occur: the header of the scratch buffer was not zero when the launch began
                if (arrived >= (unsigned int)n_parts && lane == 0 && error_flag) atomicExch(error_flag, 3);
                if (finish) {
                    __threadfence();
                    v = make_float2(0.f, 0.f);
                    if (active) {
                        for (int c = 0; c < n_parts; ++c) {
                            const float2 a = __ldcg(reinterpret_cast<const float2*>(parts + c * RED_FLOATS));
                            v.x += a.x;
                            v.y += a.y;
                        }
                    }
                    if (lane == 0) prm.counters[pr] = 0u;                    // ready for the next launch
                }
            }
            if (finish && active) {
                int layer = 0;
#pragma unroll
                for (int l = 1; l < STREAM_MAX_LAYERS; ++l) layer += (l < prm.count && pr >= prm.pr0[l]) ? 1 : 0;
                const int unit = pr - prm.pr0[layer];
                const int rho = unit >> NBL, b = unit - (rho << NBL);
                const int j = (2 * lane) / PER, s = (2 * lane) % PER;
                const int64_t col = prm.col0[layer] + (int64_t)(16 * b + j) * prm.G[layer] + PER * rho + s;
                if (prm.y_out) {
                    if (prm.bias) {
                        v.x += bf16_bits_to_float(prm.bias[col]);
                        v.y += bf16_bits_to_float(prm.bias[col + 1]);
                    }
                    const uint32_t packed = (uint32_t)float_to_bf16_bits(v.x) | ((uint32_t)float_to_bf16_bits(v.y) << 16);
                    *reinterpret_cast<uint32_t*>(prm.y_out + (int64_t)m_base * N_total + col) = packed;
                } else {
                    *reinterpret_cast<float2*>(partial + (int64_t)m_base * N_total + col) = v;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return (EncodeTiledFn) nullptr;
        }
        return (EncodeTiledFn)p;
    }();
    return fn;
}

bool tma_shape_ok(const hqm_weight* w, int G, int C) {
    if ((w->nbits != 2 && w->nbits != 4) || !meta_uniform(w)) return false;
    const int per = codes_per_word(w->nbits);
    if (w->group_size % 16 != 0 || w->K % KC != 0 || C % KC != 0 || G % per != 0) return false;
    if (w->group_size > 256 || (int64_t)G * w->K >= ((int64_t)1 << 31)) return false;
    auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    return a16(w->W_q) && a16(w->scale_q) && a16(w->zero_q) && a16(w->ms_scale) && a16(w->mz_scale) && a16(w->ms_zero) &&
           a16(w->mz_zero);
}

// The three tensor maps of a layer: codes as (K, P, group_size) bytes with box (128, 1, 16) and the 128-byte
// swizzle; scale_q and zero_q as (K, G, 1) bytes with box (128, PER, 1).
bool encode_maps(const hqm_weight* w, int G, CUtensorMap* out) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const int per = codes_per_word(w->nbits);
    const cuuint64_t K = (cuuint64_t)w->K, P = (cuuint64_t)(G / per);
    const cuuint32_t ones[3] = {1, 1, 1};
    {
        const cuuint64_t dims[3] = {K, P, (cuuint64_t)w->group_size};
        const cuuint64_t strides[2] = {K, P * K};
        const cuuint32_t box[3] = {(cuuint32_t)KC, 1, 16};
        if (enc(&out[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(w->W_q), dims, strides, box, ones,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    const void* bytes[2] = {w->scale_q, w->zero_q};
    for (int i = 0; i < 2; ++i) {
        const cuuint64_t dims[3] = {K, (cuuint64_t)G, 1};
        const cuuint64_t strides[2] = {K, (cuuint64_t)G * K};
        const cuuint32_t box[3] = {(cuuint32_t)KC, (cuuint32_t)per, 1};
        if (enc(&out[1 + i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(bytes[i]), dims, strides, box, ones,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}

struct MapKey {
    const void* q;
    const void* s;
    const void* z;
    int N, K, nbits, group;
    bool operator==(const MapKey& o) const {
        return q == o.q && s == o.s && z == o.z && N == o.N && K == o.K && nbits == o.nbits && group == o.group;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<uintptr_t>(k.q) * 0x9E3779B97F4A7C15ull;
        h ^= reinterpret_cast<uintptr_t>(k.s) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        h ^= (size_t)k.N * 1315423911u + (size_t)k.K * 2654435761u + (size_t)k.nbits * 97u + (size_t)k.group;
        return h;
    }
};
struct MapTriple {
    CUtensorMap m[3];
};

// Tensor maps of a layer, encoded once per (pointers, shape) and kept (encoding is host-only work, but not free).
bool cached_maps(const hqm_weight* w, int G, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, MapTriple, MapKeyHash> cache;
    const MapKey key{w->W_q, w->scale_q, w->zero_q, w->N, w->K, w->nbits, w->group_size};
    std::lock_guard<std::mutex> lock(mu);
    auto itr = cache.find(key);
    if (itr == cache.end()) {
        MapTriple tr;
        if (!encode_maps(w, G, tr.m)) return false;
        if (cache.size() > 16384) cache.clear();
        itr = cache.emplace(key, tr).first;
    }
    for (int i = 0; i < 3; ++i) out[i] = itr->second.m[i];
    return true;
}

size_t tma_smem_bytes(int depth, int nx, int K) {
    return (size_t)WARPS * depth * STAGE_BYTES + (size_t)nx * K * 2 + 32 + (size_t)WARPS * SEG_SLOTS * RED_FLOATS * 4 +
           (size_t)WARPS * depth * 8;
}
// Stages per warp and CTAs per SM: two CTAs per SM (so that the CTAs of the next launch of a chain find room while
// this one is still running) with 3 or 2 stages when the staged rows of x leave room, else one CTA with up to 6.
int tma_depth(int nx, int K, int* ctas_per_sm) {
    for (int d = 3; d >= 2; --d)
        if (tma_smem_bytes(d, nx, K) + 1024 <= 113 * 1024) {
            if (ctas_per_sm) *ctas_per_sm = 2;
            return d;
        }
    for (int d = 6; d >= 2; --d)
        if (tma_smem_bytes(d, nx, K) <= 227 * 1024) {
            if (ctas_per_sm) *ctas_per_sm = 1;
            return d;
        }
    return 0;
}

int distinct_xrows(const int* xrow, int count, int* xslot) {
    int nx = 0, seen[STREAM_MAX_LAYERS];
    for (int l = 0; l < count; ++l) {
        int s = -1;
        for (int i = 0; i < nx; ++i)
            if (seen[i] == xrow[l]) s = i;
        if (s < 0) {
            seen[nx] = xrow[l];
            s = nx++;
        }
        if (xslot) xslot[l] = s;
    }
    return nx;
}

// 0: never; 1: launches of a single layer that finish their row themselves (hqm_linear, hqm_expert_ffn); 2: every
// single-row launch, the decode step's multi-layer and table-driven ones included.  HQM_TMA in the environment
// gives the initial value (default 1); hqm_set_tma_mode changes it.
std::atomic<int> g_tma_mode{-1};
int tma_mode() {
    int v = g_tma_mode.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = getenv("HQM_TMA");
        v = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
        g_tma_mode.store(v, std::memory_order_relaxed);
    }
    return v;
}
bool tma_disabled() { return tma_mode() == 0; }

template <int NBITS, int DEPTH>
bool prepare_kernel(size_t smem) {
    static size_t configured[MAX_DEVICES];
    size_t& have = configured[current_device_slot()];
    if (have >= smem) return true;
    if (cudaFuncSetAttribute(gemv_tma_kernel<NBITS, DEPTH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    have = smem;
    return true;
}

}  // namespace

// cuTensorMapEncodeTiled of the installed driver (null when it cannot be had), for the other TMA users.
void* tma_encode_entry() { return (void*)encode_fn(); }

// Plans one TMA-staged launch over up to four layers for ONE row of x; false when the shapes are outside it
// (the caller then falls back to gemv_stream.cu's kernel).
size_t gemv_tma_scratch_bytes(const StreamPlan& plan, int64_t M) {
    const size_t sums = ((size_t)M * (size_t)plan.col0[plan.count] * sizeof(float) + 255) / 256 * 256;
    return sums + (size_t)plan.rho0[plan.count] * (size_t)plan.slots * RED_FLOATS * sizeof(float);
}

bool gemv_tma_plan(const hqm_weight* const* ws, int count, bool chained, StreamPlan* plan) {
    if (count < 1 || count > STREAM_MAX_LAYERS || tma_disabled() || encode_fn() == nullptr) return false;
    if ((chained || count > 1) && tma_mode() < 2) return false;
    const hqm_weight* w = ws[0];
    const int per = codes_per_word(w->nbits);
    const int nb = w->group_size / 16;
    if (nb < 1 || (nb & (nb - 1)) != 0) return false;          // blocks per residue: a power of two
    plan->count = count;
    plan->rho0[0] = 0;
    plan->col0[0] = 0;
    for (int l = 0; l < count; ++l) {
        const hqm_weight* v = ws[l];
        int G, C;
        if (check_weight(v, &G, &C) != HQM_OK) return false;
        if (v->nbits != w->nbits || v->group_size != w->group_size || v->K != w->K || v->meta_group != w->meta_group)
            return false;
        if (!tma_shape_ok(v, G, C)) return false;
        plan->G[l] = G;
        plan->C[l] = C;
        plan->rho0[l + 1] = plan->rho0[l] + (G / per) * nb;
        plan->col0[l + 1] = plan->col0[l] + v->N;
    }
    plan->nbits = w->nbits;
    plan->nb = nb;
    plan->PT = w->K / KC;
    const int64_t total = (int64_t)plan->rho0[count] * plan->PT;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // worst case two distinct rows of x per launch (the two experts' down projections)
    int per_sm = 1;
    if (tma_depth(count > 1 ? 2 : 1, w->K, &per_sm) == 0) return false;
    int64_t grid = total / WARPS;                  // at least one pass per warp
    if (grid > (int64_t)per_sm * sms) grid = (int64_t)per_sm * sms;
    if (grid < 1) grid = 1;
    if (total < grid || total * grid >= ((int64_t)1 << 31)) return false;
    if ((size_t)plan->rho0[count] * sizeof(uint32_t) > SCRATCH_HEADER) return false;      // one arrival counter per unit
    // a warp's contiguous share of a CTA's range may touch at most SEG_SLOTS units
    if (((total + grid - 1) / grid + WARPS - 1) / WARPS > (int64_t)(SEG_SLOTS - 1) * plan->PT) return false;
    plan->grid = (int)grid;
    plan->warps = (int)grid;                       // the units the passes are split over are CTAs here
    plan->toks = 1;
    const int64_t min_range = total / grid;
    plan->slots = (int)((plan->PT + min_range - 1) / min_range) + 1;
    plan->tma = 1;
    return true;
}

int launch_gemv_tma(float* partial, const uint16_t* x, const int32_t* x_idx, int64_t M, const StreamJob& job,
                    const StreamPlan& plan, cudaStream_t st) {
    TmaParams prm{};
    prm.count = plan.count;
    prm.nb_log2 = 0;
    while ((1 << prm.nb_log2) < plan.nb) ++prm.nb_log2;
    prm.K = job.w[0]->K;
    prm.PT = plan.PT;
    int xrow[STREAM_MAX_LAYERS] = {0, 0, 0, 0};
    for (int l = 0; l < plan.count; ++l) {
        const hqm_weight* w = job.w[l];
        prm.pr0[l] = plan.rho0[l];
        prm.col0[l] = plan.col0[l];
        prm.G[l] = plan.G[l];
        prm.C[l] = plan.C[l];
        prm.k_mod_c[l] = prm.K % plan.C[l];
        prm.step_mod_c[l] = (WARPS * KC) % plan.C[l];
        prm.xrow[l] = xrow[l] = job.xrow[l];
        prm.sel[l] = job.sel[l];
        prm.which[l] = job.which[l];
        if (!job.table) {
            prm.ly[l].meta[0] = w->ms_scale;
            prm.ly[l].meta[1] = w->mz_scale;
            prm.ly[l].meta[2] = w->ms_zero;
            prm.ly[l].meta[3] = w->mz_zero;
            if (!cached_maps(w, plan.G[l], prm.ly[l].maps)) {
                set_error("gemv_tma: cuTensorMapEncodeTiled failed for a %dx%d %d-bit layer", w->N, w->K, w->nbits);
                return HQM_ERR_CUDA;
            }
        }
    }
    prm.pr0[plan.count] = plan.rho0[plan.count];
    prm.col0[plan.count] = plan.col0[plan.count];
    prm.nx = distinct_xrows(xrow, plan.count, prm.xslot);
    prm.table = reinterpret_cast<const StreamEntry*>(job.table);
    prm.sel_settled = job.sel_settled;
    prm.inter = partial + ((size_t)M * (size_t)plan.col0[plan.count] * sizeof(float) + 255) / 256 * 256 / sizeof(float);
    prm.counters = job.counters;
    prm.maxc = plan.slots;
    prm.y_out = job.y_out;
    prm.bias = job.bias;
    if (job.counters == nullptr) {
        set_error("gemv_tma: the launch needs the zeroed header of a scratch buffer");
        return HQM_ERR_SCRATCH;
    }
    if (plan.nbits == 2) {
        const uint32_t mk[4] = {0x00C000C0u, 0x00300030u, 0x000C000Cu, 0x00030003u};
        const uint32_t mg[4] = {0x4C004C00u, 0x54005400u, 0x5C005C00u, 0x64006400u};
        for (int i = 0; i < 4; ++i) {
            prm.mask[i] = mk[i];
            prm.magic[i] = mg[i];
        }
    } else {
        prm.mask[0] = 0x00F000F0u;
        prm.magic[0] = 0x54005400u;
        prm.mask[1] = 0x000F000Fu;
        prm.magic[1] = 0x64006400u;
    }
    // (the plan sized the grid for the worst case of two rows of x; with one row the ring may be deeper)
    int per_sm = 1;
    int depth = tma_depth(plan.count > 1 ? 2 : 1, prm.K, &per_sm);
    if (depth == 0 || prm.nx > 2) {
        set_error("gemv_tma: %d rows of x with K = %d do not fit shared memory", prm.nx, prm.K);
        return HQM_ERR_ARG;
    }
    const size_t smem = tma_smem_bytes(depth, prm.nx, prm.K);
    const Split sp = work_split_of(plan);
    auto go = [&](auto kern, bool ready) -> int {
        if (!ready) {
            set_error("gemv_tma: cannot configure %zu bytes of shared memory", smem);
            return HQM_ERR_CUDA;
        }
        for (int m = 0; m < (int)M; ++m) {
            launch_overlapped(kern, plan.grid, WARPS * 32, smem, st, partial, x, x_idx, m, (int)M, prm, sp, tc_error_ptr());
            HQM_LAUNCH_CHECK();
        }
        return HQM_OK;
    };
#define HQM_TMA_CASE(B, D) \
    if (plan.nbits == B && depth == D) return go(gemv_tma_kernel<B, D>, prepare_kernel<B, D>(smem));
    HQM_TMA_CASE(2, 2) HQM_TMA_CASE(2, 3) HQM_TMA_CASE(2, 4) HQM_TMA_CASE(2, 5) HQM_TMA_CASE(2, 6)
    HQM_TMA_CASE(4, 2) HQM_TMA_CASE(4, 3) HQM_TMA_CASE(4, 4) HQM_TMA_CASE(4, 5) HQM_TMA_CASE(4, 6)
#undef HQM_TMA_CASE
    set_error("gemv_tma: no kernel for %d bits with %d stages", plan.nbits, depth);
    return HQM_ERR_ARG;
}

}  // namespace hqm

extern "C" {

int hqm_set_tma_mode(int mode) {
    const int prev = hqm::tma_mode();
    if (mode >= 0 && mode <= 2) hqm::g_tma_mode.store(mode, std::memory_order_relaxed);
    return prev;
}

size_t hqm_expert_table_bytes(int32_t n_weights) {
    return n_weights > 0 ? (size_t)n_weights * sizeof(hqm::StreamEntry) : 0;
}

int hqm_expert_table_build(void* host_out, const hqm_weight* weights, int32_t n_weights) {
    using namespace hqm;
    HQM_CHECK_ARG(host_out && weights && n_weights > 0, "expert_table_build: null pointer or no weights");
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(host_out) & 63u) == 0, "expert_table_build: the buffer must be 64-byte aligned");
    StreamEntry* out = static_cast<StreamEntry*>(host_out);
    for (int i = 0; i < n_weights; ++i) {
        memset(&out[i], 0, sizeof(StreamEntry));
        out[i].w = weights[i];
        int G, C;
        const int rc = check_weight(&weights[i], &G, &C);
        if (rc != HQM_OK) return rc;
        if (!tma_disabled() && encode_fn() != nullptr && tma_shape_ok(&weights[i], G, C) &&
            !encode_maps(&weights[i], G, reinterpret_cast<CUtensorMap*>(out[i].maps))) {
            set_error("expert_table_build: cuTensorMapEncodeTiled failed for weight %d (%dx%d, %d bit)", i, weights[i].N,
                      weights[i].K, weights[i].nbits);
            return HQM_ERR_CUDA;
        }
    }
    return HQM_OK;
}

}  // extern "C"
