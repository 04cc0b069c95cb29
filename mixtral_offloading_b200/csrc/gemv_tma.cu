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

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "kernels.cuh"
#include "stream_split.cuh"

namespace hqm {

namespace {

constexpr int WARPS = 8;
constexpr int DEPTH = 6;
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
    int count, nb, K, PT;
    int pr0[STREAM_MAX_LAYERS + 1];        // first (residue, block) unit of each layer
    int col0[STREAM_MAX_LAYERS + 1];
    int G[STREAM_MAX_LAYERS], C[STREAM_MAX_LAYERS];
    int xrow[STREAM_MAX_LAYERS], xslot[STREAM_MAX_LAYERS];
    int nx;                                // distinct rows of x
    const StreamEntry* table;
    const int32_t* sel[STREAM_MAX_LAYERS];
    int which[STREAM_MAX_LAYERS];
    int sel_settled;
    uint32_t mask[4], magic[4];            // bit-field extraction constants per slot
};

struct LayerConst {                        // per layer, in shared memory
    const uint16_t* meta[4];
    const CUtensorMap* maps;
    int G, C, pr0, col0, xslot, pad;
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
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
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

// Position of a pass in the launch: layer, residue, member block, 128-column chunk.
struct Cursor {
    int layer, pl, p;                      // pl: (residue, block) unit inside the layer
    __device__ __forceinline__ void set(uint32_t L, const TmaParams& prm) {
        const int pr = (int)(L / (uint32_t)prm.PT);
        p = (int)(L - (uint32_t)pr * (uint32_t)prm.PT);
        layer = 0;
#pragma unroll
        for (int l = 1; l < STREAM_MAX_LAYERS; ++l) layer += (l < prm.count && pr >= prm.pr0[l]) ? 1 : 0;
        pl = pr - prm.pr0[layer];
    }
    // advance by `n` passes (n <= PT); returns true when the unit changed
    __device__ __forceinline__ bool advance(int n, const TmaParams& prm) {
        p += n;
        if (p < prm.PT) return false;
        p -= prm.PT;
        ++pl;
        if (layer + 1 < prm.count && pl >= prm.pr0[layer + 1] - prm.pr0[layer]) {
            pl = 0;
            ++layer;
        }                                  // (a cursor past the end of the launch is never dereferenced)
        return true;
    }
};

template <int NBITS>
__global__ void __launch_bounds__(WARPS * 32, 1)
gemv_tma_kernel(float* __restrict__ partial, const uint16_t* __restrict__ x, const int32_t* __restrict__ x_idx,
                int m_base, int M_total, const __grid_constant__ TmaParams prm, const Split sp, int* error_flag) {
    constexpr int PER = NBITS == 2 ? 4 : 2;
    constexpr uint32_t TX_BYTES = 2048 + 2 * PER * KC;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ LayerConst s_ly[STREAM_MAX_LAYERS];

    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int K = prm.K, PT = prm.PT, NB = prm.nb;
    const int N_total = prm.col0[prm.count];

    unsigned char* ring_g = smem + (size_t)wi * DEPTH * STAGE_BYTES;
    const uint32_t ring = smem_addr(ring_g);
    __half* x_s = reinterpret_cast<__half*>(smem + (size_t)WARPS * DEPTH * STAGE_BYTES);        // [nx][K]
    __half* ones_s = x_s + (size_t)prm.nx * K;                                                    // 16 halves
    float* red = reinterpret_cast<float*>(ones_s + 16);                                           // [2][WARPS][64]
    uint64_t* bars_g = reinterpret_cast<uint64_t*>(red + 2 * WARPS * RED_FLOATS);                 // [WARPS][DEPTH]
    const uint32_t bars = smem_addr(bars_g + wi * DEPTH);

    // The kernel behind this one may be made resident right away; this one overlaps the tail of its
    // predecessor until `synced`: weights (and their fp16 meta) are never written inside a chain of
    // launches, so the first copies are requested before the wait; x, the row index, the expert choice
    // and the partial buffer are touched only after it.
    grid_launch_dependents();
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
        c.G = prm.G[l];
        c.C = prm.C[l];
        c.pr0 = prm.pr0[l];
        c.col0 = prm.col0[l];
        c.xslot = prm.xslot[l];
        c.pad = 0;
        s_ly[l] = c;
    }
    if (threadIdx.x < 16) ones_s[threadIdx.x] = __float2half(1.f);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < DEPTH; ++s) mbar_init(bars + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (prm.table && lane < 3) {
        // tensor maps that live in global memory: make them visible to the copy engine's proxy
        for (int l = 0; l < prm.count; ++l) {
            const void* m = s_ly[l].maps + lane;
            asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(m) : "memory");
        }
    }

    const uint32_t L0 = sp.begin(blockIdx.x), L1 = sp.begin(blockIdx.x + 1);
    const int n_cta = (int)(L1 - L0);
    const int n_mine = n_cta > wi ? (n_cta - wi + WARPS - 1) / WARPS : 0;
    bool dead = false;

    // ---- copy issue: lanes 0..2 request the codes / scale / zero tile of this warp's pass number `it`
    Cursor iss;
    iss.set(L0 + wi, prm);
    auto issue = [&](int it) {
        if (lane < 3) {
            const LayerConst& c = s_ly[iss.layer];
            const int rho = iss.pl / NB, b = iss.pl - rho * NB;
            const uint32_t stage = ring + (uint32_t)(it % DEPTH) * STAGE_BYTES;
            const uint32_t bar = bars + 8 * (it % DEPTH);
            if (lane == 0) mbar_expect_tx(bar, TX_BYTES);
            const int c1 = lane == 0 ? rho : PER * rho;
            const int c2 = lane == 0 ? 16 * b : 0;
            const uint32_t dst = stage + (lane == 0 ? 0u : (lane == 1 ? (uint32_t)S_OFF : (uint32_t)Z_OFF));
            tma_load_3d(dst, c.maps + lane, iss.p * KC, c1, c2, bar);
        }
        iss.advance(WARPS, prm);
    };
    const int n_pro = n_mine < DEPTH ? n_mine : DEPTH;
    for (int it = 0; it < n_pro; ++it) issue(it);

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
    const uint32_t bytes_off = (uint32_t)((isz ? Z_OFF : S_OFF) + slot * KC);

    // ---- meta prefetch (fp16 scale / zero of the 8-bit scale and zero bytes; L2 resident), one pass ahead
    struct MetaRegs {
        uint4 mz[2][2], ms[2][2];          // [sub-tile][half]: 16 columns each
    };
    Cursor cur;
    cur.set(L0 + wi, prm);
    const uint16_t* ms_p = nullptr;
    const uint16_t* mz_p = nullptr;
    uint32_t rowoff = 0;
    int curC = 1;
    auto bind_unit = [&](const Cursor& c) {                           // per (residue, block): this lane's meta rows
        const LayerConst& lc = s_ly[c.layer];
        const int rho = c.pl / NB;
        ms_p = lc.meta[isz ? 2 : 0];
        mz_p = lc.meta[isz ? 3 : 1];
        curC = lc.C;
        rowoff = (uint32_t)(((uint64_t)(PER * rho + slot) * (uint64_t)K) % (uint64_t)curC);
    };
    auto load_meta = [&](MetaRegs& m, int p) {
        uint32_t col = rowoff + (uint32_t)(p * KC) % (uint32_t)curC;
        col = col >= (uint32_t)curC ? col - (uint32_t)curC : col;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const uint32_t cc = col + 16u * (2 * t + u);
            m.ms[u][0] = ldg128(ms_p + cc);
            m.ms[u][1] = ldg128(ms_p + cc + 8);
            m.mz[u][0] = ldg128(mz_p + cc);
            m.mz[u][1] = ldg128(mz_p + cc + 8);
        }
    };
    MetaRegs meta;
    Cursor nxt = cur;                                                 // the pass whose meta is in `meta`
    if (n_mine > 0) {
        bind_unit(nxt);
        load_meta(meta, nxt.p);
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

    // ---- the CTA's range, residue by residue
    int it = 0;                            // passes this warp has consumed
    int seg = 0;
    uint32_t L = L0;
    int i_rel = wi;                        // CTA-relative number of this warp's next pass
    while (L < L1) {
        const int pr = (int)(L / (uint32_t)PT);
        const uint32_t seg_end_L = min(L1, (uint32_t)(pr + 1) * (uint32_t)PT);
        const int seg_end = (int)(seg_end_L - L0);

        float acc[PER][4];
        float accc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < PER; ++s)
#pragma unroll
            for (int v = 0; v < 4; ++v) acc[s][v] = 0.f;

        for (; i_rel < seg_end; i_rel += WARPS, ++it) {
            // x of this lane's role: the activations for the scale lanes, ones for the zero lanes
            const uint32_t xs_base = isz ? smem_addr(ones_s)
                                         : smem_addr(x_s + (size_t)s_ly[cur.layer].xslot * K + cur.p * KC);
            const uint32_t stage = ring + (uint32_t)(it % DEPTH) * STAGE_BYTES;
            if (!dead) {
                const bool ok = mbar_wait(bars + 8 * (it % DEPTH), (uint32_t)(it / DEPTH) & 1u);
                if (!__all_sync(0xffffffffu, ok)) {                 // give up as a warp: skip the arithmetic, issue nothing more
                    dead = true;
                    if (lane == 0 && error_flag) atomicExch(error_flag, 1);
                }
            }
            uint4 q0[2], q1[2], bq[2], xv[2][2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = 2 * t + u;
                const uint32_t co = cdoff + (uint32_t)((c ^ g) << 4);
                q0[u] = lds128(stage + co);
                q1[u] = lds128(stage + 1024 + co);
                bq[u] = lds128(stage + bytes_off + 16 * c);
                const uint32_t xo = isz ? 0u : (uint32_t)(32 * c);
                xv[u][0] = lds128(xs_base + xo);
                xv[u][1] = lds128(xs_base + xo + (isz ? 0u : 16u));
            }
            const MetaRegs mt = meta;
            __syncwarp();
            // the stage is free again: request the pass DEPTH ahead, and the next pass's meta
            if (!dead && it + DEPTH < n_mine) issue(it + DEPTH);
            const bool unit_changed = nxt.advance(WARPS, prm);
            if (it + 1 < n_mine) {
                if (unit_changed) bind_unit(nxt);
                load_meta(meta, nxt.p);
            }
            cur.advance(WARPS, prm);
            if (dead) continue;

#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const uint32_t bw[4] = {bq[u].x, bq[u].y, bq[u].z, bq[u].w};
                const uint32_t msr[8] = {mt.ms[u][0].x, mt.ms[u][0].y, mt.ms[u][0].z, mt.ms[u][0].w,
                                         mt.ms[u][1].x, mt.ms[u][1].y, mt.ms[u][1].z, mt.ms[u][1].w};
                const uint32_t mzr[8] = {mt.mz[u][0].x, mt.mz[u][0].y, mt.mz[u][0].z, mt.mz[u][0].w,
                                         mt.mz[u][1].x, mt.mz[u][1].y, mt.mz[u][1].z, mt.mz[u][1].w};
                const uint32_t xr[8] = {xv[u][0].x, xv[u][0].y, xv[u][0].z, xv[u][0].w,
                                        xv[u][1].x, xv[u][1].y, xv[u][1].z, xv[u][1].w};
                const uint32_t w0[4] = {q0[u].x, q0[u].y, q0[u].z, q0[u].w};
                const uint32_t w1[4] = {q1[u].x, q1[u].y, q1[u].z, q1[u].w};
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
            }
        }

        // ---- end of the residue inside this CTA: corrections, then the 8 warps' sums in fixed order
        {
            const float mine_z = (g & 1) ? accc[1] : accc[0];        // valid in lane (4 + s, s / 2): sum xs*z of slot s
            const float mine_o = (g & 1) ? accc[3] : accc[2];        // valid in lane (s, s / 2): OFFSET_s * sum xs
            const int sa = (2 * t) % PER;
            const float ca = __shfl_sync(0xffffffffu, mine_z, (4 + sa) * 4 + t) + __shfl_sync(0xffffffffu, mine_o, sa * 4 + t);
            const float cb = __shfl_sync(0xffffffffu, mine_z, (5 + sa) * 4 + t) + __shfl_sync(0xffffffffu, mine_o, (sa + 1) * 4 + t);
            float* mine = red + ((seg & 1) * WARPS + wi) * RED_FLOATS;
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
        }
        __syncthreads();
        if (wi == (seg & (WARPS - 1)) && lane < 16 * PER / 2) {
            int layer = 0;
#pragma unroll
            for (int l = 1; l < STREAM_MAX_LAYERS; ++l) layer += (l < prm.count && pr >= prm.pr0[l]) ? 1 : 0;
            const int pl = pr - prm.pr0[layer];
            const int rho = pl / NB, b = pl - rho * NB;
            const int slot_idx = (int)blockIdx.x - sp.owner((uint32_t)pr * (uint32_t)PT);
            const float* base = red + (seg & 1) * WARPS * RED_FLOATS + 2 * lane;
            float2 v = make_float2(0.f, 0.f);
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float2 a = *reinterpret_cast<const float2*>(base + w * RED_FLOATS);
                v.x += a.x;
                v.y += a.y;
            }
            const int j = (2 * lane) / PER, s = (2 * lane) % PER;
            float* dst = partial + ((int64_t)slot_idx * M_total + m_base) * N_total + prm.col0[layer] +
                         (int64_t)(16 * b + j) * prm.G[layer] + PER * rho + s;
            *reinterpret_cast<float2*>(dst) = v;
        }
        L = seg_end_L;
        ++seg;
    }
    if (dead) {
        // copies may still be in flight towards this CTA's shared memory: give them time before leaving
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
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
    if (w->nbits != 2 && w->nbits != 4) return false;
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

size_t tma_smem_bytes(int nx, int K) {
    return (size_t)WARPS * DEPTH * STAGE_BYTES + (size_t)nx * K * 2 + 32 + (size_t)2 * WARPS * RED_FLOATS * 4 +
           (size_t)WARPS * DEPTH * 8;
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

bool tma_disabled() {
    static const bool off = [] {
        const char* v = getenv("HQM_NO_TMA");
        return v && v[0] == '1';
    }();
    return off;
}

template <int NBITS>
bool prepare_kernel(size_t smem) {
    static size_t configured[MAX_DEVICES];
    size_t& have = configured[current_device_slot()];
    if (have >= smem) return true;
    if (cudaFuncSetAttribute(gemv_tma_kernel<NBITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    have = smem;
    return true;
}

}  // namespace

// Plans one TMA-staged launch over up to four layers for ONE row of x; false when the shapes are outside it
// (the caller then falls back to gemv_stream.cu's kernel).
bool gemv_tma_plan(const hqm_weight* const* ws, int count, StreamPlan* plan) {
    if (count < 1 || count > STREAM_MAX_LAYERS || tma_disabled() || encode_fn() == nullptr) return false;
    const hqm_weight* w = ws[0];
    const int per = codes_per_word(w->nbits);
    const int nb = w->group_size / 16;
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
    int64_t grid = total / WARPS;                  // at least one pass per warp
    if (grid > sms) grid = sms;
    if (grid < 1) grid = 1;
    if (total < grid || total * grid >= ((int64_t)1 << 31)) return false;
    // worst case two distinct rows of x per launch (the two experts' down projections)
    if (tma_smem_bytes(count > 1 ? 2 : 1, w->K) > 227 * 1024) return false;
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
    prm.nb = plan.nb;
    prm.K = job.w[0]->K;
    prm.PT = plan.PT;
    int xrow[STREAM_MAX_LAYERS] = {0, 0, 0, 0};
    for (int l = 0; l < plan.count; ++l) {
        const hqm_weight* w = job.w[l];
        prm.pr0[l] = plan.rho0[l];
        prm.col0[l] = plan.col0[l];
        prm.G[l] = plan.G[l];
        prm.C[l] = plan.C[l];
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
    const size_t smem = tma_smem_bytes(prm.nx, prm.K);
    const Split sp = split_of(plan);
    for (int m = 0; m < (int)M; ++m) {
        if (plan.nbits == 2) {
            if (!prepare_kernel<2>(smem)) return HQM_ERR_CUDA;
            launch_overlapped(gemv_tma_kernel<2>, plan.grid, WARPS * 32, smem, st, partial, x, x_idx, m, (int)M, prm, sp,
                              tc_error_ptr());
        } else {
            if (!prepare_kernel<4>(smem)) return HQM_ERR_CUDA;
            launch_overlapped(gemv_tma_kernel<4>, plan.grid, WARPS * 32, smem, st, partial, x, x_idx, m, (int)M, prm, sp,
                              tc_error_ptr());
        }
        HQM_LAUNCH_CHECK();
    }
    return HQM_OK;
}

}  // namespace hqm

extern "C" {

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
