// Weight-streaming quantized linear for small row counts (decode): the path that
// replaces triton_matmul4_transpose / triton_matmul2_transpose of the reference
// (triton_kernels.py:133-191, 321-380) together with the two per-call
// Quantizer.dequantize launches in front of them (custom_layers.py:62-66).
//
// Algebra.  With r = n % G the residue of output row n and j = n / G its position
// inside the quantisation group,
//     y[m, jG + r] = sum_k (x[m,k] s[r,k]) q[jG + r, k]  -  sum_k (x[m,k] s[r,k]) z[r,k].
// xs[m,r,k] = x[m,k] s[r,k] and the second sum depend only on (m, r): they are shared
// by the `group_size` rows {jG + r}.  So scale and zero are decoded (8 bit -> fp16)
// ONCE per (r, k) and folded into the activations; per weight only the bit-field
// extraction remains.
//
// Mapping.  The unit of work is a "pass": one storage-row residue `rho` (PER adjacent
// residues r, the rows packed into one byte) x 64 input columns.  Passes are numbered
// rho-major and cut into equal contiguous ranges, one per CTA of a single-wave
// persistent grid, one range per WARP (148 SMs x resident warps), so every SM gets the
// same number of bytes whatever the layer shape and warps never wait for each other (no
// CTA barrier anywhere); a warp keeps the next passes in flight with asynchronous copies
// while it computes the current one.  In a pass a warp
//   1. decodes s, z for its PER x 64 (r, k) pairs, 2*PER per lane, and writes
//      xs (per token) and z to warp-private shared memory as fp16;
//   2. streams the 16*NB storage rows rho + i*P (the group's members) with 128-bit
//      loads that bypass L1, 64 contiguous bytes per row;
//   3. turns each 32-bit word into fp16 fragments holding OFFSET + code with one
//      LOP3 per two codes (the field is OR-ed into the mantissa of a constant whose
//      exponent gives that bit position the weight 1) and feeds them to
//      mma.sync.m16n8k16: rows = 16 members, k = 16 input columns, columns = the
//      PER slots x 8/PER tokens (each slot keeps its own accumulator tile; only the
//      columns holding that slot's xs are read back).  The tensor core is used as the
//      cross-lane reduction, so no shuffles are needed on the way;
//   4. one extra MMA per word with A = [z ; OFFSET] yields sum xs*z and OFFSET*sum xs,
//      which are subtracted at the end.
// A residue whose passes span several warps gets one fp32 partial row-set per warp in a
// scratch buffer [slots][M][N]; a small finalize kernel adds them in fixed order
// (deterministic), applies bias and rounds to bf16.
//
// HBM traffic per launch is the packed codes + scale_q + zero_q once (the meta and x
// stay in L1/L2), which is the algorithmic minimum.
#include <stdlib.h>

#include <map>
#include <type_traits>

#include "common.cuh"
#include "kernels.cuh"
#include "stream_split.cuh"

namespace hqm {

// --------------------------------------------------------------------------- helpers
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Two consecutive bf16 (one 32-bit word) -> fp16 pair.
__device__ __forceinline__ __half2 bf16pair_to_h2(uint32_t v) {
    return __floats2half2_rn(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

// (q - mz) * ms on two 8-bit values at once: the bytes land in the mantissa of 1024.0.
__device__ __forceinline__ __half2 meta_decode(uint32_t two_bytes_as_h2, __half2 mz, __half2 ms) {
    const __half2 q = __hsub2(bits_h2(two_bytes_as_h2), bits_h2(0x64006400u));   // exact
    return __hmul2(__hsub2(q, mz), ms);
}

// Bit-field extraction.  `u` is a storage word after the byte permutation
// (B0,B2,B1,B3), so in each 16-bit half the low byte belongs to columns k0 / k1 and
// the high byte to k2 / k3.  lo(s) / hi(s) return the fp16 pair OFFSET + code of slot s
// for (k0,k1) / (k2,k3).  OFF_LO / OFF_HI are those offsets as fp16 bit patterns.
// (field & mask) | magic with mask and magic in registers: one LOP3.  Written as a literal
// expression the two 32-bit immediates do not fit one instruction and it becomes two.
__device__ __forceinline__ uint32_t and_or(uint32_t v, uint32_t mask, uint32_t magic) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(v), "r"(mask), "r"(magic));
    return d;
}

// Masks and fp16 magic numbers of the extraction, passed as a kernel parameter so that
// they live in (uniform) registers instead of being re-materialised as immediates.  A field at bit b of a
// 16-bit half lies inside the fp16 mantissa when b + width <= 10; OR-ed into the constant 2^(10-b) its lowest
// bit weighs exactly 1, so the half reads 2^(10-b) + code.  Fields above the mantissa are shifted down first.
struct FieldConsts {
    uint32_t mask_a, mask_b, mask_c, mask_d, mask_e;
    uint32_t magic_a, magic_b, magic_c, magic_d, magic_e;
};
static inline FieldConsts field_consts(int nbits) {
    if (nbits == 2)   // bits 7-6 -> 16 + c, 5-4 -> 64 + c, 9-8 -> 4 + c, 3-2 -> 256 + c, 1-0 -> 1024 + c
        return FieldConsts{0x00C000C0u, 0x00300030u, 0x03000300u, 0x000C000Cu, 0x00030003u,
                           0x4C004C00u, 0x54005400u, 0x44004400u, 0x5C005C00u, 0x64006400u};
    // 4 bit: bits 7-4 -> 64 + c, bits 3-0 -> 1024 + c
    return FieldConsts{0x00F000F0u, 0x000F000Fu, 0u, 0u, 0u, 0x54005400u, 0x64006400u, 0u, 0u, 0u};
}

template <int NBITS> struct Fields;

template <> struct Fields<2> {
    static constexpr int PER = 4;
    uint32_t v0, v2, v3;
    __device__ __forceinline__ explicit Fields(uint32_t u) : v0(u), v2(u >> 4), v3(u >> 8) {}
    template <int S> __device__ __forceinline__ uint32_t lo(const FieldConsts& c) const {
        if (S == 0) return and_or(v0, c.mask_a, c.magic_a);     // bits 7-6            -> 16 + code
        if (S == 1) return and_or(v0, c.mask_b, c.magic_b);     // bits 5-4            -> 64 + code
        if (S == 2) return and_or(v0, c.mask_d, c.magic_d);     // bits 3-2            -> 256 + code
        return and_or(v0, c.mask_e, c.magic_e);                 // bits 1-0            -> 1024 + code
    }
    template <int S> __device__ __forceinline__ uint32_t hi(const FieldConsts& c) const {
        if (S == 0) return and_or(v3, c.mask_a, c.magic_a);     // bits 15-14 moved to 7-6 -> 16 + code
        if (S == 1) return and_or(v2, c.mask_c, c.magic_c);     // bits 13-12 moved to 9-8 -> 4 + code
        if (S == 2) return and_or(v2, c.mask_a, c.magic_a);     // bits 11-10 moved to 7-6 -> 16 + code
        return and_or(v0, c.mask_c, c.magic_c);                 // bits 9-8                -> 4 + code
    }
    __host__ __device__ static constexpr uint32_t off_lo(int s) {
        return s == 0 ? 0x4C00u : (s == 1 ? 0x5400u : (s == 2 ? 0x5C00u : 0x6400u));
    }
    __host__ __device__ static constexpr uint32_t off_hi(int s) { return (s & 1) ? 0x4400u : 0x4C00u; }
};

template <> struct Fields<4> {
    static constexpr int PER = 2;
    uint32_t v0, v2, v3;
    __device__ __forceinline__ explicit Fields(uint32_t u) : v0(u), v2(u >> 4), v3(u >> 8) {}
    template <int S> __device__ __forceinline__ uint32_t lo(const FieldConsts& c) const {
        return S == 0 ? and_or(v0, c.mask_a, c.magic_a)         // bits 7-4 -> 64 + code
                      : and_or(v0, c.mask_b, c.magic_b);        // bits 3-0 -> 1024 + code
    }
    template <int S> __device__ __forceinline__ uint32_t hi(const FieldConsts& c) const {
        return and_or(S == 0 ? v3 : v2, c.mask_a, c.magic_a);   // bits 15-12 / 11-8 moved to 7-4 -> 64 + code
    }
    __host__ __device__ static constexpr uint32_t off_lo(int s) { return s == 0 ? 0x5400u : 0x6400u; }
    __host__ __device__ static constexpr uint32_t off_hi(int) { return 0x5400u; }
};

// --------------------------------------------------------------------------- kernel
// Compile-time shape of an instantiation.
//   NB   blocks of 16 group members (group_size = 16 * NB)
//   TOKS rows of x decoded per launch (1, 2, 4, 8, 16)
template <int NBITS, int NB, int TOKS>
struct Shape {
    static constexpr int PER = codes_per_word(NBITS);
    static constexpr int TPT = 8 / PER;                         // tokens per column tile
    static constexpr int NT = (TOKS + TPT - 1) / TPT;           // column tiles
    static constexpr int MTOK = NT * TPT;                       // token rows kept in shared memory
    static constexpr int LPS = 32 / PER;                        // decode lanes per slot
    static constexpr int DK = 64 / LPS;                         // decode columns per lane (8 or 4)
    static constexpr int SUB = (NB == 1) ? 2 : 1;               // 64-column sub-passes per pass
    static constexpr int PW = 64 * SUB;                         // pass width in columns
    static constexpr bool STAGE_X = TOKS <= 2;                  // x converted to fp16 in shared memory per segment
    static constexpr int ROW = 72;                              // 64 columns + padding against bank conflicts
    static constexpr int WARP_HALFS = SUB * (MTOK * PER + PER + 1) * ROW;   // xs rows, z rows, one zero row
    static constexpr int NW = 8;
    static constexpr int XPASS = (TOKS == 1) ? 16 : 8;          // longest range (passes) a warp may be given
    // Asynchronous-copy ring: per warp DEPTH slots, each one pass of 16-byte cells per lane:
    // per sub-pass 2*NB weight-row cells and 1 cell scale_q | zero_q: the bytes that come from HBM.  The fp16
    // meta of scale/zero (L2 resident) is loaded to registers one pass ahead; x comes from the per-segment
    // fp16 staging buffer, or straight from global memory when there are too many rows for that.
    static constexpr int DEPTH = 2;
    static constexpr int CELLS_SUB = 2 * NB + 1;
    static constexpr int CELLS = SUB * CELLS_SUB;
    static constexpr int SLOT_BYTES = CELLS * 32 * 16;
    static constexpr int XH_HALFS = STAGE_X ? TOKS * XPASS * PW : 0;   // per warp: its range of x as fp16
    static constexpr size_t WARP_BYTES = (size_t)WARP_HALFS * 2 + (size_t)DEPTH * SLOT_BYTES + (size_t)XH_HALFS * 2;
    static constexpr size_t smem_bytes() { return (size_t)NW * WARP_BYTES; }
};

template <int N> __device__ __forceinline__ void ld_words(uint32_t (&dst)[N], const void* p) {
    if constexpr (N == 1) {
        dst[0] = *reinterpret_cast<const uint32_t*>(p);
    } else if constexpr (N == 2) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        dst[0] = v.x; dst[1] = v.y;
    } else {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
}
template <int N> __device__ __forceinline__ void st_words(void* p, const uint32_t (&src)[N]) {
    if constexpr (N == 2) {
        *reinterpret_cast<uint2*>(p) = make_uint2(src[0], src[1]);
    } else {
        *reinterpret_cast<uint4*>(p) = make_uint4(src[0], src[1], src[2], src[3]);
    }
}

// Per-thread asynchronous global -> shared copies (the data goes to shared memory without
// occupying registers while in flight, so a warp can have several passes outstanding).
template <int BYTES>
__device__ __forceinline__ void cp_async(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    if constexpr (BYTES == 16) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(d), "l"(gmem_src), "n"(BYTES) : "memory");
    }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Up to four layers share one launch (an expert's w1 and w3; the q, k and v projections; both experts
// of a token): same K, bit width and group size, their N may differ.  Their residues are numbered one
// after the other (rho0), their output columns follow each other in the partial rows (col0), and each
// reads its own block of rows of x (xrow).
// With `table` set the layers are not the descriptors passed by value but entries of a descriptor table in
// device memory, picked by an index that is itself in device memory (the router's choice): layer l is
// table[3 * *sel[l] + which[l]].  w[l] then only carries the shape.  This keeps the host out of the
// loop when all experts are resident.
struct Layers {
    hqm_weight w[STREAM_MAX_LAYERS];
    int count;
    int rho0[STREAM_MAX_LAYERS + 1];
    int col0[STREAM_MAX_LAYERS + 1];
    int G[STREAM_MAX_LAYERS], C[STREAM_MAX_LAYERS];
    int xrow[STREAM_MAX_LAYERS];
    const StreamEntry* table;
    const int32_t* sel[STREAM_MAX_LAYERS];
    int which[STREAM_MAX_LAYERS];
    int sel_settled;    // the indices behind `sel` were complete before this kernel could start (see StreamJob)
};

template <int NBITS, int NB, int TOKS>
__global__ void __launch_bounds__(256, (NB == 1 && TOKS <= 2) ? 2 : 1)
gemv_stream_kernel(float* __restrict__ partial, const uint16_t* __restrict__ x, const int32_t* __restrict__ x_idx,
                   int M, int m_base, int M_total, Layers ly, Split sp, FieldConsts fc) {
    using F = Fields<NBITS>;
    using S = Shape<NBITS, NB, TOKS>;
    constexpr int PER = S::PER, TPT = S::TPT, NT = S::NT, MTOK = S::MTOK, LPS = S::LPS, DK = S::DK, SUB = S::SUB,
                  PW = S::PW, ROW = S::ROW, NW = S::NW;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int K = ly.w[0].K, PT = sp.PT;
    const int N_total = ly.col0[ly.count];
    unsigned char* warp_mem = smem_raw + (size_t)wi * S::WARP_BYTES;               // everything is warp-private
    __half* xs_w = reinterpret_cast<__half*>(warp_mem);                             // [SUB][MTOK][PER][ROW]
    __half* zz_w = xs_w + SUB * MTOK * PER * ROW;                                  // [SUB][PER + 1][ROW], last row zero
    unsigned char* ring = warp_mem + (size_t)S::WARP_HALFS * 2 + lane * 16;        // this lane's cell column
    __half* xh = reinterpret_cast<__half*>(warp_mem + (size_t)S::WARP_HALFS * 2 + (size_t)S::DEPTH * S::SLOT_BYTES);
    constexpr int XCOLS = S::XPASS * PW;                                           // [TOKS][XCOLS]

    // The next kernel on the stream may be made resident as SMs free up; this one overlaps the tail of the
    // kernel in front of it until `synced`: the weights are never written by a kernel of the chain, so the
    // first passes are requested before the wait; x, the row indices, the expert choice and the partial
    // buffer belong to earlier kernels and are touched only after it.
    grid_launch_dependents();
    bool synced = false;
    if (ly.table && !ly.sel_settled) {
        grid_dependency_wait();
        synced = true;
    }
    // Table mode: the (up to four) descriptors the router's choice points at are fetched once per CTA into
    // shared memory, so that a warp starting a segment does not sit through an index load and a dependent
    // descriptor load before it can request its first weights.
    // A negative index means "this layer is not here" (an expert-parallel rank that does not own the routed
    // expert): its passes are skipped and its sums are written as zeros.
    __shared__ hqm_weight s_desc[STREAM_MAX_LAYERS];
    __shared__ int s_absent[STREAM_MAX_LAYERS];
    if (ly.table) {
        constexpr int WORDS = (int)(sizeof(hqm_weight) / sizeof(uint32_t));
        if ((int)threadIdx.x < ly.count * WORDS) {
            const int l = threadIdx.x / WORDS, i = threadIdx.x % WORDS;
            // (__ldcg: the index may have been written by a kernel that finished while an earlier kernel on this
            // SM still had the previous value in L1)
            const int idx = __ldcg(ly.sel[l]);
            if (i == 0) s_absent[l] = idx < 0 ? 1 : 0;
            if (idx >= 0) {
                const hqm_weight* src = &(ly.table + 3 * idx + ly.which[l])->w;
                reinterpret_cast<uint32_t*>(s_desc)[threadIdx.x] = reinterpret_cast<const uint32_t*>(src)[i];
            }
        }
        __syncthreads();
    }

    // token rows that exist only to fill a column tile, and the extra z row, stay zero for the whole kernel
    for (int i = lane; i < S::WARP_HALFS / 2; i += 32) reinterpret_cast<uint32_t*>(xs_w)[i] = 0u;
    __syncwarp();

    const uint16_t* xr[TOKS];
    const int sd = lane / LPS;                      // slot this lane decodes
    const int kd = (lane % LPS) * DK;               // its first column inside a sub-pass
    const int sB = g % PER, mB = g / PER;           // slot / token of this lane's B column
    const int sa = (2 * t) % PER;                   // first of the two slots whose columns this lane reads back
    const uint32_t keep = (g < PER) ? 0xffffffffu : 0u;
    const int zrow = (g < PER ? g : PER) * ROW + 16 * t;      // this lane's row of the z tile (row PER is zero)
    const uint32_t olo = F::off_lo(g & 3) * 0x00010001u & keep;   // row 8 + g of the correction tile: slot g's offsets
    const uint32_t ohi = F::off_hi(g & 3) * 0x00010001u & keep;

    const int gw = blockIdx.x * NW + wi;                                           // this warp in the grid
    const uint32_t L_begin = sp.begin(gw), L_end = sp.begin(gw + 1);
    for (uint32_t L = L_begin; L < L_end;) {
        // ---- one segment: passes [pa, pb) of residue rho of layer `layer`
        const int rho_g = (int)(L / (uint32_t)PT), pa = (int)(L - (uint32_t)rho_g * (uint32_t)PT);
        const int pb_all = min(PT, pa + (int)(L_end - L));
        L += (uint32_t)(pb_all - pa);
        int layer = 0;
#pragma unroll
        for (int l = 1; l < STREAM_MAX_LAYERS; ++l) layer += (l < ly.count && rho_g >= ly.rho0[l]) ? 1 : 0;
        const int pb = (ly.table && s_absent[layer]) ? pa : pb_all;      // an absent layer: no passes, zero sums
        const int rho = rho_g - ly.rho0[layer];
        const int P = ly.rho0[layer + 1] - ly.rho0[layer], G = ly.G[layer], C = ly.C[layer];
        const hqm_weight w = ly.table ? s_desc[layer] : ly.w[layer];
        uint32_t qoff[NB];                          // this lane's weight rows, bytes from W_q + rho*K + k0
#pragma unroll
        for (int b = 0; b < NB; ++b) qoff[b] = (uint32_t)(16 * b + g) * (uint32_t)P * (uint32_t)K + 16u * t;
        const uint32_t qoff8 = 8u * (uint32_t)P * (uint32_t)K;

        float acc[NB][NT][PER][4];
        float accc[NT][4];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int tau = 0; tau < NT; ++tau)
#pragma unroll
                for (int s = 0; s < PER; ++s)
#pragma unroll
                    for (int v = 0; v < 4; ++v) acc[b][tau][s][v] = 0.f;
#pragma unroll
        for (int tau = 0; tau < NT; ++tau)
#pragma unroll
            for (int v = 0; v < 4; ++v) accc[tau][v] = 0.f;

        const uint8_t* wrow = reinterpret_cast<const uint8_t*>(w.W_q) + (size_t)rho * K;
        const uint32_t dbase = (uint32_t)(PER * rho + sd) * (uint32_t)K + kd;     // flat scale/zero index at k0 = 0
        // meta column of a flat scale/zero index: the residue-row part is reduced once per segment,
        // each pass then adds its k0 (tracked modulo C) and wraps with a compare
        const uint32_t dcol0 = dbase % (uint32_t)C;
        uint32_t kcol = (uint32_t)(pa * PW) % (uint32_t)C;            // (k0 % C) of the pass loaded next
        const uint32_t kstep = (uint32_t)PW % (uint32_t)C;
        const uint32_t ustep = 64u % (uint32_t)C;

        struct Meta {
            uint32_t sq[SUB][DK / 4], zq[SUB][DK / 4];
            uint32_t mss[SUB][DK / 2], mzs[SUB][DK / 2], msz[SUB][DK / 2], mzz[SUB][DK / 2];
            uint32_t xv[S::STAGE_X ? 1 : TOKS][SUB][DK / 2];
        };
        struct Rows {
            uint4 q0[SUB][NB], q1[SUB][NB];
        };

        // cell (c) of slot (sl): ring + sl * SLOT_BYTES + c * 512 (each lane owns 16 bytes of every cell)
        auto issue = [&](int sl, int p) {
            unsigned char* cell = ring + sl * S::SLOT_BYTES;
            const uint8_t* base = wrow + p * PW;
            const int k0 = p * PW;
            const uint32_t idx = dbase + k0;
#pragma unroll
            for (int u = 0; u < SUB; ++u) {
                unsigned char* cu = cell + u * S::CELLS_SUB * 512;
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    cp_async<16>(cu + (2 * b) * 512, base + qoff[b] + 64 * u);
                    cp_async<16>(cu + (2 * b + 1) * 512, base + qoff[b] + qoff8 + 64 * u);
                }
                unsigned char* cm = cu + 2 * NB * 512;
                cp_async<DK>(cm, w.scale_q + idx + 64 * u);
                cp_async<DK>(cm + 8, w.zero_q + idx + 64 * u);
            }
        };
        auto load_meta = [&](Meta& r) {                 // for the pass whose columns kcol points at
#pragma unroll
            for (int u = 0; u < SUB; ++u) {
                uint32_t col = dcol0 + kcol;                      // < 2C
                col = col >= (uint32_t)C ? col - (uint32_t)C : col;
                if (u == 1) {
                    col += ustep;
                    col = col >= (uint32_t)C ? col - (uint32_t)C : col;
                }
                ld_words(r.mss[u], w.ms_scale + col);
                ld_words(r.mzs[u], w.mz_scale + col);
                ld_words(r.msz[u], w.ms_zero + col);
                ld_words(r.mzz[u], w.mz_zero + col);
            }
            kcol += kstep;
            kcol = kcol >= (uint32_t)C ? kcol - (uint32_t)C : kcol;
        };
        auto fetch = [&](int sl, int p, Meta& r, Rows& q) {
            const unsigned char* cell = ring + sl * S::SLOT_BYTES;
#pragma unroll
            for (int u = 0; u < SUB; ++u) {
                const unsigned char* cu = cell + u * S::CELLS_SUB * 512;
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    q.q0[u][b] = *reinterpret_cast<const uint4*>(cu + (2 * b) * 512);
                    q.q1[u][b] = *reinterpret_cast<const uint4*>(cu + (2 * b + 1) * 512);
                }
                const unsigned char* cm = cu + 2 * NB * 512;
                ld_words(r.sq[u], cm);
                ld_words(r.zq[u], cm + 8);
                if constexpr (!S::STAGE_X) {
#pragma unroll
                    for (int m = 0; m < TOKS; ++m) ld_words(r.xv[m][u], xr[m] + p * PW + 64 * u + kd);
                }
            }
        };

        // 1. decode scale / zero of (slot sd, DK columns per sub-pass), fold into x, publish to the warp
        auto decode_pass = [&](const Meta& r, int p) {
#pragma unroll
            for (int u = 0; u < SUB; ++u) {
                uint32_t s2[DK / 2], z2[DK / 2];
#pragma unroll
                for (int j = 0; j < DK / 2; ++j) {
                    const uint32_t sel = (j & 1) ? 0x4342u : 0x4140u;      // bytes (2j, 2j+1) of the word -> two fp16
                    s2[j] = h2_bits(meta_decode(prmt(r.sq[u][j / 2], 0x64646464u, sel), bits_h2(r.mzs[u][j]),
                                                bits_h2(r.mss[u][j])));
                    z2[j] = h2_bits(meta_decode(prmt(r.zq[u][j / 2], 0x64646464u, sel), bits_h2(r.mzz[u][j]),
                                                bits_h2(r.msz[u][j])));
                }
                st_words(zz_w + (u * (PER + 1) + sd) * ROW + kd, z2);
#pragma unroll
                for (int m = 0; m < TOKS; ++m) {
                    uint32_t xs2[DK / 2];
                    if constexpr (S::STAGE_X) {
                        uint32_t xf[DK / 2];
                        ld_words(xf, xh + m * XCOLS + (p - pa) * PW + 64 * u + kd);
#pragma unroll
                        for (int j = 0; j < DK / 2; ++j) xs2[j] = h2_bits(__hmul2(bits_h2(xf[j]), bits_h2(s2[j])));
                    } else {
#pragma unroll
                        for (int j = 0; j < DK / 2; ++j)
                            xs2[j] = h2_bits(__hmul2(bf16pair_to_h2(r.xv[m][u][j]), bits_h2(s2[j])));
                    }
                    st_words(xs_w + ((u * MTOK + m) * PER + sd) * ROW + kd, xs2);
                }
            }
            __syncwarp();
        };

        auto mma_pass = [&](const Rows& r) {
#pragma unroll
            for (int u = 0; u < SUB; ++u) {
                // 2. B fragments: xs of (token, slot sB) at this lane's 16 columns
                uint32_t bf[NT][8];
#pragma unroll
                for (int tau = 0; tau < NT; ++tau) {
                    const __half* src = xs_w + ((u * MTOK + tau * TPT + mB) * PER + sB) * ROW + 16 * t;
                    const uint4 lo4 = *reinterpret_cast<const uint4*>(src);
                    const uint4 hi4 = *reinterpret_cast<const uint4*>(src + 8);
                    bf[tau][0] = lo4.x; bf[tau][1] = lo4.y; bf[tau][2] = lo4.z; bf[tau][3] = lo4.w;
                    bf[tau][4] = hi4.x; bf[tau][5] = hi4.y; bf[tau][6] = hi4.z; bf[tau][7] = hi4.w;
                }
                // 3. correction tile: rows 0..PER-1 = z of slot i, rows 8..8+PER-1 = the offsets
                {
                    uint32_t zf[8];
                    const __half* src = zz_w + u * (PER + 1) * ROW + zrow;      // lanes without a slot read zeros
                    const uint4 lo4 = *reinterpret_cast<const uint4*>(src);
                    const uint4 hi4 = *reinterpret_cast<const uint4*>(src + 8);
                    zf[0] = lo4.x; zf[1] = lo4.y; zf[2] = lo4.z; zf[3] = lo4.w;
                    zf[4] = hi4.x; zf[5] = hi4.y; zf[6] = hi4.z; zf[7] = hi4.w;
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd)
#pragma unroll
                        for (int tau = 0; tau < NT; ++tau)
                            mma_f16(accc[tau], zf[2 * wd], olo, zf[2 * wd + 1], ohi, bf[tau][2 * wd],
                                    bf[tau][2 * wd + 1]);
                }
                // 4. the weights
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const uint32_t r0[4] = {r.q0[u][b].x, r.q0[u][b].y, r.q0[u][b].z, r.q0[u][b].w};
                    const uint32_t r1[4] = {r.q1[u][b].x, r.q1[u][b].y, r.q1[u][b].z, r.q1[u][b].w};
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        const F f0(prmt(r0[wd], 0u, 0x3120u)), f1(prmt(r1[wd], 0u, 0x3120u));
#pragma unroll
                        for (int tau = 0; tau < NT; ++tau) {
                            const uint32_t b0 = bf[tau][2 * wd], b1 = bf[tau][2 * wd + 1];
                            mma_f16(acc[b][tau][0], f0.template lo<0>(fc), f1.template lo<0>(fc), f0.template hi<0>(fc),
                                    f1.template hi<0>(fc), b0, b1);
                            mma_f16(acc[b][tau][1], f0.template lo<1>(fc), f1.template lo<1>(fc), f0.template hi<1>(fc),
                                    f1.template hi<1>(fc), b0, b1);
                            if constexpr (PER == 4) {
                                mma_f16(acc[b][tau][PER - 2], f0.template lo<2>(fc), f1.template lo<2>(fc),
                                        f0.template hi<2>(fc), f1.template hi<2>(fc), b0, b1);
                                mma_f16(acc[b][tau][PER - 1], f0.template lo<3>(fc), f1.template lo<3>(fc),
                                        f0.template hi<3>(fc), f1.template hi<3>(fc), b0, b1);
                            }
                        }
                    }
                }
            }
            __syncwarp();   // the next pass overwrites this warp's shared memory
        };

        // ---- the warp's passes of this segment: DEPTH passes are requested with asynchronous copies
        // before anything is computed, and a slot is refilled as soon as its pass has been moved to
        // registers, so the copies of the next passes run under the arithmetic of the current one.
        // (One commit group per pass, empty when the warp has no pass left, keeps the count uniform.)
#pragma unroll
        for (int sl = 0; sl < S::DEPTH; ++sl) {
            if (pa + sl < pb) issue(sl, pa + sl);
            cp_async_commit();
        }
        if (!synced) {
            grid_dependency_wait();
            synced = true;
        }
#pragma unroll
        for (int m = 0; m < TOKS; ++m) {
            const int mm = (m < M) ? (m_base + m) : m_base;
            xr[m] = x + ((int64_t)(x_idx ? x_idx[mm] : mm) + ly.xrow[layer]) * K;
        }
        if constexpr (S::STAGE_X) {
            // the segment's columns of x, converted to fp16 once
            const int c0 = pa * PW, nc = (pb - pa) * PW;
#pragma unroll
            for (int m = 0; m < TOKS; ++m)
                for (int i = lane * 2; i < nc; i += 64)
                    *reinterpret_cast<__half2*>(xh + m * XCOLS + i) =
                        bf16pair_to_h2(*reinterpret_cast<const uint32_t*>(xr[m] + c0 + i));
            __syncwarp();
        }

        {
            Meta d;
            Rows r;
            int sl = 0;
            if (pa < pb) load_meta(d);
            for (int p = pa; p < pb; ++p) {
                cp_async_wait<S::DEPTH - 1>();
                fetch(sl, p, d, r);
                const int pn = p + S::DEPTH;
                if (pn < pb) issue(sl, pn);
                cp_async_commit();
                decode_pass(d, p);
                if (p + 1 < pb) load_meta(d);          // the meta registers are free again: next pass's
                mma_pass(r);
                sl = (sl + 1 == S::DEPTH) ? 0 : sl + 1;
            }
            cp_async_wait<0>();
        }

        // ---- segment epilogue: pick the valid columns, subtract the correction, store this warp's
        // partial row-set.  Lane (g, t) holds columns 2t, 2t+1 of every tile: slots sa and sa + 1 of token
        // (2t) / PER.  Column n of the correction tile is valid in the lane whose row index equals the
        // column's slot.
        const int slot_idx = gw - sp.owner((uint32_t)rho_g * (uint32_t)PT);
#pragma unroll
        for (int tau = 0; tau < NT; ++tau) {
            const float mine = (sa == g) ? accc[tau][0] + accc[tau][2] : accc[tau][1] + accc[tau][3];
            const float ca = __shfl_sync(0xffffffffu, mine, sa * 4 + t);
            const float cb = __shfl_sync(0xffffffffu, mine, (sa + 1) * 4 + t);
            const int m = tau * TPT + (2 * t) / PER;
            if (m < M) {
                float* dst = partial + ((int64_t)slot_idx * M_total + m_base + m) * N_total + ly.col0[layer] +
                             PER * rho + sa;
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    float va0 = 0.f, va1 = 0.f, vb0 = 0.f, vb1 = 0.f;
#pragma unroll
                    for (int s = 0; s < PER; s += 2) {
                        if (s == sa) {
                            va0 = acc[b][tau][s][0];      // row g,     column 2t
                            va1 = acc[b][tau][s][2];      // row g + 8, column 2t
                            vb0 = acc[b][tau][s + 1][1];  // row g,     column 2t + 1
                            vb1 = acc[b][tau][s + 1][3];  // row g + 8, column 2t + 1
                        }
                    }
                    float* d0 = dst + (int64_t)(16 * b + g) * G;        // member 16b + g
                    float* d1 = d0 + (int64_t)8 * G;                    // member 16b + g + 8
                    *reinterpret_cast<float2*>(d0) = make_float2(va0 - ca, vb0 - cb);
                    *reinterpret_cast<float2*>(d1) = make_float2(va1 - ca, vb1 - cb);
                }
            }
        }
        __syncwarp();   // the staged x is reused by the next segment
    }
}

// y = bf16( sum of the partials + bias ); the layers of the launch end up side by side in a row of y
__global__ void finalize_linear_kernel(uint16_t* __restrict__ y, const float* __restrict__ partial,
                                       const uint16_t* __restrict__ bias, int64_t M, int row, Split sp, ColMap cm) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t MR = M * row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < MR; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / row;
        const int n = (int)(i - m * row);
        float v = partial_sum<false>(partial, sp, cm, m, n, row, MR);
        if (bias) v += bf16_bits_to_float(bias[n]);
        y[i] = float_to_bf16_bits(v);
    }
}

// h[p][m, f] = bf16( bf16(silu(bf16(a))) * bf16(b) ) with a / b the summed partials of layers 2p / 2p + 1
// of the launch (an expert's w1 and w3), for each of the launch's layer pairs p.
// With `late_trigger` the next kernel may only start once everything in front of this one has completed.
__global__ void finalize_silu_mul_kernel(uint16_t* __restrict__ h, const float* __restrict__ partial, int64_t M,
                                         int F, int pairs, int row, int late_trigger, Split sp, ColMap cm) {
    if (!late_trigger) grid_launch_dependents();
    grid_dependency_wait();
    if (late_trigger) grid_launch_dependents();
    const int64_t MF = M * F, total = MF * pairs, MR = M * row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int p = (int)(i / MF);
        const int64_t m = (i - p * MF) / F;
        const int f = (int)(i - p * MF - m * F);
        float a, b;
        partial_sum_pair<false>(partial, sp, cm, m, layer_col0(cm, 2 * p) + f, layer_col0(cm, 2 * p + 1) + f, row, MR, a, b);
        a = round_bf16(a);
        b = round_bf16(b);
        const float act = round_bf16(a / (1.f + __expf(-a)));
        h[i] = float_to_bf16_bits(act * b);
    }
}

// out[t] = (accumulate ? out[t] : 0) + sum over the launch's layers l of bf16(w[l*M + i] * bf16(partial sum of
// layer l)), added in layer order with a bf16 rounding after each step (as consecutive index_add_ calls do);
// t = token_idx[i].
__global__ void finalize_scatter_kernel(uint16_t* __restrict__ out, const float* __restrict__ partial,
                                        const int32_t* __restrict__ token_idx, const float* __restrict__ route_w,
                                        int64_t M, int H, int row, int accumulate, Split sp, ColMap cm) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t MH = M * H, MR = M * row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < MH; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / H;
        const int n = (int)(i - m * H);
        const int64_t tk = token_idx ? token_idx[m] : m;
        uint16_t* dst = out + tk * H + n;
        float acc = accumulate ? bf16_bits_to_float(*dst) : 0.f;
#pragma unroll
        for (int l = 0; l < STREAM_MAX_LAYERS; ++l) {
            if (l < cm.count) {
                const float wgt = route_w ? route_w[l * M + m] : 1.f;
                const float v = round_bf16(round_bf16(partial_sum<false>(partial, sp, cm, m, cm.col0[l] + n, row, MR)) * wgt);
                acc = (l == 0 && !accumulate) ? v : round_bf16(acc + v);
            }
        }
        *dst = float_to_bf16_bits(acc);
    }
}

// --------------------------------------------------------------------------- host side
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Resident CTAs per SM of an instantiation, times the SM count (queried once per device).
template <int NBITS, int NB, int TOKS>
static int resident_grid() {
    using S = Shape<NBITS, NB, TOKS>;
    static int per_device[MAX_DEVICES];          // 0: not queried yet, otherwise grid + 1
    int& slot = per_device[current_device_slot()];
    if (slot > 0) return slot - 1;
    const int grid = [] {
        auto kern = gemv_stream_kernel<NBITS, NB, TOKS>;
        const size_t smem = S::smem_bytes();
        if (smem > 227 * 1024) return 0;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        int per_sm = 0, dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 256, smem) != cudaSuccess || per_sm < 1) {
            cudaGetLastError();
            return 0;
        }
        return per_sm * sms;
    }();
    slot = grid + 1;
    return grid;
}

// Rows of x one launch decodes for `tokens` pending rows.
static int toks_for(int nbits, int nb, int tokens) {
    const int max_toks = (nbits == 2) ? (nb == 1 ? 8 : 4) : (nb == 2 ? 16 : 8);
    int tk = 1;
    while (tk < max_toks && tk < tokens) tk *= 2;
    if (nbits == 4 && tk == 2) tk = 4;           // a 4-bit column tile holds 4 tokens anyway
    return tk;
}

template <typename Fn>
static int dispatch(int nbits, int nb, int toks, Fn&& fn) {
#define HQM_CASE(B, NBK, T) \
    if (nbits == B && nb == NBK && toks == T) \
        return fn(std::integral_constant<int, B>(), std::integral_constant<int, NBK>(), std::integral_constant<int, T>());
    HQM_CASE(2, 1, 1) HQM_CASE(2, 1, 2) HQM_CASE(2, 1, 4) HQM_CASE(2, 1, 8)
    HQM_CASE(2, 2, 1) HQM_CASE(2, 2, 2) HQM_CASE(2, 2, 4)
    HQM_CASE(4, 2, 1) HQM_CASE(4, 2, 4) HQM_CASE(4, 2, 8) HQM_CASE(4, 2, 16)
    HQM_CASE(4, 4, 1) HQM_CASE(4, 4, 4) HQM_CASE(4, 4, 8)
#undef HQM_CASE
    return -1;
}

bool gemv_stream_plan(const hqm_weight* const* ws, int count, int64_t M, StreamPlan* plan, bool chained) {
    if (count < 1 || count > STREAM_MAX_LAYERS || force_generic()) return false;
    plan->tma = 0;
    if (M == 1 && gemv_tma_plan(ws, count, chained, plan)) return true;
    plan->tma = 0;
    const hqm_weight* w = ws[0];
    if (w->nbits != 2 && w->nbits != 4) return false;
    const int per = codes_per_word(w->nbits);
    const int dk = w->nbits == 2 ? 8 : 4;
    const int g = w->group_size;
    const bool group_ok = (w->nbits == 2) ? (g == 16 || g == 32) : (g == 32 || g == 64);
    const int nb = g / 16;
    const int pw = nb == 1 ? 128 : 64;
    if (!group_ok || w->K % pw != 0) return false;
    if (M < 1 || M > 16) return false;
    plan->count = count;
    plan->rho0[0] = 0;
    plan->col0[0] = 0;
    for (int l = 0; l < count; ++l) {
        const hqm_weight* v = ws[l];
        int G, C;
        if (check_weight(v, &G, &C) != HQM_OK || !meta_uniform(v)) return false;
        if (v->nbits != w->nbits || v->group_size != g || v->K != w->K || v->meta_group != w->meta_group) return false;
        if (G % per != 0 || C % dk != 0) return false;
        if ((int64_t)G * v->K >= (int64_t)1 << 31 || (int64_t)(v->N / per) * v->K >= (int64_t)1 << 31) return false;
        if (!aligned16(v->W_q) || !aligned16(v->scale_q) || !aligned16(v->zero_q) || !aligned16(v->ms_scale) ||
            !aligned16(v->mz_scale) || !aligned16(v->ms_zero) || !aligned16(v->mz_zero))
            return false;
        plan->G[l] = G;
        plan->C[l] = C;
        plan->rho0[l + 1] = plan->rho0[l] + G / per;
        plan->col0[l + 1] = plan->col0[l] + v->N;
    }
    const int toks = toks_for(w->nbits, nb, (int)M);
    int grid = dispatch(w->nbits, nb, toks, [](auto b, auto k, auto t) {
        return resident_grid<decltype(b)::value, decltype(k)::value, decltype(t)::value>();
    });
    if (grid <= 0) return false;
    plan->nbits = w->nbits;
    plan->nb = nb;
    plan->PT = w->K / pw;
    const int64_t total = (int64_t)plan->rho0[count] * plan->PT;
    // Whole CTAs per SM, so that every SM carries the same load; fewer of them (and, for small layers,
    // fewer SMs) rather than ranges shorter than ~2 passes, each of which costs a partial row-set.
    {
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int per_sm = grid / sms;
        const int64_t want = total / ((int64_t)sms * 8 * 2);
        if (per_sm > want) per_sm = (int)(want < 1 ? 1 : want);
        grid = per_sm * sms;
        if ((int64_t)grid * 8 * 2 > total) grid = (int)(total / (8 * 2));
        if (grid < 1) grid = 1;
        if ((int64_t)grid * 8 > total) return false;
    }
    const int64_t warps = (int64_t)grid * 8;
    if (total * warps >= ((int64_t)1 << 31)) return false;
    if (toks <= 2 && (total + warps - 1) / warps + 1 > (toks == 1 ? 16 : 8)) return false;   // the x staging buffer
    plan->grid = grid;
    plan->warps = (int)warps;
    plan->toks = toks;
    const int64_t min_range = total / warps;                  // >= 1
    plan->slots = (int)((plan->PT + min_range - 1) / min_range) + 1;
    return true;
}

size_t gemv_tma_scratch_bytes(const StreamPlan& plan, int64_t M);
size_t gemv_stream_scratch_bytes(const StreamPlan& plan, int64_t M) {
    if (plan.tma) return gemv_tma_scratch_bytes(plan, M);
    return (size_t)plan.slots * (size_t)M * (size_t)plan.col0[plan.count] * sizeof(float);
}

int launch_gemv_stream(float* partial, const uint16_t* x, const int32_t* x_idx, int64_t M, const StreamJob& job,
                       const StreamPlan& plan, cudaStream_t st) {
    if (plan.tma) return launch_gemv_tma(partial, x, x_idx, M, job, plan, st);
    Layers ly{};
    ly.count = plan.count;
    for (int l = 0; l < plan.count; ++l) {
        ly.w[l] = *job.w[l];
        ly.G[l] = plan.G[l];
        ly.C[l] = plan.C[l];
        ly.rho0[l] = plan.rho0[l];
        ly.col0[l] = plan.col0[l];
        ly.xrow[l] = job.xrow[l];
        ly.sel[l] = job.sel[l];
        ly.which[l] = job.which[l];
    }
    ly.rho0[plan.count] = plan.rho0[plan.count];
    ly.col0[plan.count] = plan.col0[plan.count];
    ly.table = job.table;
    ly.sel_settled = job.sel_settled;
    const Split sp = work_split_of(plan);
    // rows beyond one launch's tokens go in further launches over the same split
    for (int m0 = 0; m0 < (int)M; m0 += plan.toks) {
        const int take = ((int)M - m0 < plan.toks) ? (int)M - m0 : plan.toks;
        const int rc = dispatch(plan.nbits, plan.nb, plan.toks, [&](auto b, auto k, auto t) {
            constexpr int B = decltype(b)::value, NBK = decltype(k)::value, T = decltype(t)::value;
            launch_overlapped(gemv_stream_kernel<B, NBK, T>, plan.grid, 256, Shape<B, NBK, T>::smem_bytes(), st, partial,
                              x, x_idx, take, m0, (int)M, ly, sp, field_consts(plan.nbits));
            return 0;
        });
        if (rc != 0) {
            set_error("gemv_stream: no instantiation for nbits=%d group_size=%d", plan.nbits, 16 * plan.nb);
            return HQM_ERR_ARG;
        }
        HQM_LAUNCH_CHECK();
    }
    return HQM_OK;
}

static inline int blocks_for(int64_t n) {
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    return (int)(blocks < 1 ? 1 : blocks);
}

int launch_finalize_linear(uint16_t* y, const float* partial, const uint16_t* bias, int64_t M, const StreamPlan& plan,
                           cudaStream_t st) {
    const int row = plan.col0[plan.count];
    launch_overlapped(finalize_linear_kernel, blocks_for(M * row), 256, 0, st, y, partial, bias, M, row, split_of(plan),
                      colmap_of(plan));
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

int launch_finalize_silu_mul(uint16_t* h, const float* partial, int64_t M, const StreamPlan& plan, cudaStream_t st,
                             bool late_trigger) {
    const int F = plan.col0[1], pairs = plan.count / 2, row = plan.col0[plan.count];
    launch_overlapped(finalize_silu_mul_kernel, blocks_for(M * F * pairs), 256, 0, st, h, partial, M, F, pairs, row,
                      late_trigger ? 1 : 0, split_of(plan), colmap_of(plan));
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

int launch_finalize_scatter(uint16_t* out, const float* partial, const int32_t* token_idx, const float* route_w,
                            int accumulate, int64_t M, const StreamPlan& plan, cudaStream_t st) {
    const int H = plan.col0[1], row = plan.col0[plan.count];
    launch_overlapped(finalize_scatter_kernel, blocks_for(M * H), 256, 0, st, out, partial, token_idx, route_w, M, H, row,
                      accumulate, split_of(plan), colmap_of(plan));
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

}  // namespace hqm
