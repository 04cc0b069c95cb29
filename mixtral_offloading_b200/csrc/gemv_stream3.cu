// Weight-streaming quantized linear for 3-bit layers (decode): replaces
// triton_matmul3_transpose of the reference (triton_kernels.py:414-564) and the two
// per-call Quantizer.dequantize launches in front of it.
//
// Same algebra as gemv_stream.cu (scale folded into the activations, one correction per
// residue), adapted to the 3-bit layout: an int32 word holds ten codes of ONE input column
// (rows 10R .. 10R+9), and because 10 does not divide G the slot of a residue drifts from
// group member to group member.  Storage rows R and R + P3 (P3 = G / gcd(G, 10)) hold the
// same ten residues in the same slots, so a pass is: storage-row class rho (R = rho + i*P3,
// the <= 16 "members" are the MMA's rows) x 64 input columns.  Lane (g, t) loads 16 bytes
// (4 columns) of members g and g+8 for each of the 4 column quarters; two words are merged
// with PRMT and one LOP3 per slot yields the fp16 pair OFFSET + code.  Ten slot MMAs (each
// with its own accumulator tile, columns = slots) and two correction MMAs per 16 columns.
// One row of x per launch.
#include <type_traits>

#include "common.cuh"
#include "kernels.cuh"

namespace hqm {
namespace s3 {

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t and_or(uint32_t v, uint32_t mask, uint32_t magic) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(v), "r"(mask), "r"(magic));
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
__device__ __forceinline__ __half2 bf16pair_to_h2(uint32_t v) {
    return __floats2half2_rn(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ __half2 meta_decode(uint32_t two_bytes_as_h2, __half2 mz, __half2 ms) {
    const __half2 q = __hsub2(bits_h2(two_bytes_as_h2), bits_h2(0x64006400u));   // exact
    return __hmul2(__hsub2(q, mz), ms);
}

struct Consts {
    uint32_t mask3, mask6;     // 3-bit field at bits 5-3 / 8-6 of each half
    uint32_t magic3, magic6;   // 128.0 / 16.0 in both halves: the field's lowest bit weighs 1
};

// Passes are numbered L = rho * PT + p; warp c of the grid owns [c*total/warps, (c+1)*total/warps).
struct Split3 {
    int P3, PT, warps;
    __host__ __device__ uint32_t total() const { return (uint32_t)P3 * (uint32_t)PT; }
    __host__ __device__ uint32_t begin(int c) const { return (uint32_t)c * total() / (uint32_t)warps; }
    __host__ __device__ int owner(uint32_t L) const {
        int c = (int)(L * (uint32_t)warps / total());
        while (c + 1 < warps && begin(c + 1) <= L) ++c;
        while (c > 0 && begin(c) > L) --c;
        return c;
    }
};

constexpr int ROW = 72;            // 64 columns + padding (halfs)
constexpr int XPASS = 8;           // longest range of a warp, in passes
constexpr int NW = 8;
// per warp: xs[10][ROW], zz[10 + 1][ROW] (row 10 zero), x staging [XPASS * 64]
constexpr int WARP_HALFS = 21 * ROW + XPASS * 64;

// The ten fp16 pairs OFFSET + code of two words (two adjacent columns k, k+1), slot s in out[s].
// lo = low halves of both words (slots 9..5 at bits 0,3,..,12), hi = the same of the words >> 15
// (slots 4..0).  Fields at bits 3 and 6 are used in place; bit 0 is moved up by 3, bits 9 and 12 down by 6.
__device__ __forceinline__ void ten_pairs(uint32_t w0, uint32_t w1, const Consts& c, uint32_t (&out)[10]) {
    const uint32_t lo = prmt(w0, w1, 0x5410u), hi = prmt(w0 >> 15, w1 >> 15, 0x5410u);
    const uint32_t lo_up = lo << 3, lo_dn = lo >> 6, hi_up = hi << 3, hi_dn = hi >> 6;
    out[9] = and_or(lo_up, c.mask3, c.magic3);   // bit 0  -> 3
    out[8] = and_or(lo, c.mask3, c.magic3);      // bit 3
    out[7] = and_or(lo, c.mask6, c.magic6);      // bit 6
    out[6] = and_or(lo_dn, c.mask3, c.magic3);   // bit 9  -> 3
    out[5] = and_or(lo_dn, c.mask6, c.magic6);   // bit 12 -> 6
    out[4] = and_or(hi_up, c.mask3, c.magic3);
    out[3] = and_or(hi, c.mask3, c.magic3);
    out[2] = and_or(hi, c.mask6, c.magic6);
    out[1] = and_or(hi_dn, c.mask3, c.magic3);
    out[0] = and_or(hi_dn, c.mask6, c.magic6);
}
// offset (fp16 bits) that ten_pairs adds to slot s
__host__ __device__ constexpr uint32_t slot_offset(int s) { return (s == 7 || s == 5 || s == 2 || s == 0) ? 0x4C00u : 0x5800u; }

__global__ void __launch_bounds__(256, 2)
gemv_stream3_kernel(float* __restrict__ partial, const uint16_t* __restrict__ x, const int32_t* __restrict__ x_idx,
                    int m, int M_total, hqm_weight w, int G, int C, int rows, Split3 sp, Consts cc) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int K = w.K, N = w.N, P3 = sp.P3, PT = sp.PT;
    __half* xs_w = reinterpret_cast<__half*>(smem_raw) + wi * WARP_HALFS;   // [10][ROW]
    __half* zz_w = xs_w + 10 * ROW;                                          // [11][ROW], row 10 stays zero
    __half* xh = zz_w + 11 * ROW;                                            // [XPASS * 64]
    grid_launch_dependents();                       // overlapped launch: set-up runs under the kernel in front
    for (int i = lane; i < 21 * ROW / 2; i += 32) reinterpret_cast<uint32_t*>(xs_w)[i] = 0u;
    __syncwarp();
    grid_dependency_wait();                         // x, the row index and the partial buffer belong to earlier kernels

    const uint16_t* xr = x + (int64_t)(x_idx ? x_idx[m] : m) * K;
    const uint32_t* Wq = reinterpret_cast<const uint32_t*>(w.W_q);
    // correction tile: rows 0..7 = z of slot g (tile 0) or of slots 8, 9 (tile 1), rows 8..15 = the offsets
    const int zrow0 = g * ROW + 16 * t;
    const int zrow1 = (g < 2 ? 8 + g : 10) * ROW + 16 * t;
    const uint32_t off0 = slot_offset(g) * 0x00010001u;
    const uint32_t off1 = g < 2 ? slot_offset(8 + g) * 0x00010001u : 0u;

    const int gw = blockIdx.x * NW + wi;
    const uint32_t L_begin = sp.begin(gw), L_end = sp.begin(gw + 1);
    for (uint32_t L = L_begin; L < L_end;) {
        const int rho = (int)(L / (uint32_t)PT), pa = (int)(L - (uint32_t)rho * (uint32_t)PT);
        const int pb = min(PT, pa + (int)(L_end - L));
        L += (uint32_t)(pb - pa);

        // this segment's columns of x as fp16
        for (int i = lane * 2; i < (pb - pa) * 64; i += 64)
            *reinterpret_cast<__half2*>(xh + i) = bf16pair_to_h2(*reinterpret_cast<const uint32_t*>(xr + pa * 64 + i));
        __syncwarp();

        float acc[10][4];
        float accc[2][4];
#pragma unroll
        for (int s = 0; s < 10; ++s)
#pragma unroll
            for (int v = 0; v < 4; ++v) acc[s][v] = 0.f;
#pragma unroll
        for (int v = 0; v < 4; ++v) accc[0][v] = accc[1][v] = 0.f;

        // members of this lane: storage rows rho + g*P3 and rho + (g+8)*P3 (absent ones read as zero codes)
        const int64_t R0 = (int64_t)rho + (int64_t)g * P3, R1 = R0 + (int64_t)8 * P3;
        const bool has0 = R0 < rows, has1 = R1 < rows;
        const uint32_t* row0 = Wq + R0 * K + 4 * t;
        const uint32_t* row1 = Wq + R1 * K + 4 * t;

        for (int p = pa; p < pb; ++p) {
            const int k0 = p * 64;
            // ---- weight words of the pass: 4 column quarters x 2 members
            uint4 q0[4], q1[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                q0[j] = has0 ? ld_stream_16(row0 + k0 + 16 * j) : make_uint4(0u, 0u, 0u, 0u);
                q1[j] = has1 ? ld_stream_16(row1 + k0 + 16 * j) : make_uint4(0u, 0u, 0u, 0u);
            }
            // ---- decode scale / zero: 80 tasks (10 slots x 8 column octets) over 3 rounds of 32 lanes
#pragma unroll
            for (int rnd = 0; rnd < 3; ++rnd) {
                const int task = rnd * 32 + lane;
                if (task < 80) {
                    const int sd = task >> 3, kd = (task & 7) * 8;
                    const uint32_t r = (uint32_t)(10 * rho + sd) % (uint32_t)G;
                    const uint32_t idx = r * (uint32_t)K + (uint32_t)(k0 + kd);
                    const uint32_t col = idx % (uint32_t)C;
                    const uint2 sq = *reinterpret_cast<const uint2*>(w.scale_q + idx);
                    const uint2 zq = *reinterpret_cast<const uint2*>(w.zero_q + idx);
                    const uint4 mss = *reinterpret_cast<const uint4*>(w.ms_scale + col);
                    const uint4 mzs = *reinterpret_cast<const uint4*>(w.mz_scale + col);
                    const uint4 msz = *reinterpret_cast<const uint4*>(w.ms_zero + col);
                    const uint4 mzz = *reinterpret_cast<const uint4*>(w.mz_zero + col);
                    const uint32_t sqw[2] = {sq.x, sq.y}, zqw[2] = {zq.x, zq.y};
                    const uint32_t a_ms[4] = {mss.x, mss.y, mss.z, mss.w}, a_mz[4] = {mzs.x, mzs.y, mzs.z, mzs.w};
                    const uint32_t b_ms[4] = {msz.x, msz.y, msz.z, msz.w}, b_mz[4] = {mzz.x, mzz.y, mzz.z, mzz.w};
                    const uint4 xv = *reinterpret_cast<const uint4*>(xh + (p - pa) * 64 + kd);
                    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
                    uint32_t z2[4], xs2[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t sel = (j & 1) ? 0x4342u : 0x4140u;
                        const __half2 s2 = meta_decode(prmt(sqw[j / 2], 0x64646464u, sel), bits_h2(a_mz[j]), bits_h2(a_ms[j]));
                        z2[j] = h2_bits(meta_decode(prmt(zqw[j / 2], 0x64646464u, sel), bits_h2(b_mz[j]), bits_h2(b_ms[j])));
                        xs2[j] = h2_bits(__hmul2(bits_h2(xw[j]), s2));
                    }
                    *reinterpret_cast<uint4*>(zz_w + sd * ROW + kd) = make_uint4(z2[0], z2[1], z2[2], z2[3]);
                    *reinterpret_cast<uint4*>(xs_w + sd * ROW + kd) = make_uint4(xs2[0], xs2[1], xs2[2], xs2[3]);
                }
            }
            __syncwarp();
            // ---- MMAs: per column quarter j the lane's 4 columns are (k, k+1) [a0/a1, b0] and (k+2, k+3) [a2/a3, b1]
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kq = 16 * j + 4 * t;
                // B: xs of slot g (tile 0) / slot 8+g for g < 2, zeros otherwise (tile 1), at this lane's 4 columns
                const uint2 bt0 = *reinterpret_cast<const uint2*>(xs_w + g * ROW + kq);
                const uint2 bt1 = *reinterpret_cast<const uint2*>((g < 2 ? xs_w + (8 + g) * ROW : zz_w + 10 * ROW) + kq);
                const uint2 zt0 = *reinterpret_cast<const uint2*>(zz_w + zrow0 - 16 * t + kq);
                const uint2 zt1 = *reinterpret_cast<const uint2*>(zz_w + zrow1 - 16 * t + kq);
                mma_f16(accc[0], zt0.x, off0, zt0.y, off0, bt0.x, bt0.y);
                mma_f16(accc[1], zt1.x, off1, zt1.y, off1, bt1.x, bt1.y);
                uint32_t a_lo0[10], a_hi0[10], a_lo1[10], a_hi1[10];
                ten_pairs(q0[j].x, q0[j].y, cc, a_lo0);
                ten_pairs(q0[j].z, q0[j].w, cc, a_hi0);
                ten_pairs(q1[j].x, q1[j].y, cc, a_lo1);
                ten_pairs(q1[j].z, q1[j].w, cc, a_hi1);
#pragma unroll
                for (int s = 0; s < 8; ++s) mma_f16(acc[s], a_lo0[s], a_lo1[s], a_hi0[s], a_hi1[s], bt0.x, bt0.y);
                mma_f16(acc[8], a_lo0[8], a_lo1[8], a_hi0[8], a_hi1[8], bt1.x, bt1.y);
                mma_f16(acc[9], a_lo0[9], a_lo1[9], a_hi0[9], a_hi1[9], bt1.x, bt1.y);
            }
            __syncwarp();
        }

        // ---- epilogue.  Tile of slot s: its valid column is s (tile 0) or s - 8 (tile 1); lane (g, t) holds
        // columns 2t and 2t+1, rows g and g+8.  Correction column n is valid in the lane whose row is n.
        const int slot_idx = gw - sp.owner((uint32_t)rho * (uint32_t)PT);
        float* dst = partial + ((int64_t)slot_idx * M_total + m) * N;
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
            // correction of column n (slot 8*tile + n) sits in lane (g = n, t = n / 2): register n & 1 (+2 for the offsets row)
            const float mine = (g & 1) ? accc[tile][1] + accc[tile][3] : accc[tile][0] + accc[tile][2];
            const float ca = __shfl_sync(0xffffffffu, mine, (2 * t) * 4 + t);           // column 2t:   lane (g = 2t, t)
            const float cb = __shfl_sync(0xffffffffu, mine, (2 * t + 1) * 4 + t);       // column 2t+1: lane (g = 2t+1, t)
#pragma unroll
            for (int s = 0; s < 10; ++s) {
                if ((s >> 3) != tile) continue;
                const int col = s & 7;
                if ((col >> 1) != t) continue;
                const float corr = (col & 1) ? cb : ca;
                const float v0 = ((col & 1) ? acc[s][1] : acc[s][0]) - corr;          // row g
                const float v1 = ((col & 1) ? acc[s][3] : acc[s][2]) - corr;          // row g + 8
                const int64_t n0 = 10 * R0 + s, n1 = 10 * R1 + s;
                if (has0 && n0 < N) dst[n0] = v0;
                if (has1 && n1 < N) dst[n1] = v1;
            }
        }
        __syncwarp();
    }
}

// y[m, n] = bf16( sum of the partial row-sets of row n's storage-row class + bias )
__global__ void finalize3_kernel(uint16_t* __restrict__ y, const float* __restrict__ partial,
                                 const uint16_t* __restrict__ bias, int64_t MN, int N, Split3 sp) {
    grid_launch_dependents();
    grid_dependency_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < MN; i += (int64_t)gridDim.x * blockDim.x) {
        const int n = (int)(i % N);
        const uint32_t rho = (uint32_t)((n / 10) % sp.P3);
        const int cnt = sp.owner(rho * sp.PT + sp.PT - 1) - sp.owner(rho * sp.PT) + 1;
        float v = 0.f;
        for (int s = 0; s < cnt; ++s) v += partial[s * MN + i];
        if (bias) v += bf16_bits_to_float(bias[n]);
        y[i] = float_to_bf16_bits(v);
    }
}

}  // namespace s3

static int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

bool gemv_stream3_plan(const hqm_weight* w, int G, int C, int64_t M, Stream3Plan* plan) {
    if (w->nbits != 3 || M < 1 || M > 16 || !meta_uniform(w)) return false;
    if (w->K % 64 != 0 || C % 8 != 0) return false;
    const int rows = (w->N + 9) / 10;
    const int P3 = G / gcd_int(G, 10);
    if ((rows + P3 - 1) / P3 > 16) return false;                          // the members must fit one MMA row block
    if ((int64_t)G * w->K >= ((int64_t)1 << 31) || (int64_t)rows * w->K >= ((int64_t)1 << 29)) return false;
    const void* ptrs[] = {w->W_q, w->scale_q, w->zero_q, w->ms_scale, w->mz_scale, w->ms_zero, w->mz_zero};
    for (const void* p : ptrs)
        if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return false;
    static int resident_dev[MAX_DEVICES];         // 0: not queried yet, otherwise CTAs per SM + 1
    int& res_slot = resident_dev[current_device_slot()];
    int resident = res_slot - 1;
    const size_t smem = (size_t)s3::NW * s3::WARP_HALFS * sizeof(__half);
    if (resident < 0) {
        resident = 0;
        int per_sm = 0;
        if (cudaFuncSetAttribute(s3::gemv_stream3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, s3::gemv_stream3_kernel, 256, smem) == cudaSuccess)
            resident = per_sm;
        else
            cudaGetLastError();
        res_slot = resident + 1;
    }
    if (resident < 1) return false;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    plan->P3 = P3;
    plan->PT = w->K / 64;
    plan->rows = rows;
    const int64_t total = (int64_t)P3 * plan->PT;
    int per_sm = resident;
    const int64_t want = total / ((int64_t)sms * 8 * 3);
    if (per_sm > want) per_sm = (int)(want < 1 ? 1 : want);
    int grid = per_sm * sms;
    if ((int64_t)grid * 8 * 3 > total) grid = (int)(total / (8 * 3));
    if (grid < 1) grid = 1;
    if ((int64_t)grid * 8 > total) return false;
    const int64_t warps = (int64_t)grid * 8;
    if (total * warps >= ((int64_t)1 << 31) || (total + warps - 1) / warps + 1 > s3::XPASS) return false;
    plan->grid = grid;
    plan->warps = (int)warps;
    const int64_t min_range = total / warps;
    plan->slots = (int)((plan->PT + min_range - 1) / min_range) + 1;
    return true;
}

size_t gemv_stream3_scratch_bytes(const Stream3Plan& plan, int64_t M, int N) {
    return ((size_t)plan.slots * (size_t)M * (size_t)N * sizeof(float) + 255) / 256 * 256;
}

int launch_gemv_stream3(uint16_t* y, float* partial, const uint16_t* x, const int32_t* x_idx, int64_t M,
                        const hqm_weight* w, const uint16_t* bias, int G, int C, const Stream3Plan& plan,
                        cudaStream_t st) {
    const s3::Split3 sp{plan.P3, plan.PT, plan.warps};
    const s3::Consts cc{0x00380038u, 0x01C001C0u, 0x58005800u, 0x4C004C00u};
    const size_t smem = (size_t)s3::NW * s3::WARP_HALFS * sizeof(__half);
    for (int m = 0; m < (int)M; ++m) {
        launch_overlapped(s3::gemv_stream3_kernel, plan.grid, 256, smem, st, partial, x, x_idx, m, (int)M, *w, G, C,
                          plan.rows, sp, cc);
        HQM_LAUNCH_CHECK();
    }
    const int64_t MN = M * w->N;
    int64_t blocks = (MN + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    launch_overlapped(s3::finalize3_kernel, (int)blocks, 256, 0, st, y, (const float*)partial, bias, MN, w->N, sp);
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

}  // namespace hqm
