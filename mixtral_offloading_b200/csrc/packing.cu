// Bit packing kernels: the layouts of src/packing.py (pack_/unpack_*_common).
// Pure byte work, HBM bound: each thread moves 16 input columns of one storage
// row with 128-bit accesses; a scalar variant covers K % 16 != 0 or unaligned
// buffers.  Results are bit exact by construction.
#include "common.cuh"

namespace hqm {

// ---- 4-bit and 2-bit (uint8 storage) --------------------------------------
// PER codes of BITS bits per byte; row PER*R + i sits at bits BITS*(PER-1-i).
template <int BITS, int PER, typename V>
__global__ void unpack_u8_kernel(uint8_t* __restrict__ codes, const uint8_t* __restrict__ packed, int64_t rows,
                                 int64_t K) {
    constexpr int W = sizeof(V);
    const int64_t chunks = K / W;
    const int64_t total = rows * chunks;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t R = i / chunks, k = (i % chunks) * W;
        V in = *reinterpret_cast<const V*>(packed + R * K + k);
        const uint8_t* ib = reinterpret_cast<const uint8_t*>(&in);
#pragma unroll
        for (int s = 0; s < PER; ++s) {
            V out;
            uint8_t* ob = reinterpret_cast<uint8_t*>(&out);
#pragma unroll
            for (int b = 0; b < W; ++b) ob[b] = (ib[b] >> (BITS * (PER - 1 - s))) & ((1 << BITS) - 1);
            *reinterpret_cast<V*>(codes + (R * PER + s) * K + k) = out;
        }
    }
}

template <int BITS, int PER, typename V>
__global__ void pack_u8_kernel(uint8_t* __restrict__ packed, const uint8_t* __restrict__ codes, int64_t rows,
                               int64_t K) {
    constexpr int W = sizeof(V);
    const int64_t chunks = K / W;
    const int64_t total = rows * chunks;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t R = i / chunks, k = (i % chunks) * W;
        V out;
        uint8_t* ob = reinterpret_cast<uint8_t*>(&out);
#pragma unroll
        for (int b = 0; b < W; ++b) ob[b] = 0;
#pragma unroll
        for (int s = 0; s < PER; ++s) {
            V in = *reinterpret_cast<const V*>(codes + (R * PER + s) * K + k);
            const uint8_t* ib = reinterpret_cast<const uint8_t*>(&in);
#pragma unroll
            for (int b = 0; b < W; ++b) ob[b] |= (uint8_t)(ib[b] << (BITS * (PER - 1 - s)));
        }
        *reinterpret_cast<V*>(packed + R * K + k) = out;
    }
}

// ---- 3-bit (int32 storage, 10 codes per word) ------------------------------
// One thread per 4 columns of one storage row: reads 4 words (16 B), writes ten
// 4-byte groups.  VEC = 1 is the scalar variant.
template <int VEC>
__global__ void unpack_3bit_kernel(uint8_t* __restrict__ codes, const int32_t* __restrict__ packed, int64_t rows,
                                   int64_t K) {
    const int64_t chunks = K / VEC;
    const int64_t total = rows * chunks;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t R = i / chunks, k = (i % chunks) * VEC;
        uint32_t w[VEC];
        if (VEC == 4) {
            uint4 v = *reinterpret_cast<const uint4*>(packed + R * K + k);
            w[0] = v.x; w[1 % VEC] = v.y; w[2 % VEC] = v.z; w[3 % VEC] = v.w;
        } else {
            w[0] = (uint32_t)packed[R * K + k];
        }
#pragma unroll
        for (int s = 0; s < 10; ++s) {
            uint8_t o[VEC];
#pragma unroll
            for (int b = 0; b < VEC; ++b) o[b] = (w[b] >> (3 * (9 - s))) & 7u;
            uint8_t* dst = codes + (R * 10 + s) * K + k;
            if (VEC == 4) {
                *reinterpret_cast<uint32_t*>(dst) = (uint32_t)o[0] | ((uint32_t)o[1 % VEC] << 8) |
                                                     ((uint32_t)o[2 % VEC] << 16) | ((uint32_t)o[3 % VEC] << 24);
            } else {
                dst[0] = o[0];
            }
        }
    }
}

// Rows past N inside the last word stay zero (packing.py:66-77).
template <int VEC>
__global__ void pack_3bit_kernel(int32_t* __restrict__ packed, const uint8_t* __restrict__ codes, int64_t N,
                                 int64_t rows, int64_t K) {
    const int64_t chunks = K / VEC;
    const int64_t total = rows * chunks;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t R = i / chunks, k = (i % chunks) * VEC;
        uint32_t w[VEC];
#pragma unroll
        for (int b = 0; b < VEC; ++b) w[b] = 0;
#pragma unroll
        for (int s = 0; s < 10; ++s) {
            const int64_t n = R * 10 + s;
            if (n < N) {
                const uint8_t* src = codes + n * K + k;
                if (VEC == 4) {
                    uint32_t v = *reinterpret_cast<const uint32_t*>(src);
#pragma unroll
                    for (int b = 0; b < VEC; ++b) w[b] |= ((v >> (8 * b)) & 7u) << (3 * (9 - s));
                } else {
                    w[0] |= ((uint32_t)src[0] & 7u) << (3 * (9 - s));
                }
            }
        }
        if (VEC == 4) {
            *reinterpret_cast<uint4*>(packed + R * K + k) = make_uint4(w[0], w[1 % VEC], w[2 % VEC], w[3 % VEC]);
        } else {
            packed[R * K + k] = (int32_t)w[0];
        }
    }
}

static inline int grid_for(int64_t total, int threads) {
    int64_t blocks = (total + threads - 1) / threads;
    const int64_t cap = 148 * 16;  // a few waves of the 148 SMs; the kernels are grid-stride
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

template <int BITS, int PER>
static int unpack_u8(uint8_t* codes, const uint8_t* packed, int64_t rows, int64_t K, void* stream) {
    HQM_CHECK_ARG(rows >= 0 && K >= 0, "unpack: negative size");
    if (rows == 0 || K == 0) return HQM_OK;
    HQM_CHECK_ARG(codes && packed, "unpack: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    if (K % 16 == 0 && aligned16(codes) && aligned16(packed)) {
        unpack_u8_kernel<BITS, PER, uint4><<<grid_for(rows * (K / 16), 256), 256, 0, st>>>(codes, packed, rows, K);
    } else {
        unpack_u8_kernel<BITS, PER, uint8_t><<<grid_for(rows * K, 256), 256, 0, st>>>(codes, packed, rows, K);
    }
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

template <int BITS, int PER>
static int pack_u8(uint8_t* packed, const uint8_t* codes, int64_t N, int64_t K, void* stream) {
    HQM_CHECK_ARG(N >= 0 && K >= 0 && N % PER == 0, "pack: the row count must be a multiple of %d", PER);
    if (N == 0 || K == 0) return HQM_OK;
    HQM_CHECK_ARG(codes && packed, "pack: null pointer");
    const int64_t rows = N / PER;
    cudaStream_t st = (cudaStream_t)stream;
    if (K % 16 == 0 && aligned16(codes) && aligned16(packed)) {
        pack_u8_kernel<BITS, PER, uint4><<<grid_for(rows * (K / 16), 256), 256, 0, st>>>(packed, codes, rows, K);
    } else {
        pack_u8_kernel<BITS, PER, uint8_t><<<grid_for(rows * K, 256), 256, 0, st>>>(packed, codes, rows, K);
    }
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

}  // namespace hqm

extern "C" {

int hqm_pack_4bit_u8(uint8_t* packed, const uint8_t* codes, int64_t N, int64_t K, void* stream) {
    return hqm::pack_u8<4, 2>(packed, codes, N, K, stream);
}
int hqm_unpack_4bit_u8(uint8_t* codes, const uint8_t* packed, int64_t rows, int64_t K, void* stream) {
    return hqm::unpack_u8<4, 2>(codes, packed, rows, K, stream);
}
int hqm_pack_2bit_u8(uint8_t* packed, const uint8_t* codes, int64_t N, int64_t K, void* stream) {
    return hqm::pack_u8<2, 4>(packed, codes, N, K, stream);
}
int hqm_unpack_2bit_u8(uint8_t* codes, const uint8_t* packed, int64_t rows, int64_t K, void* stream) {
    return hqm::unpack_u8<2, 4>(codes, packed, rows, K, stream);
}

int hqm_pack_3bit_i32(int32_t* packed, const uint8_t* codes, int64_t N, int64_t K, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(N >= 0 && K >= 0, "pack_3bit: negative size");
    if (N == 0 || K == 0) return HQM_OK;
    HQM_CHECK_ARG(codes && packed, "pack_3bit: null pointer");
    HQM_CHECK_ARG(aligned4(packed), "pack_3bit: packed must be 4-byte aligned");
    const int64_t rows = (N + 9) / 10;
    cudaStream_t st = (cudaStream_t)stream;
    if (K % 4 == 0 && aligned16(packed) && aligned4(codes)) {
        pack_3bit_kernel<4><<<grid_for(rows * (K / 4), 256), 256, 0, st>>>(packed, codes, N, rows, K);
    } else {
        pack_3bit_kernel<1><<<grid_for(rows * K, 256), 256, 0, st>>>(packed, codes, N, rows, K);
    }
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

int hqm_unpack_3bit_i32(uint8_t* codes, const int32_t* packed, int64_t rows, int64_t K, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(rows >= 0 && K >= 0, "unpack_3bit: negative size");
    if (rows == 0 || K == 0) return HQM_OK;
    HQM_CHECK_ARG(codes && packed, "unpack_3bit: null pointer");
    HQM_CHECK_ARG(aligned4(packed), "unpack_3bit: packed must be 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (K % 4 == 0 && aligned16(packed) && aligned4(codes)) {
        unpack_3bit_kernel<4><<<grid_for(rows * (K / 4), 256), 256, 0, st>>>(codes, packed, rows, K);
    } else {
        unpack_3bit_kernel<1><<<grid_for(rows * K, 256), 256, 0, st>>>(codes, packed, rows, K);
    }
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

}  // extern "C"
