// Shape-agnostic quantized linear and full dequantisation.
//
// linear_generic_kernel is the path for layers whose shape the streaming
// kernels (gemv_stream.cu) do not cover.  It decodes scale and zero per element
// from their 8-bit form, so it is instruction bound, not HBM bound; it exists
// for generality and as an independent check of the fast kernels.
#include "common.cuh"
#include "kernels.cuh"

namespace hqm {

__device__ __forceinline__ void decode_scale_zero(const hqm_weight& w, int64_t idx, int C, int64_t Cz, float& s,
                                                  float& z) {
    const int col = (int)(idx % C);
    const int64_t colz = (Cz == C) ? col : idx % Cz;
    // explicit rounding steps (no fused multiply-add) so the fp32 result equals the CPU restatement bit for bit
    s = __fmul_rn(__fsub_rn((float)w.scale_q[idx], f16_bits_to_float(w.mz_scale[col])), f16_bits_to_float(w.ms_scale[col]));
    z = __fmul_rn(__fsub_rn((float)w.zero_q[idx], f16_bits_to_float(w.mz_zero[colz])), f16_bits_to_float(w.ms_zero[colz]));
}

template <int NBITS>
__device__ __forceinline__ uint32_t load_word(const hqm_weight& w, int64_t R, int64_t k) {
    if (NBITS == 3) return (uint32_t) reinterpret_cast<const int32_t*>(w.W_q)[R * w.K + k];
    return (uint32_t) reinterpret_cast<const uint8_t*>(w.W_q)[R * w.K + k];
}

// One warp per storage row (PER output rows), lanes strided over k, MT rows of x
// per pass.  x rows may be gathered through x_idx.
template <int NBITS, int MT>
__global__ void __launch_bounds__(256)
linear_generic_kernel(uint16_t* __restrict__ y, const uint16_t* __restrict__ x, const int32_t* __restrict__ x_idx,
                      int M, hqm_weight w, int G, int C, const uint16_t* __restrict__ bias) {
    constexpr int PER = codes_per_word(NBITS);
    constexpr uint32_t MASK = (1u << NBITS) - 1u;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t R = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    const int64_t rows = storage_rows(w.N, NBITS);
    if (R >= rows) return;
    const int m0 = blockIdx.y * MT;
    const int K = w.K;
    const int64_t Cz = zero_meta_cols(w, G);

    const uint16_t* xr[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const int mm = (m0 + m < M) ? (m0 + m) : (M - 1);
        xr[m] = x + (int64_t)(x_idx ? x_idx[mm] : mm) * K;
    }
    float acc[PER][MT];
#pragma unroll
    for (int s = 0; s < PER; ++s)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[s][m] = 0.f;

    for (int k = lane; k < K; k += 32) {
        const uint32_t word = load_word<NBITS>(w, R, k);
        float xv[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) xv[m] = bf16_bits_to_float(xr[m][k]);
#pragma unroll
        for (int s = 0; s < PER; ++s) {
            const int64_t n = R * PER + s;
            if (n < w.N) {
                const float code = (float)((word >> (NBITS * (PER - 1 - s))) & MASK);
                float sc, zr;
                decode_scale_zero(w, (n % G) * K + k, C, Cz, sc, zr);
                const float wv = (code - zr) * sc;
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[s][m] = fmaf(wv, xv[m], acc[s][m]);
            }
        }
    }
#pragma unroll
    for (int s = 0; s < PER; ++s) {
        const int64_t n = R * PER + s;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float v = warp_sum(acc[s][m]);
            if (lane == 0 && n < w.N && m0 + m < M) {
                const float b = bias ? bf16_bits_to_float(bias[n]) : 0.f;
                y[(int64_t)(m0 + m) * w.N + n] = float_to_bf16_bits(v + b);
            }
        }
    }
}

int launch_linear_generic(uint16_t* y, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w, int G,
                          int C, const uint16_t* bias, cudaStream_t st) {
    constexpr int MT = 4;
    const int64_t rows = storage_rows(w->N, w->nbits);
    dim3 grid((unsigned)((rows + 7) / 8), (unsigned)((M + MT - 1) / MT));
    switch (w->nbits) {
        case 2: linear_generic_kernel<2, MT><<<grid, 256, 0, st>>>(y, x, x_idx, (int)M, *w, G, C, bias); break;
        case 3: linear_generic_kernel<3, MT><<<grid, 256, 0, st>>>(y, x, x_idx, (int)M, *w, G, C, bias); break;
        default: linear_generic_kernel<4, MT><<<grid, 256, 0, st>>>(y, x, x_idx, (int)M, *w, G, C, bias); break;
    }
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

// ---- full dequantisation (HQQLinearTritonSavable.dequantize) ----------------
template <typename T> __device__ __forceinline__ T cast_out(float v);
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }

template <int NBITS, typename T>
__global__ void dequantize_kernel(T* __restrict__ out, hqm_weight w, int G, int C) {
    constexpr int PER = codes_per_word(NBITS);
    constexpr uint32_t MASK = (1u << NBITS) - 1u;
    const int64_t rows = storage_rows(w.N, NBITS);
    const int64_t total = rows * w.K;
    const int64_t Cz = zero_meta_cols(w, G);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t R = i / w.K, k = i % w.K;
        const uint32_t word = load_word<NBITS>(w, R, k);
#pragma unroll
        for (int s = 0; s < PER; ++s) {
            const int64_t n = R * PER + s;
            if (n < w.N) {
                const float code = (float)((word >> (NBITS * (PER - 1 - s))) & MASK);
                float sc, zr;
                decode_scale_zero(w, (n % G) * w.K + k, C, Cz, sc, zr);
                out[n * w.K + k] = cast_out<T>(__fmul_rn(__fsub_rn(code, zr), sc));
            }
        }
    }
}

template <typename T>
static int launch_dequantize(void* out, const hqm_weight* w, int G, int C, cudaStream_t st) {
    const int64_t total = storage_rows(w->N, w->nbits) * w->K;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    switch (w->nbits) {
        case 2: dequantize_kernel<2, T><<<(int)blocks, 256, 0, st>>>((T*)out, *w, G, C); break;
        case 3: dequantize_kernel<3, T><<<(int)blocks, 256, 0, st>>>((T*)out, *w, G, C); break;
        default: dequantize_kernel<4, T><<<(int)blocks, 256, 0, st>>>((T*)out, *w, G, C); break;
    }
    HQM_LAUNCH_CHECK();
    return HQM_OK;
}

}  // namespace hqm

extern "C" int hqm_dequantize(void* W_out, int out_dtype, const hqm_weight* w, void* stream) {
    using namespace hqm;
    int G, C;
    int rc = check_weight(w, &G, &C);
    if (rc != HQM_OK) return rc;
    HQM_CHECK_ARG(W_out != nullptr, "dequantize: null output");
    cudaStream_t st = (cudaStream_t)stream;
    switch (out_dtype) {
        case 0: return launch_dequantize<__nv_bfloat16>(W_out, w, G, C, st);
        case 1: return launch_dequantize<__half>(W_out, w, G, C, st);
        case 2: return launch_dequantize<float>(W_out, w, G, C, st);
        default: set_error("dequantize: out_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)"); return HQM_ERR_ARG;
    }
}
