// Shared helpers for the sm_100a kernels: error reporting, dtype conversion,
// layout arithmetic of the packed weight format.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/hqq_moe.h"

namespace hqm {

// Message of the calling thread's last failure (returned by hqm_last_error()).
void set_error(const char* fmt, ...);
// Counts kernel launches made by the library (read by hqm_launch_count()).
void count_launch();

#define HQM_CHECK_ARG(cond, ...)          \
    do {                                  \
        if (!(cond)) {                    \
            hqm::set_error(__VA_ARGS__);  \
            return HQM_ERR_ARG;           \
        }                                 \
    } while (0)

#define HQM_CUDA(call)                                                                    \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            hqm::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return HQM_ERR_CUDA;                                                          \
        }                                                                                 \
    } while (0)

#define HQM_LAUNCH_CHECK()                                                                \
    do {                                                                                  \
        cudaError_t e_ = cudaGetLastError();                                              \
        hqm::count_launch();                                                              \
        if (e_ != cudaSuccess) {                                                          \
            hqm::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e_), __FILE__, __LINE__); \
            return HQM_ERR_CUDA;                                                          \
        }                                                                                 \
    } while (0)

// Index of the current device for per-device caches (function attributes and occupancy are per device).
constexpr int MAX_DEVICES = 64;
inline int current_device_slot() {
    int dev = 0;
    cudaGetDevice(&dev);
    return (dev >= 0 && dev < MAX_DEVICES) ? dev : 0;
}

__host__ __device__ constexpr int codes_per_word(int nbits) { return nbits == 2 ? 4 : (nbits == 4 ? 2 : 10); }

// Storage rows of W_q for N output rows.
__host__ __device__ inline int64_t storage_rows(int64_t N, int nbits) {
    int per = codes_per_word(nbits);
    return (N + per - 1) / per;
}

// Validates a weight descriptor; fills G (groups along N) and C (columns of the
// (meta_group, C) view of the flat scale vector; zero_meta_cols() gives the zero vector's).
int check_weight(const hqm_weight* w, int* G, int* C);
// The streaming and tensor-core kernels track ONE meta column for scale and zero: they take layers whose two
// meta group sizes are equal; the others go to the shape-agnostic kernel.
inline bool meta_uniform(const hqm_weight* w) { return w->meta_group_zero == 0 || w->meta_group_zero == w->meta_group; }
__host__ __device__ inline int64_t zero_meta_cols(const hqm_weight& w, int G) {
    const int64_t mg = w.meta_group_zero > 0 ? w.meta_group_zero : w.meta_group;
    return (int64_t)G * w.K / mg;
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
__device__ __forceinline__ float f16_bits_to_float(uint16_t b) { return __half2float(__ushort_as_half(b)); }
__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float round_bf16(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Streaming 16-byte load that does not pollute L1 (weights are read exactly once).
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// ---- programmatic dependent launch ----------------------------------------------------------------
// A kernel launched with launch_overlapped() may become resident while the kernel in front of it on the
// stream is still running.  Whatever it does before grid_dependency_wait() overlaps that kernel (set-up
// work, and reads of memory the kernels in front never write); grid_dependency_wait() returns once
// every earlier kernel has completed and its writes are visible.  grid_launch_dependents() tells the
// scheduler that the NEXT kernel may be made resident.  Both are no-ops in a kernel launched the plain way,
// and a kernel launched the plain way still waits for the whole of its predecessor.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// HQM_NO_OVERLAP=1 in the environment turns launch_overlapped() into a plain launch.
bool overlap_enabled();

// `cluster` > 1 launches thread-block clusters of that many CTAs along x (the grid must be a multiple).
template <typename... Params, typename... Args>
inline cudaError_t launch_overlapped_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                             int cluster, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (overlap_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}
template <typename... Params, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args&&... args) {
    return launch_overlapped_cluster(kernel, grid, block, smem, 1, st, static_cast<Args&&>(args)...);
}

}  // namespace hqm
