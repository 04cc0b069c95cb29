// hqm_linear_static_scratch: the quantized linear for callers that cannot provide a
// workspace.
//
// hqm_linear needs a caller-owned scratch buffer for the fp32 partial sums of its
// streaming kernel, and the usual caller (the Python layer) gets it from torch's
// allocator.  Some callers cannot do that: code running while a CUDA stream is being
// captured (cudaMalloc is not permitted there and would synchronise the device
// anyway), hosts written in another language that hand this library raw pointers but
// own no device allocator of their own, and serving loops that have frozen their
// memory plan.  For them this file keeps ONE fixed workspace inside the library image:
// a file-scope __device__ array that every GPU loading the library holds until the
// process exits.  Nothing here calls cudaMalloc, cudaFree or any allocating routine.
//
// The array's name is only a host-side handle, not a device address, so the address is
// looked up once per device with cudaGetSymbolAddress (with that device current) and
// that pointer is what the kernels receive.
#include <mutex>

#include "common.cuh"
#include "kernels.cuh"

namespace hqm {

// 2 MiB: enough for the decode-sized calls this entry point is meant for (a Mixtral
// expert projection, 14336 x 4096, needs ~172 KB per row of x).
constexpr size_t STATIC_SCRATCH_BYTES = 2u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

static void* g_static_ptr[MAX_DEVICES] = {};
static std::mutex g_static_mutex;

// Device address of the workspace on the current device; looked up on first use.
static int static_scratch_ptr(void** out) {
    int dev = 0;
    HQM_CUDA(cudaGetDevice(&dev));
    HQM_CHECK_ARG(dev >= 0 && dev < MAX_DEVICES, "static scratch: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        HQM_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        HQM_CHECK_ARG(p != nullptr, "static scratch: cudaGetSymbolAddress returned a null address");
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return HQM_OK;
}

}  // namespace hqm

extern "C" {

size_t hqm_static_scratch_capacity(void) { return hqm::STATIC_SCRATCH_BYTES; }

int hqm_linear_static_scratch(uint16_t* y, const uint16_t* x, int64_t M, const hqm_weight* w, const uint16_t* bias,
                              void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(M >= 0 && M <= INT32_MAX, "linear: bad row count %lld", (long long)M);
    HQM_CHECK_ARG(M == 0 || (y && x), "linear: null activation pointer");
    const size_t inner = linear_scratch_bytes(M, w);
    const size_t need = inner ? inner + SCRATCH_HEADER : 0;
    if (need > STATIC_SCRATCH_BYTES) {
        set_error("linear_static_scratch: this call needs %zu bytes of workspace but the built-in one holds %zu; "
                  "use hqm_linear with a caller-provided buffer", need, (size_t)STATIC_SCRATCH_BYTES);
        return HQM_ERR_SCRATCH;
    }
    void* ws = nullptr;
    if (need > 0) {
        const int rc = static_scratch_ptr(&ws);
        if (rc != HQM_OK) return rc;
    }
    // Every partial sum that is read was written earlier in the same call, so the workspace needs no
    // clearing although it still holds the previous call's contents.  The only part that must start at
    // zero is the header (arrival counters); the array is zero when the library is loaded and every call
    // leaves the header zero again.
    if (ws == nullptr) return launch_linear(y, x, nullptr, M, w, bias, nullptr, nullptr, 0, (cudaStream_t)stream);
    return launch_linear(y, x, nullptr, M, w, bias, (uint32_t*)ws, (uint8_t*)ws + SCRATCH_HEADER, inner,
                         (cudaStream_t)stream);
}

}  // extern "C"
