// Error reporting, argument validation and the hqm_linear entry point.
#include <stdarg.h>

#include <atomic>

#include "common.cuh"
#include "kernels.cuh"

namespace hqm {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int check_weight(const hqm_weight* w, int* G, int* C) {
    HQM_CHECK_ARG(w != nullptr, "weight descriptor is null");
    HQM_CHECK_ARG(w->nbits == 2 || w->nbits == 3 || w->nbits == 4, "nbits == %d isn't supported (2, 3 or 4)", w->nbits);
    HQM_CHECK_ARG(w->N > 0 && w->K > 0, "weight shape (%d, %d) must be positive", w->N, w->K);
    HQM_CHECK_ARG(w->group_size > 0 && w->N % w->group_size == 0, "N = %d is not a multiple of group_size = %d", w->N,
                  w->group_size);
    if (w->nbits != 3)
        HQM_CHECK_ARG(w->N % codes_per_word(w->nbits) == 0, "N = %d is not a multiple of %d codes per byte", w->N,
                      codes_per_word(w->nbits));
    const int64_t g = w->N / w->group_size;
    const int64_t L = g * (int64_t)w->K;
    HQM_CHECK_ARG(w->meta_group > 0 && L % w->meta_group == 0,
                  "scale/zero length %lld is not a multiple of meta_group = %d", (long long)L, w->meta_group);
    HQM_CHECK_ARG(L / w->meta_group <= INT32_MAX, "scale/zero vector too long");
    HQM_CHECK_ARG(w->W_q && w->scale_q && w->zero_q && w->ms_scale && w->mz_scale && w->ms_zero && w->mz_zero,
                  "weight descriptor holds a null tensor pointer");
    *G = (int)g;
    *C = (int)(L / w->meta_group);
    return HQM_OK;
}

int launch_linear(uint16_t* y, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w,
                  const uint16_t* bias, cudaStream_t st) {
    int G, C;
    int rc = check_weight(w, &G, &C);
    if (rc != HQM_OK) return rc;
    if (M == 0) return HQM_OK;
    return launch_linear_generic(y, x, x_idx, M, w, G, C, bias, st);
}

}  // namespace hqm

extern "C" {

const char* hqm_last_error(void) { return hqm::g_error; }
int hqm_version(void) { return 1; }
int64_t hqm_launch_count(void) { return (int64_t)hqm::launches(); }

size_t hqm_linear_scratch_bytes(int64_t M, const hqm_weight* w) {
    (void)M;
    (void)w;
    return 0;
}

int hqm_linear(uint16_t* y, const uint16_t* x, int64_t M, const hqm_weight* w, const uint16_t* bias, void* scratch,
               size_t scratch_bytes, void* stream) {
    using namespace hqm;
    (void)scratch;
    (void)scratch_bytes;
    HQM_CHECK_ARG(M >= 0 && M <= INT32_MAX, "linear: bad row count %lld", (long long)M);
    HQM_CHECK_ARG(M == 0 || (y && x), "linear: null activation pointer");
    return launch_linear(y, x, nullptr, M, w, bias, (cudaStream_t)stream);
}

}  // extern "C"
