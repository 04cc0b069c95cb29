// Error reporting, argument validation and the hqm_linear entry point.
#include <stdarg.h>
#include <stdlib.h>

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
    HQM_CHECK_ARG(w->meta_group_zero >= 0 && (w->meta_group_zero == 0 || L % w->meta_group_zero == 0),
                  "zero length %lld is not a multiple of meta_group_zero = %d", (long long)L, w->meta_group_zero);
    HQM_CHECK_ARG(w->W_q && w->scale_q && w->zero_q && w->ms_scale && w->mz_scale && w->ms_zero && w->mz_zero,
                  "weight descriptor holds a null tensor pointer");
    *G = (int)g;
    *C = (int)(L / w->meta_group);
    return HQM_OK;
}

// HQM_FORCE_GENERIC=1 in the environment routes every linear through the shape-agnostic
// kernel (used by the tests to check the two paths against each other).
bool force_generic() {
    static const bool on = [] {
        const char* v = getenv("HQM_FORCE_GENERIC");
        return v && v[0] == '1';
    }();
    return on;
}

static std::atomic<int> g_overlap{-1};
bool overlap_enabled() {
    int v = g_overlap.load(std::memory_order_relaxed);
    if (v < 0) {
        const char* e = getenv("HQM_NO_OVERLAP");
        v = (e && e[0] == '1') ? 0 : 1;
        g_overlap.store(v, std::memory_order_relaxed);
    }
    return v != 0;
}
int set_overlap(int on) {
    const int prev = overlap_enabled() ? 1 : 0;
    g_overlap.store(on ? 1 : 0, std::memory_order_relaxed);
    return prev;
}

size_t linear_scratch_bytes(int64_t M, const hqm_weight* w) {
    int G, C;
    StreamPlan plan;
    if (M <= 0 || check_weight(w, &G, &C) != HQM_OK) return 0;
    if (force_generic()) return 0;
    if (M >= TC_MIN_ROWS && gemm_tc_supported(w, G, C, M)) return ((size_t)M * w->N * sizeof(float) + 255) / 256 * 256;
    if (gemm_tc3_supported(w, G, C, M)) return gemm_tc3_scratch_bytes(w, G, M);
    Stream3Plan plan3;
    if (gemv_stream3_plan(w, G, C, M, &plan3)) return gemv_stream3_scratch_bytes(plan3, M, w->N);
    const hqm_weight* one[1] = {w};
    if (!gemv_stream_plan(one, 1, M, &plan, /*chained=*/false)) return 0;
    return (gemv_stream_scratch_bytes(plan, M) + 255) / 256 * 256;
}

int launch_linear(uint16_t* y, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w,
                  const uint16_t* bias, uint32_t* counters, void* scratch, size_t scratch_bytes, cudaStream_t st) {
    int G, C;
    int rc = check_weight(w, &G, &C);
    if (rc != HQM_OK) return rc;
    if (M == 0) return HQM_OK;
    StreamPlan plan;
    const bool x_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    if (!x_ok || force_generic()) return launch_linear_generic(y, x, x_idx, M, w, G, C, bias, st);
    if (M >= TC_MIN_ROWS && gemm_tc_supported(w, G, C, M)) {
        const size_t need = (size_t)M * w->N * sizeof(float);
        if (scratch == nullptr || scratch_bytes < need) {
            set_error("linear: scratch of %zu bytes given, %zu needed", scratch_bytes, need);
            return HQM_ERR_SCRATCH;
        }
        HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 15u) == 0, "linear: scratch must be 16-byte aligned");
        rc = launch_gemm_tc((float*)scratch, x, x_idx, M, w, nullptr, G, C, st);
        if (rc != HQM_OK) return rc;
        return launch_rows_from_sums(y, (const float*)scratch, bias, M, w->N, st);
    }
    if (gemm_tc3_supported(w, G, C, M)) {
        const size_t need = gemm_tc3_scratch_bytes(w, G, M);
        if (scratch == nullptr || scratch_bytes < need) {
            set_error("linear: scratch of %zu bytes given, %zu needed", scratch_bytes, need);
            return HQM_ERR_SCRATCH;
        }
        HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 15u) == 0, "linear: scratch must be 16-byte aligned");
        return launch_gemm_tc3(y, scratch, x, x_idx, M, w, bias, G, C, st);
    }
    Stream3Plan plan3;
    if (gemv_stream3_plan(w, G, C, M, &plan3)) {
        const size_t need = gemv_stream3_scratch_bytes(plan3, M, w->N);
        if (scratch == nullptr || scratch_bytes < need) {
            set_error("linear: scratch of %zu bytes given, %zu needed", scratch_bytes, need);
            return HQM_ERR_SCRATCH;
        }
        HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 15u) == 0, "linear: scratch must be 16-byte aligned");
        return launch_gemv_stream3(y, (float*)scratch, x, x_idx, M, w, bias, G, C, plan3, st);
    }
    const hqm_weight* one[1] = {w};
    if (gemv_stream_plan(one, 1, M, &plan, /*chained=*/false)) {
        const size_t need = gemv_stream_scratch_bytes(plan, M);
        if (scratch == nullptr || scratch_bytes < need) {
            set_error("linear: scratch of %zu bytes given, %zu needed", scratch_bytes, need);
            return HQM_ERR_SCRATCH;
        }
        HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 15u) == 0, "linear: scratch must be 16-byte aligned");
        StreamJob job{};
        job.w[0] = w;
        job.counters = counters;
        if (plan.tma) {                      // the launch finishes the row itself: bf16, bias added
            job.y_out = y;
            job.bias = bias;
            return launch_gemv_stream((float*)scratch, x, x_idx, M, job, plan, st);
        }
        rc = launch_gemv_stream((float*)scratch, x, x_idx, M, job, plan, st);
        if (rc != HQM_OK) return rc;
        return launch_finalize_linear(y, (const float*)scratch, bias, M, plan, st);
    }
    return launch_linear_generic(y, x, x_idx, M, w, G, C, bias, st);
}

}  // namespace hqm

extern "C" {

const char* hqm_last_error(void) { return hqm::g_error; }
int hqm_version(void) { return 1; }
int64_t hqm_launch_count(void) { return (int64_t)hqm::launches(); }
int hqm_set_overlap(int on) { return hqm::set_overlap(on); }

size_t hqm_scratch_header_bytes(void) { return hqm::SCRATCH_HEADER; }

int hqm_scratch_init(void* scratch, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(scratch != nullptr, "scratch_init: null pointer");
    HQM_CUDA(cudaMemsetAsync(scratch, 0, SCRATCH_HEADER, (cudaStream_t)stream));
    return HQM_OK;
}

size_t hqm_linear_scratch_bytes(int64_t M, const hqm_weight* w) {
    const size_t inner = hqm::linear_scratch_bytes(M, w);
    return inner ? inner + hqm::SCRATCH_HEADER : 0;
}

int hqm_linear(uint16_t* y, const uint16_t* x, int64_t M, const hqm_weight* w, const uint16_t* bias, void* scratch,
               size_t scratch_bytes, void* stream) {
    using namespace hqm;
    HQM_CHECK_ARG(M >= 0 && M <= INT32_MAX, "linear: bad row count %lld", (long long)M);
    HQM_CHECK_ARG(M == 0 || (y && x), "linear: null activation pointer");
    if (scratch == nullptr || scratch_bytes <= SCRATCH_HEADER)
        return launch_linear(y, x, nullptr, M, w, bias, nullptr, nullptr, 0, (cudaStream_t)stream);
    HQM_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "linear: scratch must be 256-byte aligned");
    return launch_linear(y, x, nullptr, M, w, bias, (uint32_t*)scratch, (uint8_t*)scratch + SCRATCH_HEADER,
                         scratch_bytes - SCRATCH_HEADER, (cudaStream_t)stream);
}

}  // extern "C"
