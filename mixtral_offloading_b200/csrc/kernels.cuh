// Internal launchers shared between the translation units of the library.
#pragma once
#include "common.cuh"

namespace hqm {

// linear_generic.cu — any shape check_weight() accepts.
int launch_linear_generic(uint16_t* y, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w, int G,
                          int C, const uint16_t* bias, cudaStream_t st);

// gemv_stream.cu — the weight-streaming path for small row counts.
constexpr int STREAM_MAX_LAYERS = 4;
// What one launch multiplies: up to four layers of the same K, bit width and group size (N may differ).
// Layer l reads rows x_idx?[m] + xrow[l] of x.  With `table` set, layer l's descriptor is read on the
// device: table[3 * *sel[l] + which[l]] (3 entries per expert: w1, w2, w3), and w[l] only gives the shape.
// One entry of the device-side expert table (hqm_expert_table_build): the layer's descriptor and the three
// tensor maps (packed codes, scale bytes, zero bytes) the TMA-staged kernel copies its tiles with.
struct alignas(128) StreamEntry {
    hqm_weight w;
    unsigned char pad[128 - sizeof(hqm_weight)];
    unsigned char maps[3][128];
};
static_assert(sizeof(StreamEntry) == 512, "table entries are 512 bytes");

struct StreamJob {
    const hqm_weight* w[STREAM_MAX_LAYERS];
    int xrow[STREAM_MAX_LAYERS];
    const StreamEntry* table;
    const int32_t* sel[STREAM_MAX_LAYERS];
    int which[STREAM_MAX_LAYERS];
    // Set only when the kernel launched in front of this one lets its successor start after everything
    // before it has completed (launch_finalize_silu_mul(..., late_trigger = true)) and the indices behind
    // `sel` are older than that: the launch then reads them, and starts on the weights, without waiting.
    int sel_settled;
    // TMA-staged launches (plan.tma) only.  counters: the zeroed header of the caller's scratch buffer (arrival
    // counters of units split over several CTAs; left zero again).  y_out: when set, the launch writes the finished
    // row as bf16 (+ bias) there itself, and no finalize launch follows.
    uint32_t* counters;
    uint16_t* y_out;
    const uint16_t* bias;
};
// Every scratch buffer handed to the library starts with this many bytes of library state, zero when the buffer is
// first used (hqm_scratch_init) and zero again after every call.
constexpr size_t SCRATCH_HEADER = 64 * 1024;
struct StreamPlan {
    int count;                          // layers in the launch
    int nbits, nb;                      // bit width, group size / 16
    int G[STREAM_MAX_LAYERS], C[STREAM_MAX_LAYERS];
    int rho0[STREAM_MAX_LAYERS + 1];    // first storage-row residue of each layer; [count] = all of them
    int col0[STREAM_MAX_LAYERS + 1];    // first column of each layer in a partial row; [count] = row length
    int PT;      // passes per residue (K / pass width)
    int grid;    // CTAs of the single-wave persistent grid
    int warps;   // warps of that grid: the units the passes are split over
    int toks;    // rows of x decoded per launch
    int slots;   // upper bound on the warps contributing to one residue: fp32 partials [slots][M][row length]
    int tma;     // 1: the TMA-staged single-row kernel (gemv_tma.cu): units are (residue, block of 16 members),
                 // rho0 counts those units, and `warps` counts CTAs
};
// False when the layers / row count are outside what the streaming kernels cover.  `chained`: the launch is a
// link of the decode step's launch chain (its consumers read the sums); false for a linear that stands alone.
bool gemv_stream_plan(const hqm_weight* const* ws, int count, int64_t M, StreamPlan* plan, bool chained = true);
size_t gemv_stream_scratch_bytes(const StreamPlan& plan, int64_t M);
int launch_gemv_stream(float* partial, const uint16_t* x, const int32_t* x_idx, int64_t M, const StreamJob& job,
                       const StreamPlan& plan, cudaStream_t st);
// y (M, row length) = bf16(sums + bias)
int launch_finalize_linear(uint16_t* y, const float* partial, const uint16_t* bias, int64_t M, const StreamPlan& plan,
                           cudaStream_t st);
// h[p] (M, F) = silu(layer 2p) * layer 2p+1 for each pair of layers of the launch
int launch_finalize_silu_mul(uint16_t* h, const float* partial, int64_t M, const StreamPlan& plan, cudaStream_t st,
                             bool late_trigger = false);
// out[token_idx[m]] (+)= sum over the launch's layers l of route_w[l * M + m] * layer l
int launch_finalize_scatter(uint16_t* out, const float* partial, const int32_t* token_idx, const float* route_w,
                            int accumulate, int64_t M, const StreamPlan& plan, cudaStream_t st);
bool force_generic();
// gemv_tma.cu — the same for ONE row of x, tiles staged by TMA.
bool gemv_tma_plan(const hqm_weight* const* ws, int count, bool chained, StreamPlan* plan);
int launch_gemv_tma(float* partial, const uint16_t* x, const int32_t* x_idx, int64_t M, const StreamJob& job,
                    const StreamPlan& plan, cudaStream_t st);

// router.cu — logits, top-2 indices and weights of M tokens (no per-expert lists).
int launch_router_top2(uint16_t* router_logits, float* topk_w, int32_t* topk_idx, const uint16_t* x,
                       const uint16_t* gate_w, int64_t M, int64_t K, int32_t E, cudaStream_t st);

// gemv_stream3.cu — the weight-streaming path for 3-bit layers.
struct Stream3Plan {
    int P3;      // storage-row classes (rows R and R + P3 hold the same residues in the same slots)
    int PT;      // 64-column passes per class
    int rows;    // storage rows, ceil(N / 10)
    int grid, warps, slots;
};
bool gemv_stream3_plan(const hqm_weight* w, int G, int C, int64_t M, Stream3Plan* plan);
size_t gemv_stream3_scratch_bytes(const Stream3Plan& plan, int64_t M, int N);
int launch_gemv_stream3(uint16_t* y, float* partial, const uint16_t* x, const int32_t* x_idx, int64_t M,
                        const hqm_weight* w, const uint16_t* bias, int G, int C, const Stream3Plan& plan,
                        cudaStream_t st);

// gemm_tc.cu — tcgen05 / TMEM path for many rows of x.
bool gemm_tc_supported(const hqm_weight* w, int G, int C, int64_t M);
int launch_gemm_tc(float* sums, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w0,
                   const hqm_weight* w1, int G, int C, cudaStream_t st);
int launch_rows_from_sums(uint16_t* y, const float* sums, const uint16_t* bias, int64_t M, int N, cudaStream_t st);
int launch_silu_mul_from_sums(uint16_t* h, const float* sums, int64_t M, int F, cudaStream_t st);
int launch_scatter_from_sums(uint16_t* out, const float* sums, const int32_t* token_idx, const float* route_w,
                             int accumulate, int64_t M, int H, cudaStream_t st);
int* tc_error_ptr();                  // device flag the bounded waits set when they give up
// gemm_tma.cu — the same GEMM with every operand staged by TMA, persistent stream-K CTAs (contiguous rows of x).
void* tma_encode_entry();
bool gemm_tma_supported(const hqm_weight* w, int G, int C, int64_t M);
int launch_gemm_tma(float* sums, const uint16_t* x, int64_t M, const hqm_weight* w0, const hqm_weight* w1, int G, int C,
                    cudaStream_t st);
int launch_gather_rows(uint16_t* dst, const uint16_t* x, const int32_t* idx, int64_t M, int K, cudaStream_t st);
constexpr int64_t TC_MIN_ROWS = 17;   // fewer rows go to the streaming kernels

// gemm_tc3.cu — the same for 3-bit layers (row counts >= 5).
bool gemm_tc3_supported(const hqm_weight* w, int G, int C, int64_t M);
size_t gemm_tc3_scratch_bytes(const hqm_weight* w, int G, int64_t M);
int launch_gemm_tc3(uint16_t* y, void* scratch, const uint16_t* x, const int32_t* x_idx, int64_t M,
                    const hqm_weight* w, const uint16_t* bias, int G, int C, cudaStream_t st);

// ffn.cu — launches of the single-token MoE block: [w1; w3] of both chosen experts (4 layers), then both w2.
struct MoeDecodePlan {
    StreamPlan up, down;
    size_t router_bytes, up_bytes, h_bytes, down_bytes;
};
bool moe_decode_plan(int E, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3, MoeDecodePlan* mp);
// `slots` (1 or 2) experts per launch instead of the two routed ones (an expert-parallel rank's share).
bool moe_decode_plan_slots(int E, int slots, const hqm_weight* w1, const hqm_weight* w2, const hqm_weight* w3,
                           MoeDecodePlan* mp);

// Dispatcher used by hqm_linear and by the expert FFN: picks the streaming
// kernel when the layer's shape allows it, the generic one otherwise.
// (scratch excludes the header; counters points at it)
size_t linear_scratch_bytes(int64_t M, const hqm_weight* w);
int launch_linear(uint16_t* y, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w,
                  const uint16_t* bias, uint32_t* counters, void* scratch, size_t scratch_bytes, cudaStream_t st);

}  // namespace hqm
