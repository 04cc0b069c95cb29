// Internal launchers shared between the translation units of the library.
#pragma once
#include "common.cuh"

namespace hqm {

// linear_generic.cu — any shape check_weight() accepts.
int launch_linear_generic(uint16_t* y, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w, int G,
                          int C, const uint16_t* bias, cudaStream_t st);

// Dispatcher used by hqm_linear and by the expert FFN: picks the streaming
// kernel when the layer's shape allows it, the generic one otherwise.
int launch_linear(uint16_t* y, const uint16_t* x, const int32_t* x_idx, int64_t M, const hqm_weight* w,
                  const uint16_t* bias, cudaStream_t st);

}  // namespace hqm
