// How a streaming launch splits its passes over warps, and how the fp32 partial row-sets it leaves
// behind are summed: shared by the streaming kernel and every kernel that consumes its partials.
#pragma once
#include "common.cuh"
#include "kernels.cuh"

namespace hqm {

// Work split shared by the kernel and the finalize step: passes are numbered
// L = rho * PT + p (PT passes per residue); warp c of the grid owns [c*Ltot/grid, (c+1)*Ltot/grid).
// (32-bit arithmetic throughout: the planner rejects layers with total() * grid >= 2^31.)
struct Split {
    int P, PT, grid;
    __host__ __device__ uint32_t total() const { return (uint32_t)P * (uint32_t)PT; }
    __host__ __device__ uint32_t begin(int c) const { return (uint32_t)c * total() / (uint32_t)grid; }
    // warp whose range contains pass L
    __host__ __device__ int owner(uint32_t L) const {
        int c = (int)(L * (uint32_t)grid / total());
        while (c + 1 < grid && begin(c + 1) <= L) ++c;
        while (c > 0 && begin(c) > L) --c;
        return c;
    }
};

// Where the columns of a partial row come from: the layers of the launch side by side.
struct ColMap {
    int count, per;
    int col0[STREAM_MAX_LAYERS + 1];
    int rho0[STREAM_MAX_LAYERS];
    int G[STREAM_MAX_LAYERS];
};

// Number of partial row-sets that hold a piece of column `col` of a partial row.
__device__ __forceinline__ int partial_count(const Split& sp, const ColMap& cm, int col) {
    int layer = 0;
#pragma unroll
    for (int l = 1; l < STREAM_MAX_LAYERS; ++l) layer += (l < cm.count && col >= cm.col0[l]) ? 1 : 0;
    const int nn = col - cm.col0[layer];
    const uint32_t rho_g = (uint32_t)(cm.rho0[layer] + (nn % cm.G[layer]) / cm.per);
    return sp.owner(rho_g * sp.PT + sp.PT - 1) - sp.owner(rho_g * sp.PT) + 1;
}

// Sum of the partial row-sets of element (m, col); `row` is the row length, MR = rows * row.  The row-sets
// are read eight at a time (independent loads in flight together) and added in a fixed order.
__device__ __forceinline__ float partial_sum(const float* __restrict__ partial, const Split& sp, const ColMap& cm,
                                             int64_t m, int col, int row, int64_t MR) {
    const int cnt = partial_count(sp, cm, col);
    const float* p = partial + m * row + col;
    float v = 0.f;
    for (int s = 0; s < cnt; s += 8) {
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = (s + j < cnt) ? p[(int64_t)(s + j) * MR] : 0.f;
        v += ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
    }
    return v;
}

inline Split split_of(const StreamPlan& plan) { return Split{plan.rho0[plan.count], plan.PT, plan.warps}; }
inline ColMap colmap_of(const StreamPlan& plan) {
    ColMap cm{};
    cm.count = plan.count;
    cm.per = codes_per_word(plan.nbits);
    for (int l = 0; l < plan.count; ++l) {
        cm.col0[l] = plan.col0[l];
        cm.rho0[l] = plan.rho0[l];
        cm.G[l] = plan.G[l];
    }
    cm.col0[plan.count] = plan.col0[plan.count];
    return cm;
}

}  // namespace hqm
