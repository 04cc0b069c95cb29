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
    int nb;          // blocks of 16 group members that are separate units of the split (1: a unit is a whole residue)
    int col0[STREAM_MAX_LAYERS + 1];
    int rho0[STREAM_MAX_LAYERS];
    int G[STREAM_MAX_LAYERS];
};

// First column of layer l (l may be a run-time value: the selects keep the arrays in the parameter bank).
__device__ __forceinline__ int layer_col0(const ColMap& cm, int l) {
    int c = cm.col0[0];
#pragma unroll
    for (int i = 1; i <= STREAM_MAX_LAYERS; ++i) c = (l == i) ? cm.col0[i] : c;
    return c;
}

// Number of partial row-sets that hold a piece of column `col` of a partial row.
__device__ __forceinline__ int partial_count(const Split& sp, const ColMap& cm, int col) {
    int c0 = cm.col0[0], r0 = cm.rho0[0], G = cm.G[0];
#pragma unroll
    for (int l = 1; l < STREAM_MAX_LAYERS; ++l) {
        const bool in = l < cm.count && col >= cm.col0[l];
        c0 = in ? cm.col0[l] : c0;
        r0 = in ? cm.rho0[l] : r0;
        G = in ? cm.G[l] : G;
    }
    const int rel = col - c0;
    const uint32_t rho_g = (uint32_t)(r0 + ((rel % G) / cm.per) * cm.nb + ((rel / G) >> 4) % cm.nb);
    return sp.owner(rho_g * sp.PT + sp.PT - 1) - sp.owner(rho_g * sp.PT) + 1;
}

// Sum of the partial row-sets of element (m, col), added in a fixed order; `row` is the row length,
// MR = rows * row.  BATCHED = false is a plain loop (the compiler groups its loads): best when a residue has
// few row-sets (the kernels behind hqm_linear / hqm_expert_ffn).  BATCHED = true keeps eight loads in flight at
// a time: best for the decode step's small layers, whose K dimension is cut into about twenty pieces.  (Each
// measured a few percent slower in the other's place.)
template <bool BATCHED>
__device__ __forceinline__ float partial_sum(const float* __restrict__ partial, const Split& sp, const ColMap& cm,
                                             int64_t m, int col, int row, int64_t MR) {
    const int cnt = partial_count(sp, cm, col);
    const float* p = partial + m * row + col;
    float v = 0.f;
    if constexpr (!BATCHED) {
        for (int s = 0; s < cnt; ++s) v += p[(int64_t)s * MR];
    } else {
        for (int s = 0; s < cnt; s += 8) {
            float a[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = (s + j < cnt) ? p[(int64_t)(s + j) * MR] : 0.f;
            v += ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
        }
    }
    return v;
}

// Two elements of the same row at once (a rotation pair, the gate and up halves of an FFN, the two experts of a
// token): the row-sets of both are requested together, so the pair costs the round trips of one.
template <bool BATCHED>
__device__ __forceinline__ void partial_sum_pair(const float* __restrict__ partial, const Split& sp, const ColMap& cm,
                                                 int64_t m, int col_a, int col_b, int row, int64_t MR, float& out_a,
                                                 float& out_b) {
    const int cnt_a = partial_count(sp, cm, col_a), cnt_b = partial_count(sp, cm, col_b);
    const float* pa = partial + m * row + col_a;
    const float* pb = partial + m * row + col_b;
    float va = 0.f, vb = 0.f;
    if constexpr (!BATCHED) {
        const int both = cnt_a < cnt_b ? cnt_a : cnt_b;
        for (int s = 0; s < both; ++s) {
            va += pa[(int64_t)s * MR];
            vb += pb[(int64_t)s * MR];
        }
        for (int s = both; s < cnt_a; ++s) va += pa[(int64_t)s * MR];
        for (int s = both; s < cnt_b; ++s) vb += pb[(int64_t)s * MR];
    } else {
        const int cnt = cnt_a > cnt_b ? cnt_a : cnt_b;
        for (int s = 0; s < cnt; s += 8) {
            float a[8], b[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                a[j] = (s + j < cnt_a) ? pa[(int64_t)(s + j) * MR] : 0.f;
                b[j] = (s + j < cnt_b) ? pb[(int64_t)(s + j) * MR] : 0.f;
            }
            va += ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
            vb += ((b[0] + b[1]) + (b[2] + b[3])) + ((b[4] + b[5]) + (b[6] + b[7]));
        }
    }
    out_a = va;
    out_b = vb;
}

// The split the CONSUMERS of a launch's sums see.  A TMA-staged launch finishes its sums itself (one fp32 row-set,
// `grid` = 1: every element has exactly one part); the other kernel leaves one row-set per warp that touched a residue.
inline Split split_of(const StreamPlan& plan) {
    return Split{plan.rho0[plan.count], plan.PT, plan.tma ? 1 : plan.warps};
}
// The split of the passes over the launch's CTAs / warps.
inline Split work_split_of(const StreamPlan& plan) { return Split{plan.rho0[plan.count], plan.PT, plan.warps}; }
inline ColMap colmap_of(const StreamPlan& plan) {
    ColMap cm{};
    cm.count = plan.count;
    cm.per = codes_per_word(plan.nbits);
    cm.nb = plan.tma ? plan.nb : 1;
    for (int l = 0; l < plan.count; ++l) {
        cm.col0[l] = plan.col0[l];
        cm.rho0[l] = plan.rho0[l];
        cm.G[l] = plan.G[l];
    }
    cm.col0[plan.count] = plan.col0[plan.count];
    return cm;
}

}  // namespace hqm
