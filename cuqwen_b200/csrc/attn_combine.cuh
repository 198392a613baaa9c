// Constants and scratch geometry of the split-KV attention: a partial is, per query head, an un-normalised output
// O[HD] (fp32), the running maximum m (log2 units) and the sum l.  Slots: O [8][HD] floats, (m, l) [8][2] floats.
// The merge of the partials (the reference's stage 2, src/kernels.cu:222-288) is attn_fold_kernel in attn_split.cuh.
#pragma once
#include "common.cuh"

namespace cq {

constexpr int kMaxSplit = 128;  // upper bound on nsplit
constexpr int kMaxGroup = 8;    // query heads per KV head that one MMA column block can hold
constexpr int kAttnFanIn = 8;   // sizing unit of the scratch (an earlier tree merge folded this many partials per node)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Scratch geometry for (n_kv, nsplit): slots [n_kv][nsplit] for the partials, plus head-room that callers of the C ABI
// were told to allocate (one extra slot per group of kAttnFanIn splits, one counter per group and per KV head).
__host__ __device__ inline int attn_groups(int nsplit) { return (nsplit + kAttnFanIn - 1) / kAttnFanIn; }
__host__ __device__ inline size_t attn_slots(int n_kv, int nsplit) { return (size_t)n_kv * (nsplit + attn_groups(nsplit)); }
__host__ __device__ inline size_t attn_counters(int n_kv, int nsplit) { return (size_t)n_kv * (attn_groups(nsplit) + 1); }

}  // namespace cq
