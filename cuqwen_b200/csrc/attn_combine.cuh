// Merge of split-KV partial results (the reference's stage 2, src/kernels.cu:222-288) as a two-level tree driven by
// tickets, so that no CTA ever waits for another: the last CTA of a group of kAttnFanIn splits folds that group's
// partials into one level-2 partial, and the last group of a KV head to do so folds the level-2 partials into the
// fp16 output.  A partial is, per query head, an un-normalised output O[HD] (fp32), the running maximum m (log2
// units) and the sum l.  Slots: O [8][HD] floats, (m, l) [8][2] floats.
#pragma once
#include "common.cuh"

namespace cq {

constexpr int kMaxSplit = 128;  // upper bound on nsplit
constexpr int kMaxGroup = 8;    // query heads per KV head that one MMA column block can hold
constexpr int kAttnFanIn = 8;   // partials folded per tree node

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Fold `count` consecutive slots starting at (po, pml).  Run by whole warps (warp index `warp` of `nwarps`); warp w
// takes heads w, w+nwarps, ...; lane = 4-float column of the head (HD/4 <= 32 columns).  FINAL: write fp16 out_h[head*HD..]
// normalised by l; otherwise write one slot (out_o, out_ml).
template <int HD, bool FINAL>
__device__ __forceinline__ void attn_fold(const float* po, const float* pml, int count, int grp, int warp, int nwarps, int lane,
                                          __half* out_h, float* out_o, float* out_ml) {
    constexpr int NCOL = HD / 4;
    for (int h = warp; h < grp; h += nwarps) {
        float M = -INFINITY;
        for (int s = lane; s < count; s += 32) M = fmaxf(M, __ldcg(pml + (size_t)(s * kMaxGroup + h) * 2));
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
        for (int s0 = 0; s0 < count; s0 += kAttnFanIn) {
            const int n = min(kAttnFanIn, count - s0);
            // this batch's weights: lane s holds w_s and l_s
            float w = 0.f, l = 0.f;
            if (lane < n) {
                const float m = __ldcg(pml + (size_t)((s0 + lane) * kMaxGroup + h) * 2);
                l = __ldcg(pml + (size_t)((s0 + lane) * kMaxGroup + h) * 2 + 1);
                w = (m == -INFINITY) ? 0.f : ex2(m - M);
            }
            float4 v[kAttnFanIn];
#pragma unroll
            for (int s = 0; s < kAttnFanIn; ++s)
                v[s] = (s < n && lane < NCOL) ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)((s0 + s) * kMaxGroup + h) * HD) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            L += warp_sum(w * l);
#pragma unroll
            for (int s = 0; s < kAttnFanIn; ++s) {
                const float ws = __shfl_sync(0xffffffffu, w, s);
                acc.x += v[s].x * ws; acc.y += v[s].y * ws; acc.z += v[s].z * ws; acc.w += v[s].w * ws;
            }
        }
        if (FINAL) {
            if (lane < NCOL) {
                const float inv = 1.0f / L;
                __half2* dst = reinterpret_cast<__half2*>(out_h + (size_t)h * HD + lane * 4);
                dst[0] = __floats2half2_rn(acc.x * inv, acc.y * inv);
                dst[1] = __floats2half2_rn(acc.z * inv, acc.w * inv);
            }
        } else {
            if (lane < NCOL) reinterpret_cast<float4*>(out_o + (size_t)h * HD)[lane] = acc;
            if (lane == 0) { out_ml[h * 2] = M; out_ml[h * 2 + 1] = L; }
        }
    }
}

// Scratch geometry for (n_kv, nsplit): level-1 slots [n_kv][nsplit], level-2 slots [n_kv][ngroups]; counters: level-1
// tickets [n_kv][ngroups] then level-2 tickets [n_kv].
__host__ __device__ inline int attn_groups(int nsplit) { return (nsplit + kAttnFanIn - 1) / kAttnFanIn; }
__host__ __device__ inline size_t attn_slots(int n_kv, int nsplit) { return (size_t)n_kv * (nsplit + attn_groups(nsplit)); }
__host__ __device__ inline size_t attn_counters(int n_kv, int nsplit) { return (size_t)n_kv * (attn_groups(nsplit) + 1); }

}  // namespace cq
