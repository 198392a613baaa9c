// Split-KV FlashDecoding for one query token over the fp16 head-major KV cache
// [n_kv][max_seq][hd] (reference layout, include/model.cuh:25), all query heads
// of a KV head processed together so K and V are read once per group.
//
// Reference behaviour being replaced: src/kernels.cu:105-219 (stage 1, 64 fixed
// partitions, WMMA) and :222-288 (stage 2 combine).  This kernel keeps scores
// and the softmax in fp32 (the reference rounds scores to fp16), uses
// mma.sync.m16n8k16 with operands loaded straight from global memory in
// fragment order (no shared-memory staging of K or V), and folds the combine
// into the same launch: every CTA writes its partial (m, l, O) to scratch and
// the last CTA of a KV head to arrive merges them.
//
// Scratch: part_o  [n_kv][nsplit][8][hd] fp32, part_ml [n_kv][nsplit][8][2] fp32,
// counters [n_kv] u32 (must be zero before the first launch; the kernel leaves
// them zero).
#pragma once
#include "common.cuh"

namespace cq {

constexpr int kAttnWarps = 4;
constexpr int kMaxSplit = 128; // upper bound on nsplit (sizes a shared-memory table)
constexpr int kMaxGroup = 8;   // query heads per KV head that one MMA column block can hold

struct AttnArgs {
    const __half* q;        // [n_kv*grp][hd]
    const __half* kc;       // [n_kv][max_seq][hd]
    const __half* vc;
    __half* out;            // [n_kv*grp][hd]
    const int* d_pos;       // attends to keys [0, *d_pos]
    int n_kv, grp, max_seq, nsplit;
    float scale_log2;       // (1/sqrt(hd)) * log2(e)
    float* part_o;
    float* part_ml;
    unsigned* counters;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_decode_kernel(const AttnArgs a) {
    constexpr int NCH = HD / 32;   // 16-byte chunks of a K row per lane (4 lanes cover 64 B)
    constexpr int NC = HD / 64;    // 16-byte chunks of a V row per lane (8 lanes cover 128 B)
    constexpr int NMT = HD / 16;   // output m-tiles (16 d values each)
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    __shared__ float sm_o[kAttnWarps][kMaxGroup][HD];
    __shared__ float sm_m[kAttnWarps][kMaxGroup], sm_l[kAttnWarps][kMaxGroup];
    __shared__ float sm_w[kMaxGroup][kMaxSplit];
    __shared__ int sm_last;

    pdl_launch_dependents();
    pdl_wait();

    const int len = *a.d_pos + 1;
    int chunk = (len + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + 15) & ~15;
    const int t0 = split * chunk;
    const int t1 = min(t0 + chunk, len);
    const bool nonempty_cta = t0 < len;

    if (nonempty_cta) {
        // A operand of QK^T: q of head g (zero rows for g >= grp)
        uint32_t qa[NCH][4];
        {
            const __half* qrow = a.q + (size_t)(kvh * a.grp + g) * HD;
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (g < a.grp) v = *reinterpret_cast<const uint4*>(qrow + (i * 4 + t) * 8);
                qa[i][0] = v.x; qa[i][1] = v.y; qa[i][2] = v.z; qa[i][3] = v.w;
            }
        }
        const __half* kbase = a.kc + (size_t)kvh * a.max_seq * HD;
        const __half* vbase = a.vc + (size_t)kvh * a.max_seq * HD;

        float o[NMT][4];
#pragma unroll
        for (int m = 0; m < NMT; ++m) o[m][0] = o[m][1] = o[m][2] = o[m][3] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;

        const int ntile = (t1 - t0 + 15) >> 4;
        for (int tile = warp; tile < ntile; tile += kAttnWarps) {
            const int kb = t0 + tile * 16;
            // K: two 8-key column blocks; lane reads key kb+g and kb+8+g
            uint4 kA[NCH], kB[NCH];
            const bool vA = kb + g < t1, vB = kb + 8 + g < t1;
#pragma unroll
            for (int i = 0; i < NCH; ++i) { kA[i] = make_uint4(0, 0, 0, 0); kB[i] = make_uint4(0, 0, 0, 0); }
            if (vA) {
#pragma unroll
                for (int i = 0; i < NCH; ++i) kA[i] = ldg_stream(kbase + (size_t)(kb + g) * HD + (i * 4 + t) * 8);
            }
            if (vB) {
#pragma unroll
                for (int i = 0; i < NCH; ++i) kB[i] = ldg_stream(kbase + (size_t)(kb + 8 + g) * HD + (i * 4 + t) * 8);
            }
            // V: lane reads keys kb+2t, +2t+1, +2t+8, +2t+9, d chunk (c*8+g)
            uint4 vv[4][NC];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int key = kb + 2 * t + (r & 1) + (r >> 1) * 8;
#pragma unroll
                for (int c = 0; c < NC; ++c) vv[r][c] = make_uint4(0, 0, 0, 0);
                if (key < t1) {
#pragma unroll
                    for (int c = 0; c < NC; ++c) vv[r][c] = ldg_stream(vbase + (size_t)key * HD + (c * 8 + g) * 8);
                }
            }

            float sA[4] = {0.f, 0.f, 0.f, 0.f}, sB[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                mma16816(sA, qa[i][0], 0u, qa[i][1], 0u, kA[i].x, kA[i].y);
                mma16816(sA, qa[i][2], 0u, qa[i][3], 0u, kA[i].z, kA[i].w);
                mma16816(sB, qa[i][0], 0u, qa[i][1], 0u, kB[i].x, kB[i].y);
                mma16816(sB, qa[i][2], 0u, qa[i][3], 0u, kB[i].z, kB[i].w);
            }
            // lane holds head g, keys kb+2t, kb+2t+1 (sA) and kb+8+2t, kb+9+2t (sB)
            float s0 = kb + 2 * t < t1 ? sA[0] * a.scale_log2 : -INFINITY;
            float s1 = kb + 2 * t + 1 < t1 ? sA[1] * a.scale_log2 : -INFINITY;
            float s2 = kb + 8 + 2 * t < t1 ? sB[0] * a.scale_log2 : -INFINITY;
            float s3 = kb + 9 + 2 * t < t1 ? sB[1] * a.scale_log2 : -INFINITY;
            float mx = fmaxf(fmaxf(s0, s1), fmaxf(s2, s3));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);       // finite: key kb is always valid
            const float alpha = ex2(m_run - m_new);
            const float p0 = ex2(s0 - m_new), p1 = ex2(s1 - m_new), p2 = ex2(s2 - m_new), p3 = ex2(s3 - m_new);
            l_run = l_run * alpha + ((p0 + p1) + (p2 + p3));
            m_run = m_new;
            const uint32_t pb0 = pack_h2(p0, p1), pb1 = pack_h2(p2, p3);
            // O columns of this lane are heads 2t and 2t+1
            const float al = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4), ah = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
            if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
                for (int m = 0; m < NMT; ++m) { o[m][0] *= al; o[m][1] *= ah; o[m][2] *= al; o[m][3] *= ah; }
            }
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int ep = 0; ep < 4; ++ep) {
                    uint32_t wA = u4c(vv[0][c], ep), wB = u4c(vv[1][c], ep), wC = u4c(vv[2][c], ep), wD = u4c(vv[3][c], ep);
                    mma16816(o[c * 4 + ep], prmt(wA, wB, 0x5410), prmt(wA, wB, 0x7632), prmt(wC, wD, 0x5410), prmt(wC, wD, 0x7632), pb0, pb1);
                }
        }
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        if (t == 0) { sm_m[warp][g] = m_run; sm_l[warp][g] = l_run; }
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int ep = 0; ep < 4; ++ep) {
                const int d = (c * 8 + g) * 8 + 2 * ep, m = c * 4 + ep;
                sm_o[warp][2 * t][d] = o[m][0]; sm_o[warp][2 * t + 1][d] = o[m][1];
                sm_o[warp][2 * t][d + 1] = o[m][2]; sm_o[warp][2 * t + 1][d + 1] = o[m][3];
            }
        __syncthreads();
        // merge the warps of this CTA and publish the partial
        float* po = a.part_o + ((size_t)(kvh * a.nsplit + split) * kMaxGroup) * HD;
        float* pml = a.part_ml + ((size_t)(kvh * a.nsplit + split) * kMaxGroup) * 2;
        for (int idx = threadIdx.x; idx < a.grp * HD; idx += blockDim.x) {
            const int h = idx / HD, d = idx % HD;
            float M = sm_m[0][h];
#pragma unroll
            for (int w = 1; w < kAttnWarps; ++w) M = fmaxf(M, sm_m[w][h]);
            float acc = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) {
                const float f = ex2(sm_m[w][h] - M);
                acc += sm_o[w][h][d] * f;
                L += sm_l[w][h] * f;
            }
            po[h * HD + d] = acc;
            if (d == 0) { pml[h * 2] = M; pml[h * 2 + 1] = L; }
        }
    }
    // ticket: the last CTA of this KV head merges all partials
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned old = atomicAdd(a.counters + kvh, 1u);
        sm_last = old == (unsigned)(a.nsplit - 1);
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    const int nne = (len + chunk - 1) / chunk;     // non-empty splits: 0..nne-1
    const float* pml0 = a.part_ml + (size_t)kvh * a.nsplit * kMaxGroup * 2;
    const float* po0 = a.part_o + (size_t)kvh * a.nsplit * kMaxGroup * HD;
    for (int h = warp; h < a.grp; h += kAttnWarps) {
        float M = -INFINITY;
        for (int s = lane; s < nne; s += 32) M = fmaxf(M, __ldcg(pml0 + (size_t)(s * kMaxGroup + h) * 2));
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
        float L = 0.f;
        for (int s = lane; s < nne; s += 32) {
            const float f = ex2(__ldcg(pml0 + (size_t)(s * kMaxGroup + h) * 2) - M);
            sm_w[h][s] = f;
            L += f * __ldcg(pml0 + (size_t)(s * kMaxGroup + h) * 2 + 1);
        }
        L = warp_sum(L);
        const float inv = 1.0f / L;
        for (int s = lane; s < nne; s += 32) sm_w[h][s] *= inv;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < a.grp * (HD / 4); idx += blockDim.x) {
        const int h = idx / (HD / 4), d4 = idx % (HD / 4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4* src = reinterpret_cast<const float4*>(po0 + (size_t)h * HD) + d4;
#pragma unroll 8
        for (int s = 0; s < nne; ++s) {
            const float4 v = __ldcg(src + (size_t)s * kMaxGroup * (HD / 4));
            const float w = sm_w[h][s];
            acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
        }
        __half2* dst = reinterpret_cast<__half2*>(a.out + (size_t)(kvh * a.grp + h) * HD + d4 * 4);
        dst[0] = __floats2half2_rn(acc.x, acc.y);
        dst[1] = __floats2half2_rn(acc.z, acc.w);
    }
    if (threadIdx.x == 0) a.counters[kvh] = 0u;
}

}  // namespace cq
