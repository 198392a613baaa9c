// Split-KV FlashDecoding for one query token over the fp16 head-major KV cache [n_kv][max_seq][hd] (reference
// layout, include/model.cuh:25), all query heads of a KV head processed together so K and V are read once per group.
//
// Reference behaviour being replaced: src/kernels.cu:105-219 (stage 1, 64 fixed partitions, WMMA) and :222-288
// (stage 2 combine).  Here scores and the softmax stay in fp32 (the reference rounds scores to fp16), and the combine
// is folded into the same launch: every CTA writes its partial (m, l, O) to scratch and the last CTA of a KV head to
// arrive merges them.
//
// Data path: grid (n_kv, nsplit); a CTA owns a contiguous key range.  Keys of one KV head are contiguous in memory,
// so a producer warp streams them with plain bulk copies (cp.async.bulk, 64 keys of K and of V per stage) into a ring
// of shared-memory stages guarded by mbarriers; four consumer warps take one 16-key tile each, form Q.K^T and P.V with
// mma.sync.m16n8k16 (query heads on the M side of Q.K^T and on the N side of P.V, so the C fragment of the first is
// the B fragment of the second) and keep an online softmax per head.  Exactly the bytes of keys [0, pos] are copied:
// rows past the context are never read.  All mbarrier waits are bounded; on expiry *err is set.
//
// Scratch (sizes from attn_slots / attn_counters): part_o [slots][8][hd] fp32, part_ml [slots][8][2] fp32, counters
// u32 (zero before the first launch; the kernel leaves them zero).
#pragma once
#include "attn_combine.cuh"
#include "tma.cuh"

namespace cq {

constexpr int kAttnWarps = 4;          // consumer warps
constexpr int kAttnThreads = (kAttnWarps + 1) * 32;
constexpr int kAttnStageKeys = 16 * kAttnWarps;
constexpr int kAttnStages = 3;

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
    unsigned* err;          // receives a non-zero code when a bounded wait expires (may be null)
};

inline size_t attn_smem_bytes(int hd) { return (size_t)kAttnStages * 2 * kAttnStageKeys * hd * 2 + 128; }

template <int HD>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnArgs a) {
    constexpr int NCH = HD / 32;   // 16-byte chunks of a K row per lane (4 lanes cover 64 B)
    constexpr int NC = HD / 64;    // 16-byte chunks of a V row per lane (8 lanes cover 128 B)
    constexpr int NMT = HD / 16;   // output m-tiles (16 d values each)
    constexpr int ROWB = HD * 2;   // bytes of one key row
    constexpr int HALF = kAttnStageKeys * ROWB;   // bytes of the K (or V) half of a stage
    constexpr int NCT = kAttnWarps * 32;
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ float sm_o[kAttnWarps][kMaxGroup][HD];
    __shared__ float sm_m[kAttnWarps][kMaxGroup], sm_l[kAttnWarps][kMaxGroup];
    __shared__ __align__(8) unsigned long long sm_bar[2 * kAttnStages];
    __shared__ int sm_last;

    pdl_launch_dependents();
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t stage0 = smem_u32(dyn), bar_full = smem_u32(sm_bar), bar_empty = bar_full + kAttnStages * 8;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kAttnStages; ++s) { mbar_init(bar_full + s * 8, 1); mbar_init(bar_empty + s * 8, kAttnWarps); }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();                 // K/V row `pos` and q come from the previous kernel

    const int len = *a.d_pos + 1;
    int chunk = (len + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + 15) & ~15;
    const int t0 = split * chunk;
    const int t1 = min(t0 + chunk, len);
    const int nstage = t0 < len ? (t1 - t0 + kAttnStageKeys - 1) / kAttnStageKeys : 0;

    if (warp == kAttnWarps) {
        // producer: K and V of one KV head are contiguous [key][hd], so a stage is two plain bulk copies
        if (lane == 0) {
            const unsigned char* kb = reinterpret_cast<const unsigned char*>(a.kc) + ((size_t)kvh * a.max_seq + t0) * ROWB;
            const unsigned char* vb = reinterpret_cast<const unsigned char*>(a.vc) + ((size_t)kvh * a.max_seq + t0) * ROWB;
            bool failed = false;
            for (int st = 0; st < nstage; ++st) {
                const int s = st % kAttnStages;
                if (!failed && !mbar_wait(bar_empty + s * 8, ((st / kAttnStages) & 1) ^ 1)) { failed = true; if (a.err) atomicExch(a.err, 5u); }
                const int n = min(kAttnStageKeys, t1 - t0 - st * kAttnStageKeys);
                const uint32_t bytes = (uint32_t)n * ROWB;
                mbar_expect_tx(bar_full + s * 8, 2 * bytes);
                bulk_g2s(stage0 + s * 2 * HALF, kb + (size_t)st * HALF, bytes, bar_full + s * 8);
                bulk_g2s(stage0 + s * 2 * HALF + HALF, vb + (size_t)st * HALF, bytes, bar_full + s * 8);
            }
        }
        return;
    }
    // ---------------------------------------------- consumers --------------------------------------------------------
    auto csync = [] { asm volatile("bar.sync 1, %0;" ::"r"(NCT) : "memory"); };
    if (nstage > 0) {
        // A operand of Q.K^T: q of head g (zero rows for g >= grp)
        uint32_t qa[NCH][4];
        {
            const __half* qrow = a.q + (size_t)(kvh * a.grp + g) * HD;
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (g < a.grp) v = __ldcg(reinterpret_cast<const uint4*>(qrow + (i * 4 + t) * 8));
                qa[i][0] = v.x; qa[i][1] = v.y; qa[i][2] = v.z; qa[i][3] = v.w;
            }
        }
        float o[NMT][4];
#pragma unroll
        for (int m = 0; m < NMT; ++m) o[m][0] = o[m][1] = o[m][2] = o[m][3] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        bool failed = false;
        for (int st = 0; st < nstage; ++st) {
            const int s = st % kAttnStages;
            if (!failed && !mbar_wait(bar_full + s * 8, (st / kAttnStages) & 1)) { failed = true; if (a.err) atomicExch(a.err, 6u); }
            const int kb = t0 + st * kAttnStageKeys + 16 * warp;       // first key of this warp's tile
            if (kb < t1) {
                const unsigned char* sK = dyn + s * 2 * HALF + 16 * warp * ROWB;
                const unsigned char* sV = sK + HALF;
                uint4 kA[NCH], kB[NCH], vv[4][NC];
                const bool vA = kb + g < t1, vB = kb + 8 + g < t1;
#pragma unroll
                for (int i = 0; i < NCH; ++i) {
                    kA[i] = vA ? *reinterpret_cast<const uint4*>(sK + g * ROWB + (i * 4 + t) * 16) : make_uint4(0, 0, 0, 0);
                    kB[i] = vB ? *reinterpret_cast<const uint4*>(sK + (g + 8) * ROWB + (i * 4 + t) * 16) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int kr = 2 * t + (r & 1) + (r >> 1) * 8;
#pragma unroll
                    for (int c = 0; c < NC; ++c)
                        vv[r][c] = kb + kr < t1 ? *reinterpret_cast<const uint4*>(sV + kr * ROWB + (c * 8 + g) * 16) : make_uint4(0, 0, 0, 0);
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
                const float s0 = kb + 2 * t < t1 ? sA[0] * a.scale_log2 : -INFINITY;
                const float s1 = kb + 2 * t + 1 < t1 ? sA[1] * a.scale_log2 : -INFINITY;
                const float s2 = kb + 8 + 2 * t < t1 ? sB[0] * a.scale_log2 : -INFINITY;
                const float s3 = kb + 9 + 2 * t < t1 ? sB[1] * a.scale_log2 : -INFINITY;
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
                        const uint32_t wA = u4c(vv[0][c], ep), wB = u4c(vv[1][c], ep), wC = u4c(vv[2][c], ep), wD = u4c(vv[3][c], ep);
                        mma16816(o[c * 4 + ep], prmt(wA, wB, 0x5410), prmt(wA, wB, 0x7632), prmt(wC, wD, 0x5410), prmt(wC, wD, 0x7632), pb0, pb1);
                    }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + s * 8);
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
        csync();
        // merge the warps of this CTA and publish the partial
        float* po = a.part_o + ((size_t)(kvh * a.nsplit + split) * kMaxGroup) * HD;
        float* pml = a.part_ml + ((size_t)(kvh * a.nsplit + split) * kMaxGroup) * 2;
        for (int idx = threadIdx.x; idx < a.grp * HD; idx += NCT) {
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
    // two-level ticket tree (attn_combine.cuh): nobody waits, the last arrival of each node does that node's fold
    const int G = attn_groups(a.nsplit), gidx = split / kAttnFanIn;
    const int gfirst = gidx * kAttnFanIn, gsize = min(kAttnFanIn, a.nsplit - gfirst);
    const int nne = (len + chunk - 1) / chunk;                       // non-empty splits: 0 .. nne-1
    float* l1_o = a.part_o + (size_t)(kvh * a.nsplit + gfirst) * kMaxGroup * HD;
    float* l1_ml = a.part_ml + (size_t)(kvh * a.nsplit + gfirst) * kMaxGroup * 2;
    float* l2_o = a.part_o + ((size_t)a.n_kv * a.nsplit + (size_t)kvh * G) * kMaxGroup * HD;
    float* l2_ml = a.part_ml + ((size_t)a.n_kv * a.nsplit + (size_t)kvh * G) * kMaxGroup * 2;
    __half* out_kv = a.out + (size_t)kvh * a.grp * HD;
    __threadfence();
    csync();
    if (threadIdx.x == 0) sm_last = atomicAdd(a.counters + kvh * G + gidx, 1u) == (unsigned)(gsize - 1);
    csync();
    if (!sm_last) return;
    __threadfence();
    const int cnt1 = max(0, min(gsize, nne - gfirst));
    if (G == 1) {
        attn_fold<HD, true>(l1_o, l1_ml, cnt1, a.grp, warp, kAttnWarps, lane, out_kv, nullptr, nullptr);
        if (threadIdx.x == 0) a.counters[kvh * G + gidx] = 0u;
        return;
    }
    attn_fold<HD, false>(l1_o, l1_ml, cnt1, a.grp, warp, kAttnWarps, lane, nullptr, l2_o + (size_t)gidx * kMaxGroup * HD, l2_ml + (size_t)gidx * kMaxGroup * 2);
    if (threadIdx.x == 0) a.counters[kvh * G + gidx] = 0u;
    __threadfence();
    csync();
    if (threadIdx.x == 0) sm_last = atomicAdd(a.counters + a.n_kv * G + kvh, 1u) == (unsigned)(G - 1);
    csync();
    if (!sm_last) return;
    __threadfence();
    attn_fold<HD, true>(l2_o, l2_ml, G, a.grp, warp, kAttnWarps, lane, out_kv, nullptr, nullptr);
    if (threadIdx.x == 0) a.counters[a.n_kv * G + kvh] = 0u;
}

}  // namespace cq
