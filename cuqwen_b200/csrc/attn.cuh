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
#include "attn_tile.cuh"
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
    int stages;             // two-launch variant: ring depth (0 = its default)
};

inline size_t attn_smem_bytes(int hd) { return (size_t)kAttnStages * 2 * kAttnStageKeys * hd * 2 + 128; }

template <int HD>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnArgs a) {
    constexpr int NCH = HD / 32;   // 16-byte chunks of a K row per lane (4 lanes cover 64 B)
    constexpr int ROWB = HD * 2;   // bytes of one key row
    constexpr int HALF = kAttnStageKeys * ROWB;   // bytes of the K (or V) half of a stage
    constexpr int NCT = kAttnWarps * 32;
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ float sm_o[kAttnWarps][kMaxGroup][HD];
    __shared__ float sm_ml[kAttnWarps][kMaxGroup][2];
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
        uint32_t qa[NCH][4];
        attn_load_q<HD>(qa, a.q + (size_t)kvh * a.grp * HD, a.grp, g, t);
        AttnState<HD> st;
        st.reset();
        bool failed = false;
        for (int sn = 0; sn < nstage; ++sn) {
            const int s = sn % kAttnStages;
            if (!failed && !mbar_wait(bar_full + s * 8, (sn / kAttnStages) & 1)) { failed = true; if (a.err) atomicExch(a.err, 6u); }
            const int kb = t0 + sn * kAttnStageKeys + 16 * warp;       // first key of this warp's tile
            if (kb < t1) {
                const unsigned char* sK = dyn + s * 2 * HALF + 16 * warp * ROWB;
                attn_tile<HD, false>(st, qa, sK, sK + HALF, t1 - kb, a.scale_log2, g, t);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + s * 8);
        }
        attn_state_to_smem<HD>(st, &sm_o[warp][0][0], &sm_ml[warp][0][0], g, t);
        csync();
        // merge the warps of this CTA and publish the partial
        float* po = a.part_o + ((size_t)(kvh * a.nsplit + split) * kMaxGroup) * HD;
        float* pml = a.part_ml + ((size_t)(kvh * a.nsplit + split) * kMaxGroup) * 2;
        attn_merge_warps<HD>(&sm_o[0][0][0], &sm_ml[0][0][0], kAttnWarps, a.grp, po, pml, threadIdx.x, NCT);
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
