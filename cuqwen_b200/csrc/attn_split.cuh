// Split-KV decode attention as two launches: attn_partial_kernel (grid n_kv x nsplit) streams a contiguous key range
// per CTA and writes an un-normalised partial (O, m, l) per query head; attn_fold_kernel (one CTA per query head)
// merges the non-empty partials of its head and writes fp16.  Reference stages: src/kernels.cu:105-219 and :222-288.
//
// Compared with the single-launch variant in attn.cuh (partials merged by a ticket tree inside the same kernel) this
// trades one small extra launch - started early through programmatic dependent launch, so it is already resident when
// the partials land - for two fence + atomic + reload round trips on the critical path of the last CTAs, and it puts
// eight consumer warps on the key stream instead of four (warp pair p takes the stages sn with sn % 4 == p, each
// warp 32 of the stage's 64 keys).  Sixteen consumer warps of 16 keys each were measured and are slower (8K keys,
// 28/4 heads: 11.7 against 10.1 us for both launches; 32K: 21.0 against 17.5): the per-tile costs - one rescale of
// the output, one round of shuffles and exponentials - double while the chain a warp waits on gets no shorter.
#pragma once
#include "attn.cuh"
#include "gemv_stage.cuh"

namespace cq {

constexpr int kSplitWarps = 8;                                  // consumer warps of the partial kernel
constexpr int kSplitThreads = (kSplitWarps + 1) * 32;
constexpr int kSplitStages = 6;    // four stages being worked on by the four warp pairs, two on their way
constexpr int kFoldWarps = 16;

// stage: 64 K rows, 64 V rows and - 8-bit cache - the 64 + 64 fp32 scales of those rows
inline size_t attn_stage_bytes(int hd, bool kv8) { return kv8 ? (size_t)2 * kAttnStageKeys * hd + 2 * kAttnStageKeys * 4 : (size_t)2 * kAttnStageKeys * hd * 2; }
inline size_t attn_split_smem_bytes(int hd, int stages, bool kv8 = false) { return (size_t)stages * attn_stage_bytes(hd, kv8) + 128; }

// One cache row to its 8-bit form: scale = max|x| / 127, q = rint(x / scale) (an all-zero row: scale 0, q 0).  One warp,
// HD / 32 values per lane; `row8` and `scale` are the row's place in the cache.
template <int HD>
__device__ __forceinline__ void kv8_store_row(const __half* src, signed char* row8, float* scale, int lane) {
    constexpr int N = HD / 32;
    float v[N];
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) { v[i] = __half2float(__ldcg(src + lane * N + i)); m = fmaxf(m, fabsf(v[i])); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float sc = m / 127.0f, inv = m > 0.f ? 127.0f / m : 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) row8[lane * N + i] = (signed char)__float2int_rn(v[i] * inv);
    if (lane == 0) *scale = sc;
}

// Keys per split: an equal share rounded up to whole 16-key tiles, and never less than one ring stage - at short
// contexts fewer, fuller splits beat many splits of a tile each (512 keys over 4 KV heads: 8 splits 6.7 us, 37 splits
// 7.3 us); the splits beyond the context stay empty and the fold skips them.
__device__ __forceinline__ int attn_chunk(int len, int nsplit) {
    int chunk = (len + nsplit - 1) / nsplit;
    chunk = (chunk + 15) & ~15;
    return chunk < kAttnStageKeys ? kAttnStageKeys : chunk;
}

// (One CTA per SM by its shared memory anyway: saying so lets the compiler spend registers - 151 instead of 114 at head
// dimension 128 - which is worth 1.4 % of the 7B step.)
template <int HD, bool KV8 = false>
__global__ void __launch_bounds__(kSplitThreads, 1) attn_partial_kernel(const AttnArgs a) {
    constexpr int NCH = HD / 32, ROWB = KV8 ? HD : HD * 2, HALF = kAttnStageKeys * ROWB, NCT = kSplitWarps * 32;
    constexpr int STAGE = 2 * HALF + (KV8 ? 2 * kAttnStageKeys * 4 : 0);      // K rows, V rows, then (8-bit cache) K scales, V scales
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ float sm_o[kSplitWarps][kMaxGroup][HD];
    __shared__ float sm_ml[kSplitWarps][kMaxGroup][2];
    __shared__ __align__(8) unsigned long long sm_bar[2 * kSplitStages];

    pdl_launch_dependents();
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nst = a.stages >= 2 && a.stages <= kSplitStages ? a.stages : kSplitStages;      // ring depth of this launch
    const uint32_t stage0 = smem_u32(dyn), bar_full = smem_u32(sm_bar), bar_empty = bar_full + kSplitStages * 8;
    if (threadIdx.x == 0) {
        trace_first(a.trace, 0); trace_last(a.trace, 1); trace_start(a.trace);
        for (int s = 0; s < nst; ++s) { mbar_init(bar_full + s * 8, 1); mbar_init(bar_empty + s * 8, kSplitWarps); }
        mbar_fence_init();
    }
    __syncthreads();

    // The position is stable for the whole step (the step's first kernel is not launched early), and cache rows before
    // it were written by earlier steps: the split's key range and every stage below row `pos` need not wait for the
    // kernel before this one.  Row `pos` itself and q come from that kernel.
    const int len = *a.d_pos + 1;
    const int chunk = attn_chunk(len, a.nsplit);
    const int t0 = split * chunk;
    const int t1 = min(t0 + chunk, len);
    if (t0 >= len) return;                                       // an empty split publishes nothing; the fold skips it
    // 8-bit cache: row `pos` is not in the cache yet (this kernel puts it there); the ring carries the rows below it
    const int t1c = KV8 ? min(t1, len - 1) : t1;
    const bool owns_cur = KV8 && t1 == len;                      // this split ends with the step's own key
    const int nstage = (t1c - t0 + kAttnStageKeys - 1) / kAttnStageKeys;

    if (warp == kSplitWarps) {
        if (lane == 0) {
            const unsigned char* kb = reinterpret_cast<const unsigned char*>(a.kc) + ((size_t)kvh * a.max_seq + t0) * ROWB;
            const unsigned char* vb = reinterpret_cast<const unsigned char*>(a.vc) + ((size_t)kvh * a.max_seq + t0) * ROWB;
            bool failed = false, waited = false;
            for (int sn = 0; sn < nstage; ++sn) {
                const int s = sn % nst;
                if (!failed && !mbar_wait(bar_empty + s * 8, ((sn / nst) & 1) ^ 1)) { failed = true; if (a.err) atomicExch(a.err, 5u); }
                const int n = min(kAttnStageKeys, t1c - t0 - sn * kAttnStageKeys);
                if (!KV8 && !waited && t0 + sn * kAttnStageKeys + n == len) { pdl_wait(); waited = true; }      // the stage that holds row `pos`
                const uint32_t bytes = (uint32_t)n * ROWB;
                if (KV8) {
                    const uint32_t sbytes = (uint32_t)((n + 3) & ~3) * 4;       // whole 16-byte units; the scale arrays have room past the last row
                    const size_t k0 = (size_t)kvh * a.max_seq + t0 + (size_t)sn * kAttnStageKeys;
                    mbar_expect_tx(bar_full + s * 8, 2 * bytes + 2 * sbytes);
                    bulk_g2s(stage0 + s * STAGE + 2 * HALF, a.kscale + k0, sbytes, bar_full + s * 8);
                    bulk_g2s(stage0 + s * STAGE + 2 * HALF + kAttnStageKeys * 4, a.vscale + k0, sbytes, bar_full + s * 8);
                } else {
                    mbar_expect_tx(bar_full + s * 8, 2 * bytes);
                }
                bulk_g2s(stage0 + s * STAGE, kb + (size_t)sn * HALF, bytes, bar_full + s * 8);
                bulk_g2s(stage0 + s * STAGE + HALF, vb + (size_t)sn * HALF, bytes, bar_full + s * 8);
            }
        }
        if (owns_cur) {
            // the step's own key and value go into the cache in 8-bit form, for the steps to come (nobody reads row `pos` now)
            pdl_wait();
            const size_t row = (size_t)kvh * a.max_seq + (len - 1);
            kv8_store_row<HD>(a.k_cur + (size_t)kvh * HD, reinterpret_cast<signed char*>(const_cast<__half*>(a.kc)) + row * HD, a.kscale + row, lane);
            kv8_store_row<HD>(a.v_cur + (size_t)kvh * HD, reinterpret_cast<signed char*>(const_cast<__half*>(a.vc)) + row * HD, a.vscale + row, lane);
        }
        return;
    }
    pdl_wait();                 // q comes from the previous kernel
    if (threadIdx.x == 0) trace_first(a.trace, 2);
    const int pair = warp >> 1, wh = warp & 1;                  // stage sn belongs to the warp pair sn % 4; each warp takes 32 of its keys
    uint32_t qa[NCH][4];
    attn_load_q<HD>(qa, a.q + (size_t)kvh * a.grp * HD, a.grp, g, t);
    if (a.trace) { asm volatile("" ::"r"(qa[0][0]), "r"(qa[NCH - 1][3])); if (threadIdx.x == 0) trace_last(a.trace, 3); }
    AttnState<HD> st;
    st.reset();
    bool failed = false;
    for (int sn = 0; sn < nstage; ++sn) {
        const int s = sn % nst;
        if (!failed && !mbar_wait(bar_full + s * 8, (sn / nst) & 1)) { failed = true; if (a.err) atomicExch(a.err, 6u); }
        if (threadIdx.x == 0 && sn == 0) trace_last(a.trace, 6);
        if (threadIdx.x == 0 && sn == nstage - 1) trace_last(a.trace, 7);
        const int kb = t0 + sn * kAttnStageKeys + 32 * wh;       // first key of this warp's 32
        if ((sn & 3) == pair && kb < t1c) {
            const unsigned char* sK = dyn + s * STAGE + 32 * wh * ROWB;
            const float* sKs = reinterpret_cast<const float*>(dyn + s * STAGE + 2 * HALF) + 32 * wh;
            if constexpr (KV8) attn_tile32_q8<HD>(st, qa, sK, sK + HALF, t1c - kb, a.scale_log2, g, t, sKs, sKs + kAttnStageKeys);
            else attn_tile32<HD>(st, qa, sK, sK + HALF, t1c - kb, a.scale_log2, g, t);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + s * 8);
    }
    if (owns_cur && warp == kSplitWarps - 1)      // the step's own key, in fp16, straight from the q/k/v kernel's output
        attn_tile<HD, true>(st, qa, reinterpret_cast<const unsigned char*>(a.k_cur + (size_t)kvh * HD), reinterpret_cast<const unsigned char*>(a.v_cur + (size_t)kvh * HD),
                            1, a.scale_log2, g, t);
    if (threadIdx.x == 0) trace_last(a.trace, 4);
    attn_state_to_smem<HD>(st, &sm_o[warp][0][0], &sm_ml[warp][0][0], g, t);
    asm volatile("bar.sync 1, %0;" ::"r"(NCT) : "memory");
    float* po = a.part_o + ((size_t)(kvh * a.nsplit + split) * kMaxGroup) * HD;
    float* pml = a.part_ml + ((size_t)(kvh * a.nsplit + split) * kMaxGroup) * 2;
    attn_merge_warps<HD>(&sm_o[0][0][0], &sm_ml[0][0][0], kSplitWarps, a.grp, po, pml, threadIdx.x, NCT);
    if (threadIdx.x == 0) trace_last(a.trace, 5);
}

// One CTA per query head; warp w takes splits w, w + 16, ...; lane = 4-float column of the head.
template <int HD>
__global__ void __launch_bounds__(kFoldWarps * 32) attn_fold_kernel(const AttnArgs a) {
    constexpr int NCOL = HD / 4;
    __shared__ float4 o_w[kFoldWarps][NCOL];
    __shared__ float ml_w[kFoldWarps][2];
    pdl_launch_dependents();
    unsigned long long* tr = a.trace ? a.trace + kTraceWords : nullptr;
    if (threadIdx.x == 0) { trace_first(tr, 0); trace_last(tr, 1); }
    pdl_wait();                 // the partials come from the kernel before this one
    if (threadIdx.x == 0) trace_first(tr, 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, kvh = head / a.grp, h = head - kvh * a.grp;
    const int len = *a.d_pos + 1;
    const int chunk = attn_chunk(len, a.nsplit);
    const int nne = (len + chunk - 1) / chunk;                   // non-empty splits: 0 .. nne-1
    float M = -INFINITY, L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int NB = 4;                                        // splits in flight per warp
    for (int s0 = warp; s0 < nne; s0 += kFoldWarps * NB) {
        float mm[NB], ll[NB];
        float4 vv[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int s = s0 + i * kFoldWarps;
            mm[i] = -INFINITY; ll[i] = 0.f; vv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s < nne) {
                const size_t slot = (size_t)(kvh * a.nsplit + s) * kMaxGroup + h;
                mm[i] = __ldcg(a.part_ml + slot * 2); ll[i] = __ldcg(a.part_ml + slot * 2 + 1);
                if (lane < NCOL) vv[i] = __ldcg(reinterpret_cast<const float4*>(a.part_o + slot * HD) + lane);
            }
        }
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const float Mn = fmaxf(M, mm[i]);
            if (Mn == -INFINITY) continue;
            const float fo = M == -INFINITY ? 0.f : ex2(M - Mn), fn = mm[i] == -INFINITY ? 0.f : ex2(mm[i] - Mn);
            acc.x = acc.x * fo + vv[i].x * fn; acc.y = acc.y * fo + vv[i].y * fn; acc.z = acc.z * fo + vv[i].z * fn; acc.w = acc.w * fo + vv[i].w * fn;
            L = L * fo + ll[i] * fn; M = Mn;
        }
    }
    if (lane < NCOL) o_w[warp][lane] = acc;
    if (lane == 0) { ml_w[warp][0] = M; ml_w[warp][1] = L; }
    __syncthreads();
    if (warp == 0) {
        float Mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kFoldWarps; ++w) Mx = fmaxf(Mx, ml_w[w][0]);
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        float Ls = 0.f;
#pragma unroll
        for (int w = 0; w < kFoldWarps; ++w) {
            const float mw = ml_w[w][0];
            const float f = mw == -INFINITY ? 0.f : ex2(mw - Mx);
            if (lane < NCOL) { const float4 v = o_w[w][lane]; o.x += v.x * f; o.y += v.y * f; o.z += v.z * f; o.w += v.w * f; }
            Ls += ml_w[w][1] * f;
        }
        const float inv = 1.0f / Ls;
        const uint32_t h01 = pack_h2(o.x * inv, o.y * inv), h23 = pack_h2(o.z * inv, o.w * inv);
        if (lane < NCOL) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(a.out + (size_t)head * HD + lane * 4);
            dst[0] = h01; dst[1] = h23;
        }
        if (HD == 128 && a.xd_out) {
            // the head's 128 values are one scale group: lane l < 16 collects chunk l (the values of lanes 2l, 2l+1)
            uint4 v;
            v.x = __shfl_sync(0xffffffffu, h01, (2 * lane) & 31); v.y = __shfl_sync(0xffffffffu, h23, (2 * lane) & 31);
            v.z = __shfl_sync(0xffffffffu, h01, (2 * lane + 1) & 31); v.w = __shfl_sync(0xffffffffu, h23, (2 * lane + 1) & 31);
            if (a.quant_out == Q_I4) digits_of_chunk<Q_I4>(v, head * 16 + (lane & 15), lane < 16, a.xd_out, a.corr_out, a.xscale_out);
            else digits_of_chunk<Q_I8>(v, head * 16 + (lane & 15), lane < 16, a.xd_out, a.corr_out, a.xscale_out);
        }
        if (lane == 0) trace_last(tr, 5);
    }
}

}  // namespace cq
