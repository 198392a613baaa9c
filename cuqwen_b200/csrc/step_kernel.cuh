// One decode step's matrix and attention work as ONE persistent kernel: a CTA per SM walks a table of phases
// (per layer: RMSNorm+QKV+RoPE+KV-store, attention, o_proj+residual, RMSNorm+gate/up+SwiGLU, down+residual; then the
// final RMSNorm + lm_head), with a grid-wide barrier between phases.  Replaces the chain of launches the reference
// records into its graph (src/model.cu:76-181) by one node.
//
// Why: at batch 1 every phase is a few microseconds of HBM streaming, so kernel boundaries (drain, launch, cold
// pipeline) cost more than the streaming itself.  Here the producer warp of each CTA never stops: weights and cached
// K/V do not depend on the step's activations, so it runs ahead through the phase table, bounded only by the ring
// in shared memory, and the consumers of phase p+1 find their first stages already resident when the barrier after
// phase p opens.
//
// Rules that keep this correct:
//  * the producer reads only weights, scales and K/V rows of EARLIER tokens; the current token's K/V row (written by
//    the QKV phase of this very step) is read by a consumer warp, through L2, after the barrier;
//  * activations cross phases through global memory; writers fence before arriving at the barrier, readers use L2
//    loads (L1 may hold lines from an earlier phase);
//  * all CTAs must be co-resident (cooperative launch, grid <= SM count, one CTA per SM);
//  * every wait (mbarrier or grid barrier) is bounded; on expiry a code goes to *err and waiting stops.
#pragma once
#include "attn.cuh"
#include "gemv_kernel.cuh"

namespace cq {

enum PhaseKind : int { PH_GEMV = 0, PH_ATTN = 1, PH_FOLD = 2 };

struct alignas(64) StepPhase {
    GemvArgs g;               // PH_GEMV
    AttnArgs at;              // PH_ATTN: kc / vc = this layer's caches; part_* / counters = scratch
    const __half* k_cur;      // PH_ATTN: the current token's K and V, [n_kv][hd] (what the QKV phase wrote)
    const __half* v_cur;
    int kind, quant, epi, pad;
};

struct StepArgs {
    const StepPhase* phases;
    int nphases;
    unsigned* bar;            // grid barrier counter, zero at launch
    unsigned* err;
    unsigned long long* trace;// optional [nphases][grid][4] %globaltimer stamps (consumers enter a phase, x staged, leave, spare), else null
    int hd;                   // head dimension (64 or 128)
    int debug;                // development aid: bit 0 = consumers skip the arithmetic (measures the copy path alone)
    // shared-memory map (see RingCtx); the x area at offset 0 also serves as the attention merge scratch
    int off_corr, off_xscale, off_red, off_scales, scale_block_bytes, off_stages, slot_bytes, nslots, off_bars, smem_bytes;
};

constexpr int kStepAttnKeys = 64;     // keys per ring slot in the attention phase (K half, then V half)

// Grid-wide barrier among the consumer threads of all CTAs.  `target` = arrivals expected so far.
__device__ __forceinline__ void grid_sync(unsigned* bar, unsigned target, RingCtx& R) {
    consumer_sync(kConsumerThreads);
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(bar, 1u);
        if (!R.failed) {
            const unsigned long long t0 = global_ns();
            for (;;) {
                unsigned v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
                if ((int)(v - target) >= 0) break;
                if (R.err && *reinterpret_cast<volatile unsigned*>(R.err)) { R.failed = true; break; }      // someone already gave up
                if (global_ns() - t0 > 2000000000ull) { R.failed = true; if (R.err) atomicExch(R.err, 7u); break; }
            }
        }
    }
    consumer_sync(kConsumerThreads);
}

struct AttnSpan { int kvh, split, len, t0, t1, t1c, nstage, chunk; bool active; };
// Key range of CTA `cta` in the attention phase.  t1c: end of the part that comes from the cache (keys before pos).
__device__ __forceinline__ AttnSpan attn_span(const AttnArgs& a, int cta) {
    AttnSpan s;
    s.active = cta < a.n_kv * a.nsplit;
    s.kvh = cta / a.nsplit; s.split = cta - s.kvh * a.nsplit;
    s.len = *a.d_pos + 1;
    int chunk = (s.len + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + 15) & ~15;
    s.chunk = chunk;
    s.t0 = s.split * chunk;
    s.t1 = min(s.t0 + chunk, s.len);
    s.t1c = min(s.t1, s.len - 1);
    s.nstage = (s.active && s.t0 < s.t1c) ? (s.t1c - s.t0 + kStepAttnKeys - 1) / kStepAttnKeys : 0;     // producer and consumers agree on this
    return s;
}

template <int HD>
__device__ __forceinline__ void step_attn_produce(const StepPhase& ph, RingCtx& ring, int cta) {
    RingCtx R = ring;
    struct Back { RingCtx& dst; RingCtx& src; __device__ ~Back() { dst = src; } } back{ring, R};     // every return path hands the ring position back
    constexpr int ROWB = HD * 2, HALF = kStepAttnKeys * ROWB;
    const AttnArgs& a = ph.at;
    const AttnSpan sp = attn_span(a, cta);
    const int lane = threadIdx.x & 31;
    const unsigned char* kb = reinterpret_cast<const unsigned char*>(a.kc) + ((size_t)sp.kvh * a.max_seq + sp.t0) * ROWB;
    const unsigned char* vb = reinterpret_cast<const unsigned char*>(a.vc) + ((size_t)sp.kvh * a.max_seq + sp.t0) * ROWB;
    for (int sn = 0; sn < sp.nstage; ++sn) {
        const int s = R.slot;
        R.wait(R.bar_empty + s * 8, R.par ^ 1u, 5u);
        if (lane == 0) {
            const int n = min(kStepAttnKeys, sp.t1c - sp.t0 - sn * kStepAttnKeys);
            const uint32_t bytes = (uint32_t)n * ROWB, dst = R.sm0 + R.off_stages + s * R.slot_bytes;
            mbar_expect_tx(R.bar_full + s * 8, 2 * bytes);
            bulk_g2s(dst, kb + (size_t)sn * HALF, bytes, R.bar_full + s * 8);
            bulk_g2s(dst + HALF, vb + (size_t)sn * HALF, bytes, R.bar_full + s * 8);
        }
        __syncwarp();
        R.advance();
    }
}

constexpr int kStepAttnWarps = 8;      // consumer warps that compute in the attention phase; the others only pass the ring on

// Consumers: warps 0-3 take the even stages, warps 4-7 the odd ones (one 16-key tile per warp per stage); warp 7 of
// the CTA whose range holds the current position adds that key from the QKV phase's output.  The CTA's partial
// (un-normalised O, m, l per head) goes to slot [kvh][split]; the fold phase that follows merges the slots.
template <int HD>
__device__ __forceinline__ void step_attn_consume(const StepPhase& ph, RingCtx& ring, int cta) {
    RingCtx R = ring;
    struct Back { RingCtx& dst; RingCtx& src; __device__ ~Back() { dst = src; } } back{ring, R};     // every return path hands the ring position back
    constexpr int ROWB = HD * 2, HALF = kStepAttnKeys * ROWB, NCH = HD / 32, NC = kConsumerThreads;
    const AttnArgs& a = ph.at;
    const AttnSpan sp = attn_span(a, cta);
    if (!sp.active || sp.t0 >= sp.len) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int half_id = warp >> 2, wq = warp & 3;
    const bool worker = warp < kStepAttnWarps;
    float* o_all = reinterpret_cast<float*>(R.base);                                  // [8 warps][kMaxGroup][HD]
    float* ml_all = o_all + (size_t)kStepAttnWarps * kMaxGroup * HD;                  // [8 warps][kMaxGroup][2]
    const bool owns_cur = sp.t0 <= sp.len - 1 && sp.len - 1 < sp.t1;
    uint32_t qa[NCH][4];
    AttnState<HD> st;
    if (worker) { attn_load_q<HD>(qa, a.q + (size_t)sp.kvh * a.grp * HD, a.grp, g, t); st.reset(); }
    for (int sn = 0; sn < sp.nstage; ++sn) {
        const int s = R.slot;
        R.wait(R.bar_full + s * 8, R.par, 6u);
        const int kb = sp.t0 + sn * kStepAttnKeys + 16 * wq;
        if (worker && (sn & 1) == half_id && kb < sp.t1c) {
            const unsigned char* sK = R.base + R.off_stages + s * R.slot_bytes + 16 * wq * ROWB;
            attn_tile<HD, false>(st, qa, sK, sK + HALF, sp.t1c - kb, a.scale_log2, g, t);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(R.bar_empty + s * 8);
        R.advance();
    }
    if (worker) {
        if (owns_cur && warp == kStepAttnWarps - 1)
            attn_tile<HD, true>(st, qa, reinterpret_cast<const unsigned char*>(ph.k_cur + (size_t)sp.kvh * HD),
                                reinterpret_cast<const unsigned char*>(ph.v_cur + (size_t)sp.kvh * HD), 1, a.scale_log2, g, t);
        attn_state_to_smem<HD>(st, o_all + (size_t)warp * kMaxGroup * HD, ml_all + warp * kMaxGroup * 2, g, t);
    }
    consumer_sync(NC);
    float* po = a.part_o + ((size_t)(sp.kvh * a.nsplit + sp.split) * kMaxGroup) * HD;
    float* pml = a.part_ml + ((size_t)(sp.kvh * a.nsplit + sp.split) * kMaxGroup) * 2;
    attn_merge_warps<HD>(o_all, ml_all, kStepAttnWarps, a.grp, po, pml, threadIdx.x, NC);
}

// Fold phase: CTA `head` (then head + grid, ...) merges the non-empty splits of one query head.  Warp w takes splits
// w, w + 16, ...; lane = 4-float column of the head; the warps' results meet in shared memory and warp 0 writes fp16.
// Reference: stage 2 of the split-KV attention, src/kernels.cu:222-288.
template <int HD>
__device__ __forceinline__ void step_attn_fold(const StepPhase& ph, RingCtx& R, int cta, int ncta) {
    constexpr int NCOL = HD / 4, NC = kConsumerThreads;
    const AttnArgs& a = ph.at;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int len = *a.d_pos + 1;
    int chunk = (len + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + 15) & ~15;
    const int nne = (len + chunk - 1) / chunk;                       // non-empty splits: 0 .. nne-1
    float4* o_w = reinterpret_cast<float4*>(R.base);                 // [16 warps][NCOL]
    float* ml_w = reinterpret_cast<float*>(R.base + kConsumerWarps * HD * 4);     // [16 warps][2]
    for (int head = cta; head < a.n_kv * a.grp; head += ncta) {
        const int kvh = head / a.grp, h = head - kvh * a.grp;
        float M = -INFINITY, L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        constexpr int NB = 4;                                        // splits in flight per warp (L2 round trips overlap)
        for (int s0 = warp; s0 < nne; s0 += kConsumerWarps * NB) {
          float mm[NB], ll[NB]; float4 vv[NB];
#pragma unroll
          for (int i = 0; i < NB; ++i) {
            const int s = s0 + i * kConsumerWarps;
            mm[i] = -INFINITY; ll[i] = 0.f; vv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s < nne) {
                const size_t slot = (size_t)(kvh * a.nsplit + s) * kMaxGroup + h;
                mm[i] = __ldcg(a.part_ml + slot * 2); ll[i] = __ldcg(a.part_ml + slot * 2 + 1);
                if (lane < NCOL) vv[i] = __ldcg(reinterpret_cast<const float4*>(a.part_o + slot * HD) + lane);
            }
          }
#pragma unroll
          for (int i = 0; i < NB; ++i) {
            const float m = mm[i], l = ll[i]; const float4 v = vv[i];
            const float Mn = fmaxf(M, m);
            if (Mn == -INFINITY) continue;
            const float fo = M == -INFINITY ? 0.f : ex2(M - Mn), fn = m == -INFINITY ? 0.f : ex2(m - Mn);
            acc.x = acc.x * fo + v.x * fn; acc.y = acc.y * fo + v.y * fn; acc.z = acc.z * fo + v.z * fn; acc.w = acc.w * fo + v.w * fn;
            L = L * fo + l * fn; M = Mn;
          }
        }
        if (lane < NCOL) o_w[warp * NCOL + lane] = acc;
        if (lane == 0) { ml_w[warp * 2] = M; ml_w[warp * 2 + 1] = L; }
        consumer_sync(NC);
        if (warp == 0) {
            float Mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) Mx = fmaxf(Mx, ml_w[w * 2]);
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            float Ls = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                const float mw = ml_w[w * 2];
                const float f = mw == -INFINITY ? 0.f : ex2(mw - Mx);
                if (lane < NCOL) { const float4 v = o_w[w * NCOL + lane]; o.x += v.x * f; o.y += v.y * f; o.z += v.z * f; o.w += v.w * f; }
                Ls += ml_w[w * 2 + 1] * f;
            }
            if (lane < NCOL) {
                const float inv = 1.0f / Ls;
                __half2* dst = reinterpret_cast<__half2*>(a.out + (size_t)head * HD + lane * 4);
                dst[0] = __floats2half2_rn(o.x * inv, o.y * inv);
                dst[1] = __floats2half2_rn(o.z * inv, o.w * inv);
            }
        }
        consumer_sync(NC);
    }
}

template <int Q, int EPI>
__device__ __forceinline__ void step_gemv_produce(const GemvArgs& a, RingCtx& ring, int cta, int ncta) {
    RingCtx R = ring;
    gemv_produce<Q, EPI>(a, R, cta, ncta);
    ring = R;
}
template <int Q, int EPI>
__device__ __forceinline__ void step_gemv_consume(const GemvArgs& a, RingCtx& ring, int cta, int ncta) {
    RingCtx R = ring;
    gemv_consume<Q, EPI>(a, R, cta, ncta);
    ring = R;
}

template <int Q, bool PRODUCER>
__device__ __forceinline__ void step_gemv_phase(const StepPhase& ph, RingCtx& R, int cta, int ncta) {
#define CQ_RUN(QQ, EE) do { if (PRODUCER) step_gemv_produce<QQ, EE>(ph.g, R, cta, ncta); else step_gemv_consume<QQ, EE>(ph.g, R, cta, ncta); } while (0)
    switch (ph.epi) {
        case EPI_QKV: CQ_RUN(Q, EPI_QKV); break;
        case EPI_RESID: CQ_RUN(Q, EPI_RESID); break;
        case EPI_SWIGLU: CQ_RUN(Q, EPI_SWIGLU); break;
        default:   // the lm_head: int8 in quantised untied files, fp16 otherwise
            if (Q != Q_F16 && ph.quant == Q_I8) CQ_RUN(Q_I8, EPI_F16); else CQ_RUN(Q_F16, EPI_F16);
            break;
    }
#undef CQ_RUN
}

// Q: quantisation of the layer matrices.
template <int Q>
__global__ void __launch_bounds__(kGemvThreads, 1) decode_step_kernel(const __grid_constant__ StepArgs sa) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    RingCtx R;
    R.sm0 = smem_u32(smem_raw); R.base = smem_raw;
    R.off_corr = sa.off_corr; R.off_xscale = sa.off_xscale; R.off_red = sa.off_red; R.off_scales = sa.off_scales;
    R.scale_block_bytes = sa.scale_block_bytes; R.off_stages = sa.off_stages; R.slot_bytes = sa.slot_bytes; R.nslots = sa.nslots;
    R.bar_full = R.sm0 + sa.off_bars; R.bar_empty = R.bar_full + sa.nslots * 8; R.bar_sfull = R.bar_empty + sa.nslots * 8; R.bar_sempty = R.bar_sfull + 16;
    R.bar_x = R.bar_sempty + 16; R.xpar = 0u;
    R.slot = 0; R.par = 0; R.sj = 0; R.err = sa.err; R.failed = false; R.skip_math = (sa.debug & 1) != 0; R.stamp = nullptr;
    if (threadIdx.x == 0) ring_init_barriers(R);
    __syncthreads();
    const int cta = blockIdx.x, ncta = gridDim.x;
    if ((threadIdx.x >> 5) == kConsumerWarps) {
        for (int p = 0; p < sa.nphases; ++p) {
            const StepPhase& ph = sa.phases[p];
            if (ph.kind == PH_ATTN) { if (sa.hd == 128) step_attn_produce<128>(ph, R, cta); else step_attn_produce<64>(ph, R, cta); }
            else if (ph.kind == PH_GEMV) step_gemv_phase<Q, true>(ph, R, cta, ncta);
        }
        return;
    }
    for (int p = 0; p < sa.nphases; ++p) {
        const StepPhase& ph = sa.phases[p];
        if (sa.trace) { R.stamp = sa.trace + ((size_t)p * ncta + cta) * 4 + 1; if (threadIdx.x == 0) { R.stamp[-1] = global_ns(); R.stamp[0] = 0; } }
        if (ph.kind == PH_ATTN) { if (sa.hd == 128) step_attn_consume<128>(ph, R, cta); else step_attn_consume<64>(ph, R, cta); }
        else if (ph.kind == PH_FOLD) { if (sa.hd == 128) step_attn_fold<128>(ph, R, cta, ncta); else step_attn_fold<64>(ph, R, cta, ncta); }
        else step_gemv_phase<Q, false>(ph, R, cta, ncta);
        if (sa.trace && threadIdx.x == 0) sa.trace[((size_t)p * ncta + cta) * 4 + 2] = global_ns();
        if (p + 1 < sa.nphases && threadIdx.x < (int)(sizeof(StepPhase) + 127) / 128)      // next phase's descriptor: into L1 while the barrier settles
            asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const char*>(sa.phases + p + 1) + threadIdx.x * 128));
        if (p + 1 < sa.nphases) grid_sync(sa.bar, (unsigned)(p + 1) * (unsigned)ncta, R);
    }
}

}  // namespace cq
