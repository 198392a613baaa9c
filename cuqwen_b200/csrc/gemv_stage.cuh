// Prologue of the GEMV kernels: bring the activation vector into shared memory in the form the inner loop wants,
// optionally applying RMSNorm first (reference src/kernels.cu:689-751: out = half(float(x) * inv_rms * float(w))).
//
// The vector lives in L2 (another SM wrote it moments ago), so a load costs a full L2 round trip.  Staging is
// therefore two steps: (1) every thread issues all its loads of x (and of the norm weight) at once and parks the raw
// fp16 data in shared memory, summing squares on the way; (2) after one barrier the data is converted in place from
// shared memory (normalise, then either leave fp16 or rewrite as integer digits), one chunk per lane per turn, with
// short latencies and small register needs.
#pragma once
#include "gemv_math.cuh"

namespace cq {

// Barrier among the first `nthreads` threads of the CTA (the consumer warps); a producer warp beyond them does not take part.
__device__ __forceinline__ void consumer_sync(int nthreads) { asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory"); }

// Block-wide sum over the first `nthreads` threads -> rsqrt(sum / dim + eps).  `red` holds >= 33 floats.
// Contains two barriers; everything written to shared memory before the call is visible after it.
__device__ __forceinline__ float consumers_rsqrt_mean(float ss, int dim, float eps, float* red, int nthreads) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    consumer_sync(nthreads);
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (nthreads >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[32] = rsqrtf(v / (float)dim + eps);
    }
    consumer_sync(nthreads);
    return red[32];
}

__device__ __forceinline__ float chunk_sumsq(const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h[k]); ss += f.x * f.x + f.y * f.y; }
    return ss;
}

__device__ __forceinline__ uint4 apply_norm(uint4 v, const uint4& wv, float inv) {
    __half2* xh = reinterpret_cast<__half2*>(&v);
    const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 xf = __half22float2(xh[k]), wf = __half22float2(wh[k]);
        xh[k] = __floats2half2_rn(xf.x * inv * wf.x, xf.y * inv * wf.y);
    }
    return v;
}

// Step 1 for NB chunks per thread per turn: chunk i of a turn is c8 = base + i * nthreads + threadIdx.x.  x through L2
// (coherent), the norm weight through the read-only path; all loads of a turn are issued before the first store.
template <int NB, bool NORM, bool PARKW>
__device__ __forceinline__ float park_raw(const __half* x, const __half* norm_w, int nchunk, uint4* raw, uint4* wraw, int nthreads) {
    float ss = 0.f;
    for (int base = 0; base < nchunk; base += nthreads * NB) {
        uint4 v[NB], w[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int c8 = base + i * nthreads + threadIdx.x;
            if (c8 < nchunk) {
                v[i] = __ldcg(reinterpret_cast<const uint4*>(x) + c8);
                if (PARKW) w[i] = __ldg(reinterpret_cast<const uint4*>(norm_w) + c8);
            }
        }
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int c8 = base + i * nthreads + threadIdx.x;
            if (c8 < nchunk) {
                raw[c8] = v[i];
                if (PARKW) wraw[c8] = w[i];
                if (NORM) ss += chunk_sumsq(v[i]);
            }
        }
    }
    return ss;
}

// Tensor-parallel consumer side of an exchange (see GemvArgs): what park_raw does, for x_new = half(float(x) + sum over
// ranks of the fp32 partials in this rank's receive slots), summed in rank order so every rank forms the same bits.
// A slot word is {value bits, sequence number}; a word whose number is not `seq` yet has not arrived and is read again
// (bounded: after `limit` SM cycles, by default 4e9 = two to four seconds, *err is set and the stale value is used).
// store_next: this CTA also writes x_new to global memory for the kernels after this one.
struct GatherSrc {
    const uint2* slots;      // [n][K] words
    int n;
    unsigned seq;
    __half* x_next;          // written when store_next
    bool store_next;
    unsigned* err;
    long long limit;         // SM cycles after which the re-read loop gives up
};
// One chunk of eight values: x's chunk plus the ranks' partials for it, summed in rank order.  gave_up: set (and kept)
// once the bounded re-read loop has expired for this thread.
__device__ __forceinline__ uint4 gather_chunk(const GatherSrc& gs, int K, int c8, const uint4& xo, bool& gave_up) {
    constexpr int RB = 2;                                  // source ranks whose loads are in flight together
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r0 = 0; r0 < gs.n; r0 += RB) {
        unsigned long long q[RB][8];
        unsigned long long t0 = 0ull;
        for (;;) {
            bool ok = true;
#pragma unroll
            for (int j = 0; j < RB; ++j)
                if (r0 + j < gs.n) {
                    const uint2* p = gs.slots + (size_t)(r0 + j) * K + (size_t)c8 * 8;
#pragma unroll
                    for (int i = 0; i < 4; ++i) ld_pair2(p + 2 * i, q[j][2 * i], q[j][2 * i + 1]);
                }
#pragma unroll
            for (int j = 0; j < RB; ++j)
                if (r0 + j < gs.n) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) ok = ok && pair_seq(q[j][i]) == gs.seq;
                }
            if (ok || gave_up) break;
            const unsigned long long now = (unsigned long long)sm_cycles();      // the SM's cycle counter: cheap to read
            if (t0 == 0ull) t0 = now | 1ull;
            else if (now - t0 > (unsigned long long)gs.limit) { gave_up = true; if (gs.err) atomicExch(gs.err, 8u); break; }
        }
#pragma unroll
        for (int j = 0; j < RB; ++j)
            if (r0 + j < gs.n) {
#pragma unroll
                for (int i = 0; i < 8; ++i) s[i] += pair_val(q[j][i]);
            }
    }
    uint4 xn;
    const __half2* h = reinterpret_cast<const __half2*>(&xo);
    __half2* o = reinterpret_cast<__half2*>(&xn);
#pragma unroll
    for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h[k]); o[k] = __floats2half2_rn(f.x + s[2 * k], f.y + s[2 * k + 1]); }
    return xn;
}
template <bool PARKW>
__device__ __forceinline__ float park_gather(const __half* x, const __half* norm_w, const GatherSrc& gs, int K, int nchunk, uint4* raw, uint4* wraw, int nthreads) {
    float ss = 0.f;
    bool gave_up = false;
    for (int c8 = threadIdx.x; c8 < nchunk; c8 += nthreads) {
        const uint4 xo = __ldcg(reinterpret_cast<const uint4*>(x) + c8);
        uint4 wv = make_uint4(0u, 0u, 0u, 0u);
        if (PARKW) wv = __ldg(reinterpret_cast<const uint4*>(norm_w) + c8);
        const uint4 xn = gather_chunk(gs, K, c8, xo, gave_up);
        raw[c8] = xn;
        if (PARKW) wraw[c8] = wv;
        if (gs.store_next) reinterpret_cast<uint4*>(gs.x_next)[c8] = xn;
        ss += chunk_sumsq(xn);
    }
    return ss;
}

// Quantised weights: per 128-column group, integers X = rint(x * 2^e) with |X| < 2^14, as two signed byte digits in
// the order the B operand wants (see mma_group_int), plus per group  corr = 8 * sum(X)  (int4 only, else 0) and
// xscale = 2^-e.  Digit block of a group: [half jj (2)][t (4)][plane (2)][16 bytes]; the 16 bytes are two 8-byte
// units, each the eight elements of one 32-bit weight word: int4 order e0,e2,e4,e6,e1,e3,e5,e7, int8 natural order.
// Sixteen consecutive lanes hold the sixteen chunks of one group; whole warps call this together (full shuffles).
// The digit block of a group occupies the very 256 bytes its fp16 values came from: the shuffles below sit between a
// lane's read of its chunk and anybody's write, so the rewrite in place is safe within the warp.
template <int Q>
__device__ __forceinline__ void digits_of_chunk(uint4 v, int c8, bool live, unsigned char* xd, int* corr, float* xscale) {
    float f[8];
    {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) { const float2 p = __half22float2(h[k]); f[2 * k] = p.x; f[2 * k + 1] = p.y; }
    }
    float m = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(f[k]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // m in [2^p, 2^(p+1))  ->  e = 13 - p  ->  |X| < 2^14
    int e = 0;
    if (m > 0.f) e = 13 - ((int)((__float_as_uint(m) >> 23) & 0xff) - 127);
    const float up = __uint_as_float((uint32_t)(e + 127) << 23);
    int X[8], sum = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) { X[k] = __float2int_rn(f[k] * up); sum += X[k]; }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncwarp();
    if (!live) return;
    uint32_t d0[8], d1[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int lo = (int)(signed char)(X[k] & 0xff);
        d0[k] = (uint32_t)lo & 0xffu;
        d1[k] = (uint32_t)((X[k] - lo) >> 8) & 0xffu;
    }
    const int grp = c8 >> 4, r = c8 & 15;
    uint2 p0, p1;
    int off;
    if (Q == Q_I4) {
        const int t = r >> 2, j = r & 3;
        off = grp * 256 + (j >> 1) * 128 + t * 32 + (j & 1) * 8;
        p0.x = d0[0] | d0[2] << 8 | d0[4] << 16 | d0[6] << 24; p0.y = d0[1] | d0[3] << 8 | d0[5] << 16 | d0[7] << 24;
        p1.x = d1[0] | d1[2] << 8 | d1[4] << 16 | d1[6] << 24; p1.y = d1[1] | d1[3] << 8 | d1[5] << 16 | d1[7] << 24;
    } else {
        const int i = r >> 3, t = (r >> 1) & 3;
        off = grp * 256 + i * 128 + t * 32 + (r & 1) * 8;
        p0.x = d0[0] | d0[1] << 8 | d0[2] << 16 | d0[3] << 24; p0.y = d0[4] | d0[5] << 8 | d0[6] << 16 | d0[7] << 24;
        p1.x = d1[0] | d1[1] << 8 | d1[2] << 16 | d1[3] << 24; p1.y = d1[4] | d1[5] << 8 | d1[6] << 16 | d1[7] << 24;
    }
    *reinterpret_cast<uint2*>(xd + off) = p0;          // plane 0
    *reinterpret_cast<uint2*>(xd + off + 16) = p1;     // plane 1
    if (r == 0) {
        corr[grp] = Q == Q_I4 ? 8 * sum : 0;
        xscale[grp] = __uint_as_float((uint32_t)(127 - e) << 23);
    }
}

// Short vectors (at most NB * nthreads chunks of eight values): the whole vector fits the consumers' registers, so it
// is fetched with plain loads - every load of the CTA in flight at once, an L2 hit each - normalised and converted
// straight from registers, and only the final form touches shared memory.  Same arithmetic, same bits as the staged
// path below.  Thread tid owns chunks tid, tid + nthreads, ...: a warp's lanes hold consecutive chunks, sixteen lanes
// one 128-column group, as digits_of_chunk wants.
template <int Q, int NB>
__device__ __forceinline__ void stage_x_regs(const __half* x, const __half* norm_w, float eps, int K, unsigned char* xd, int* corr, float* xscale,
                                             float* red, int nthreads, unsigned long long* trace = nullptr) {
    const int nchunk = K / 8;
    uint4 v[NB], w[NB];
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const int c8 = i * nthreads + threadIdx.x;
        v[i] = make_uint4(0u, 0u, 0u, 0u); w[i] = v[i];
        if (c8 < nchunk) {
            v[i] = __ldcg(reinterpret_cast<const uint4*>(x) + c8);
            if (norm_w) w[i] = __ldg(reinterpret_cast<const uint4*>(norm_w) + c8);
        }
    }
    if (norm_w) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NB; ++i) ss += chunk_sumsq(v[i]);
        if (trace && threadIdx.x == 0 && ss >= 0.f) trace_last(trace, 6);
        const float inv = consumers_rsqrt_mean(ss, K, eps, red, nthreads);
        if (trace && threadIdx.x == 0 && inv >= 0.f) trace_last(trace, 7);
#pragma unroll
        for (int i = 0; i < NB; ++i) v[i] = apply_norm(v[i], w[i], inv);
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const int c8 = i * nthreads + threadIdx.x;
        if ((i * nthreads + (threadIdx.x & ~31)) >= nchunk) break;        // whole warp beyond the vector (uniform)
        if (Q == Q_F16) { if (c8 < nchunk) reinterpret_cast<uint4*>(xd)[c8] = v[i]; }
        else digits_of_chunk<Q>(v[i], c8, c8 < nchunk, xd, corr, xscale);
    }
    consumer_sync(nthreads);
}

// Stage x for the kernel of quantisation Q: digits (int4 / int8, into xd + corr + xscale) or plain fp16 (xd as uint4[]).
// xarea_bytes: shared memory available from xd on; the norm weight is parked at xd + 2K when 4K bytes fit (else it
// is re-read from global memory during the conversion).
// bar_x / xpar: an mbarrier (shared-window address) and its current parity; when given and the sources are 16-byte
// aligned, step 1 is two bulk copies issued by one thread (x through L2, the norm weight beside it) instead of
// per-thread loads: one instruction, no registers, the whole vector in flight at once.  Returns whether the barrier
// was used (the caller then flips the parity).
template <int Q>
__device__ __forceinline__ bool stage_x(const __half* x, const __half* norm_w, float eps, int K, unsigned char* xd, int xarea_bytes, int* corr, float* xscale,
                                        float* red, int nthreads, const GatherSrc* gs = nullptr, uint32_t bar_x = 0u, uint32_t xpar = 0u, unsigned long long* trace = nullptr) {
    const int nchunk = K / 8, lane = threadIdx.x & 31;
    uint4* raw = reinterpret_cast<uint4*>(xd);
    uint4* wraw = raw + nchunk;
    const bool w_parked = norm_w && 4 * K <= xarea_bytes;
    const bool gather = gs && gs->n > 0;
    // (The tensor-parallel gather stays out of the register path: inlined there it raised every GEMV kernel from 96-110
    // to 124-126 registers, which ends two CTAs sharing an SM - 690 -> 570 tok/s on one GPU.)
    if (!gather && nchunk <= 3 * nthreads && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (!norm_w || (reinterpret_cast<uintptr_t>(norm_w) & 15) == 0)) {
        if (nchunk <= 2 * nthreads) stage_x_regs<Q, 2>(x, norm_w, eps, K, xd, corr, xscale, red, nthreads, trace);
        else stage_x_regs<Q, 3>(x, norm_w, eps, K, xd, corr, xscale, red, nthreads, trace);
        return false;
    }
    const bool bulk = bar_x != 0u && !gather && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (!norm_w || (w_parked && (reinterpret_cast<uintptr_t>(norm_w) & 15) == 0));
    float inv = 0.f;
    if (bulk) {
        if (threadIdx.x == 0) {
            fence_async_smem();                        // earlier generic-proxy accesses to this area come before the copy's writes
            mbar_expect_tx(bar_x, (uint32_t)(K * 2) * (norm_w ? 2u : 1u));
            bulk_g2s(smem_u32(raw), x, (uint32_t)(K * 2), bar_x);
            if (norm_w) bulk_g2s(smem_u32(wraw), norm_w, (uint32_t)(K * 2), bar_x);
        }
        mbar_wait(bar_x, xpar);                        // bounded; on expiry the vector is garbage and the ring waits report it
        if (norm_w) {
            float ss = 0.f;
            for (int c8 = threadIdx.x; c8 < nchunk; c8 += nthreads) ss += chunk_sumsq(raw[c8]);
            inv = consumers_rsqrt_mean(ss, K, eps, red, nthreads);
        }
    } else if (norm_w) {
        float ss;
        if (gather) ss = w_parked ? park_gather<true>(x, norm_w, *gs, K, nchunk, raw, wraw, nthreads) : park_gather<false>(x, norm_w, *gs, K, nchunk, raw, wraw, nthreads);
        else ss = w_parked ? park_raw<4, true, true>(x, norm_w, nchunk, raw, wraw, nthreads) : park_raw<4, true, false>(x, norm_w, nchunk, raw, wraw, nthreads);
        inv = consumers_rsqrt_mean(ss, K, eps, red, nthreads);
    } else {
        park_raw<5, false, false>(x, nullptr, nchunk, raw, nullptr, nthreads);
        consumer_sync(nthreads);
    }
    if (Q == Q_F16 && !norm_w) return bulk;            // raw fp16 is what the fp16 kernel wants
#pragma unroll 1
    for (int base = threadIdx.x & ~31; base < nchunk; base += nthreads) {
        const int c8 = base + lane;
        const bool live = c8 < nchunk;
        uint4 xv = make_uint4(0u, 0u, 0u, 0u);
        if (live) {
            xv = raw[c8];
            if (norm_w) xv = apply_norm(xv, w_parked ? wraw[c8] : __ldg(reinterpret_cast<const uint4*>(norm_w) + c8), inv);
        }
        if (Q == Q_F16) { if (live) raw[c8] = xv; }
        else digits_of_chunk<Q>(xv, c8, live, xd, corr, xscale);
    }
    consumer_sync(nthreads);
    return bulk;                                       // true: the barrier completed a phase, its parity flips
}

}  // namespace cq
