// Prologue of the GEMV kernels: bring the activation vector into shared memory in the form the inner loop wants,
// optionally applying RMSNorm first (reference src/kernels.cu:689-751: out = half(float(x) * inv_rms * float(w))).
#pragma once
#include "gemv_math.cuh"

namespace cq {

// Barrier among the first `nthreads` threads of the CTA (the consumer warps); a producer warp beyond them does not take part.
__device__ __forceinline__ void consumer_sync(int nthreads) { asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory"); }

// sum of squares -> 1/rms over the first `nthreads` threads.  `red` holds >= 33 floats.
__device__ __forceinline__ float consumers_inv_rms(const __half* __restrict__ x, int dim, float eps, float* red, int nthreads) {
    float ss = 0.f;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int i = threadIdx.x; i < dim / 8; i += nthreads) {
        const uint4 v = __ldcg(xv + i);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h[k]); ss += f.x * f.x + f.y * f.y; }
    }
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

// One 8-element chunk of x, normalised if asked, as fp16 bits.  Coherent (L2) loads: x may have been written by
// another SM moments ago.
__device__ __forceinline__ uint4 load_x_chunk(const __half* x, const __half* norm_w, float inv, int c8) {
    uint4 v = __ldcg(reinterpret_cast<const uint4*>(x) + c8);
    if (norm_w) {
        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(norm_w) + c8);
        __half2* xh = reinterpret_cast<__half2*>(&v);
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 xf = __half22float2(xh[k]), wf = __half22float2(wh[k]);
            xh[k] = __floats2half2_rn(xf.x * inv * wf.x, xf.y * inv * wf.y);
        }
    }
    return v;
}

// fp16 weights: x in natural order.
__device__ __forceinline__ void stage_x_f16(const __half* x, const __half* norm_w, float eps, int K, uint4* xs, float* red, int nthreads) {
    float inv = 0.f;
    if (norm_w) inv = consumers_inv_rms(x, K, eps, red, nthreads);
    for (int c8 = threadIdx.x; c8 < K / 8; c8 += nthreads) xs[c8] = load_x_chunk(x, norm_w, inv, c8);
    consumer_sync(nthreads);
}

// Quantised weights: per 128-column group, integers X = rint(x * 2^e) with |X| < 2^14, as two signed byte digits in
// the order the B operand wants (see compute_group_int), plus per group  corr = 8 * sum(X)  (int4 only, else 0) and
// xscale = 2^-e.  Digit block of a group: [half jj (2)][t (4)][plane (2)][16 bytes]; the 16 bytes are two 8-byte
// units, each the eight elements of one 32-bit weight word: int4 order e0,e2,e4,e6,e1,e3,e5,e7, int8 natural order.
template <int Q>
__device__ __forceinline__ void stage_x_digits(const __half* x, const __half* norm_w, float eps, int K, unsigned char* xd, int* corr, float* xscale, float* red, int nthreads) {
    float inv = 0.f;
    if (norm_w) inv = consumers_inv_rms(x, K, eps, red, nthreads);
    const int nchunk = K / 8, lane = threadIdx.x & 31;
    // sixteen consecutive lanes hold the sixteen chunks of one group; whole warps iterate together so the shuffles are full
    for (int base = (threadIdx.x & ~31); base < nchunk; base += nthreads) {
        const int c8 = base + lane;
        const bool live = c8 < nchunk;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (live) v = load_x_chunk(x, norm_w, inv, c8);
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
        if (live) {
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
    }
    consumer_sync(nthreads);
}

}  // namespace cq
