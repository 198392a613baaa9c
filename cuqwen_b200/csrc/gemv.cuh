// Weight-streaming GEMV family for batch-1 decode on sm_100a.
//
// y[r] = sum_k W[r,k] * x[k], W row-major fp16 / int8 / packed int4 with one
// fp16 scale per 128 input columns (the on-disk layout of the reference,
// export_weights.py:123-205).  The math of one 8-wide chunk in the reference is
// "p = sum float(q)*float(x); acc += p*scale" (src/kernels.cu:11-57); here the
// integer-times-activation products of one whole 128-column group are summed in
// fp32 by the tensor core and the group scale is applied once per group, which
// is the same real-number expression with a different summation order.
//
// How a warp works: it owns 16 output rows (x MT matrices).  Lane 4g+t streams
// 16 bytes per row-group from rows g and g+8 straight from HBM into registers,
// turns the integers into fp16 with a magic-exponent trick (two weights per
// LOP3/PRMT, no int->float converts), and feeds them as the A operand of
// mma.sync.m16n8k16; the activation vector sits in shared memory, pre-permuted
// so one LDS.128 yields the B operand of two MMA steps.  The fp16 magic adds a
// constant offset (72 for int4, 1152 for int8) to every weight; it is removed
// per group with offset * sum(x over the group), computed once per CTA.
#pragma once
#include "common.cuh"

namespace cq {

enum Epi : int { EPI_F16 = 0, EPI_F32 = 1, EPI_RESID = 2, EPI_SWIGLU = 3, EPI_QKV = 4 };

struct GemvArgs {
    const uint8_t* w[3];      // matrices: [0] generic / gate / q, [1] up / k, [2] v
    const __half* s[3];       // their group scales (null for fp16 weights)
    const __half* x;          // input vector [K]
    const __half* norm_w;     // non-null: x is RMS-normalised with this weight in the prologue
    float eps;
    int K;                    // input columns, multiple of 128
    int rows;                 // output rows of one matrix (QKV: unused)
    int nsets;                // number of 16-row tile sets
    int ksplit;               // 1: CTA per tile set, K split over its warps; 0: warp per tile set
    __half* out_h;            // EPI_F16 / EPI_RESID (in-out) / EPI_SWIGLU
    float* out_f;             // EPI_F32
    // EPI_QKV
    const __half* bias[3];
    __half *q_out, *k_out, *v_out;
    __half *kcache, *vcache;  // this layer's [n_kv][max_seq][hd] caches, may be null
    const int* d_pos;
    int n_heads, n_kv, hd, max_seq;
    float theta;
    int rope_fast;
};

template <int Q> struct QT;
template <> struct QT<Q_I4> { static constexpr int NI = 1, GB = 64;  static constexpr float OFF = 72.f; };
template <> struct QT<Q_I8> { static constexpr int NI = 2, GB = 128; static constexpr float OFF = 1152.f; };
template <> struct QT<Q_F16> { static constexpr int NI = 4, GB = 256; static constexpr float OFF = 0.f; };

template <int Q, int MT> struct Depth { static constexpr int D = Q == Q_I4 ? 4 : Q == Q_I8 ? (MT == 2 ? 2 : 3) : (MT == 2 ? 1 : 2); };

template <int Q, int MT>
struct Stage {
    uint4 w[MT][2][QT<Q>::NI];
    uint16_t s[MT][2];
};

template <int Q, int MT>
struct TileSet {
    const uint8_t* rp[MT][2];   // row g and row g+8 of each tile
    const __half* sp[MT][2];    // their scale rows
};

template <int Q, int MT>
__device__ __forceinline__ void load_stage(Stage<Q, MT>& st, const TileSet<Q, MT>& ts, int grp, int t) {
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < QT<Q>::NI; ++i)
                st.w[m][h][i] = ldg_stream(ts.rp[m][h] + (size_t)grp * QT<Q>::GB + (i * 4 + t) * 16);
            if (Q != Q_F16) st.s[m][h] = ldg_u16(ts.sp[m][h] + grp);
        }
}

__device__ __forceinline__ uint32_t dq4(uint32_t v) { return and_xor(v, 0x00f000f0u, 0x54805480u); }

// One 128-column group for all MT tiles of the warp.
template <int Q, int MT>
__device__ __forceinline__ void compute_stage(const Stage<Q, MT>& st, float (&c)[MT][4], float (&tot)[MT][2],
                                              const uint4* __restrict__ xg, float corr, int t) {
    if (Q == Q_I4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 xv = xg[j * 4 + t];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                uint32_t a = u4c(st.w[m][0][0], j), b = u4c(st.w[m][1][0], j);
                mma16816(c[m], dq4(a << 4), dq4(b << 4), dq4(a), dq4(b), xv.x, xv.y);
                mma16816(c[m], dq4(a >> 4), dq4(b >> 4), dq4(a >> 8), dq4(b >> 8), xv.z, xv.w);
            }
        }
    } else if (Q == Q_I8) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                uint4 xv = xg[(i * 2 + jj) * 4 + t];
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    uint32_t a0 = u4c(st.w[m][0][i], 2 * jj) ^ 0x80808080u, b0 = u4c(st.w[m][1][i], 2 * jj) ^ 0x80808080u;
                    uint32_t a1 = u4c(st.w[m][0][i], 2 * jj + 1) ^ 0x80808080u, b1 = u4c(st.w[m][1][i], 2 * jj + 1) ^ 0x80808080u;
                    const uint32_t M = 0x64646464u;
                    mma16816(c[m], prmt(a0, M, 0x4140), prmt(b0, M, 0x4140), prmt(a0, M, 0x4342), prmt(b0, M, 0x4342), xv.x, xv.y);
                    mma16816(c[m], prmt(a1, M, 0x4140), prmt(b1, M, 0x4140), prmt(a1, M, 0x4342), prmt(b1, M, 0x4342), xv.z, xv.w);
                }
            }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 xv = xg[i * 4 + t];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint4& a = st.w[m][0][i];
                const uint4& b = st.w[m][1][i];
                mma16816(c[m], a.x, b.x, a.y, b.y, xv.x, xv.y);
                mma16816(c[m], a.z, b.z, a.w, b.w, xv.z, xv.w);
            }
        }
    }
    if (Q != Q_F16) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float s0 = __half2float(__ushort_as_half(st.s[m][0])), s1 = __half2float(__ushort_as_half(st.s[m][1]));
            tot[m][0] = fmaf(c[m][0] - corr, s0, tot[m][0]);
            tot[m][1] = fmaf(c[m][2] - corr, s1, tot[m][1]);
            c[m][0] = c[m][1] = c[m][2] = c[m][3] = 0.f;
        }
    }
}

// Stage the activation vector into shared memory in the order the B operand
// wants, optionally RMS-normalising it first (reference src/kernels.cu:689-751:
// out = half(float(x) * inv_rms * float(w))), and compute the per-group offset
// corrections.
template <int Q>
__device__ __forceinline__ void stage_x(const GemvArgs& a, uint4* xs, float* corr, float* red) {
    const int nchunk = a.K / 8;
    float inv = 0.f;
    if (a.norm_w) inv = block_inv_rms(a.x, a.K, a.eps, red);
    const uint4* xg = reinterpret_cast<const uint4*>(a.x);
    const uint4* wg = reinterpret_cast<const uint4*>(a.norm_w);
    for (int c8 = threadIdx.x; c8 < nchunk; c8 += blockDim.x) {
        uint4 v = xg[c8];
        if (a.norm_w) {
            uint4 wv = wg[c8];
            __half2* xh = reinterpret_cast<__half2*>(&v);
            const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 xf = __half22float2(xh[k]), wf = __half22float2(wh[k]);
                xh[k] = __floats2half2_rn(xf.x * inv * wf.x, xf.y * inv * wf.y);
            }
        }
        int grp = c8 >> 4, r = c8 & 15, dst;
        if (Q == Q_I4) {
            int t = r >> 2, j = r & 3;
            dst = grp * 16 + j * 4 + t;
            uint4 p;
            p.x = prmt(v.x, v.z, 0x5410); p.y = prmt(v.x, v.z, 0x7632);
            p.z = prmt(v.y, v.w, 0x5410); p.w = prmt(v.y, v.w, 0x7632);
            v = p;
        } else if (Q == Q_I8) {
            int i = r >> 3, t = (r >> 1) & 3, jj = r & 1;
            dst = grp * 16 + (i * 2 + jj) * 4 + t;
        } else {
            dst = c8;
        }
        xs[dst] = v;
    }
    __syncthreads();
    if (Q != Q_F16) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
        const uint2* x2 = reinterpret_cast<const uint2*>(xs);
        for (int g = warp; g < a.K / kGroup; g += nw) {
            uint2 v = x2[g * 32 + lane];
            float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&v.x)), f1 = __half22float2(*reinterpret_cast<__half2*>(&v.y));
            float sum = warp_sum((f0.x + f0.y) + (f1.x + f1.y));
            if (lane == 0) corr[g] = QT<Q>::OFF * sum;
        }
        __syncthreads();
    }
}

template <int EPI> struct EpiMT { static constexpr int MT = (EPI == EPI_SWIGLU || EPI == EPI_QKV) ? 2 : 1; };

// Row addressing of tile set `ts`.  Returns the first output row (generic) in
// *row0; QKV returns the row inside the virtual [q|k|v] concatenation.
template <int Q, int EPI>
__device__ __forceinline__ void map_tileset(const GemvArgs& a, int ts, int g, TileSet<Q, EpiMT<EPI>::MT>& out, int* row0, int* mat) {
    constexpr int MT = EpiMT<EPI>::MT;
    const size_t rb = Q == Q_I4 ? a.K / 2 : Q == Q_I8 ? a.K : (size_t)a.K * 2;
    const int ng = a.K / kGroup;
    if (EPI == EPI_QKV) {
        const int spt = a.hd / 32;              // tile sets per head
        int hh = ts / spt, sub = ts % spt;
        int m = hh < a.n_heads ? 0 : hh < a.n_heads + a.n_kv ? 1 : 2;
        int lh = m == 0 ? hh : m == 1 ? hh - a.n_heads : hh - a.n_heads - a.n_kv;
        int r = lh * a.hd + sub * 16;
        *row0 = r; *mat = m;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                size_t row = (size_t)r + mt * (a.hd / 2) + g + 8 * h;
                out.rp[mt][h] = a.w[m] + row * rb;
                out.sp[mt][h] = a.s[m] ? a.s[m] + row * ng : nullptr;
            }
    } else {
        *row0 = ts * 16; *mat = 0;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int row = ts * 16 + g + 8 * h;
                row = row < a.rows ? row : a.rows - 1;     // ragged last tile: read a valid row, never store it
                out.rp[mt][h] = a.w[mt] + (size_t)row * rb;
                out.sp[mt][h] = a.s[mt] ? a.s[mt] + (size_t)row * ng : nullptr;
            }
    }
}

// Finish one output row (pair).  r = row slot 0..15 inside the tile set.
template <int EPI>
__device__ __forceinline__ void epilogue(const GemvArgs& a, int row0, int mat, int r, float v0, float v1) {
    if (EPI == EPI_F16) {
        int row = row0 + r;
        if (row < a.rows) a.out_h[row] = __float2half(v0);
    } else if (EPI == EPI_F32) {
        int row = row0 + r;
        if (row < a.rows) a.out_f[row] = v0;
    } else if (EPI == EPI_RESID) {
        // reference src/kernels.cu:670-671 and :620-621
        int row = row0 + r;
        if (row < a.rows) a.out_h[row] = __float2half(__half2float(a.out_h[row]) + v0);
    } else if (EPI == EPI_SWIGLU) {
        // reference src/kernels.cu:565-567 (fast-math exp and divide, as that build uses)
        int row = row0 + r;
        if (row < a.rows) {
            float sig = __fdividef(1.0f, 1.0f + __expf(-v0));
            a.out_h[row] = __float2half(v0 * sig * v1);
        }
    } else {
        // bias in fp32, one rounding to fp16 (src/kernels.cu:468-472); rotate-half RoPE on q and k
        // from the rounded values (src/kernels.cu:370-398); k and v also go to the cache row `pos`
        // (src/kernels.cu:326-347).
        const int half_hd = a.hd / 2;
        int ra = row0 + r, rb2 = ra + half_hd;
        const __half* bias = a.bias[mat];
        float f0 = __half2float(__float2half(v0 + __half2float(bias[ra])));
        float f1 = __half2float(__float2half(v1 + __half2float(bias[rb2])));
        __half o0, o1;
        const int pos = *a.d_pos;
        if (mat < 2) {
            float c, s;
            rope_cs(ra % a.hd, a.hd, pos, a.theta, a.rope_fast, &c, &s);
            o0 = __float2half(f0 * c - f1 * s);
            o1 = __float2half(f1 * c + f0 * s);
        } else {
            o0 = __float2half(f0); o1 = __float2half(f1);
        }
        __half* dst = mat == 0 ? a.q_out : mat == 1 ? a.k_out : a.v_out;
        if (dst) { dst[ra] = o0; dst[rb2] = o1; }
        __half* cache = mat == 1 ? a.kcache : mat == 2 ? a.vcache : nullptr;
        if (cache) {
            int head = ra / a.hd, d = ra % a.hd;
            size_t base = ((size_t)head * a.max_seq + pos) * a.hd;
            cache[base + d] = o0; cache[base + d + half_hd] = o1;
        }
    }
}

template <int Q, int EPI>
__global__ void __launch_bounds__(256, 2) gemv_kernel(const GemvArgs a) {
    constexpr int MT = EpiMT<EPI>::MT;
    constexpr int D = Depth<Q, MT>::D;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint4* xs = reinterpret_cast<uint4*>(smem_raw);
    float* corr = reinterpret_cast<float*>(smem_raw + (size_t)a.K * 2);
    float* red = corr + a.K / kGroup;                 // 8 warps x 32 row slots, also norm scratch (>= 33)
    int* next_ts = reinterpret_cast<int*>(red + 8 * 32);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ngrp = a.K / kGroup;

    // Work range.  ksplit: CTA b owns tile sets b, b+grid, ...  Otherwise CTA b owns a contiguous
    // share [lo,hi) of the tile sets and its warps pull from it (first one statically).
    int lo, hi;
    if (a.ksplit) { lo = blockIdx.x; hi = a.nsets; }
    else {
        lo = (int)((long long)a.nsets * blockIdx.x / gridDim.x);
        hi = (int)((long long)a.nsets * (blockIdx.x + 1) / gridDim.x);
    }
    int ts = a.ksplit ? lo : lo + warp;
    const int g0 = a.ksplit ? warp : 0, gstep = a.ksplit ? nw : 1;
    const int my_n = g0 < ngrp ? (ngrp - g0 + gstep - 1) / gstep : 0;

    TileSet<Q, MT> tsp;
    Stage<Q, MT> st[D];
    int row0 = 0, mat = 0;
    bool have = ts < hi;
    if (have) {
        map_tileset<Q, EPI>(a, ts, g, tsp, &row0, &mat);
#pragma unroll
        for (int d = 0; d < D; ++d)
            if (d < my_n) load_stage<Q, MT>(st[d], tsp, g0 + d * gstep, t);
    }
    if (threadIdx.x == 0) *next_ts = lo + nw;

    pdl_wait();                 // everything above reads only weights
    pdl_launch_dependents();
    stage_x<Q>(a, xs, corr, red);

    while (true) {
        if (!a.ksplit && !have) break;
        if (a.ksplit && ts >= hi) break;
        float c[MT][4], tot[MT][2];
#pragma unroll
        for (int m = 0; m < MT; ++m) { c[m][0] = c[m][1] = c[m][2] = c[m][3] = 0.f; tot[m][0] = tot[m][1] = 0.f; }
        if (have) {
            for (int it = 0; it < my_n; it += D) {
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    if (it + d < my_n) {
                        int grp = g0 + (it + d) * gstep;
                        compute_stage<Q, MT>(st[d], c, tot, xs + grp * 16, Q != Q_F16 ? corr[grp] : 0.f, t);
                        if (it + d + D < my_n) load_stage<Q, MT>(st[d], tsp, g0 + (it + d + D) * gstep, t);
                    }
                }
            }
            if (Q == Q_F16) {
#pragma unroll
                for (int m = 0; m < MT; ++m) { tot[m][0] = c[m][0]; tot[m][1] = c[m][2]; }
            }
        }
        const int cur_row0 = row0, cur_mat = mat;
        if (a.ksplit) {
            if (t == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) { red[warp * 32 + m * 16 + g] = tot[m][0]; red[warp * 32 + m * 16 + g + 8] = tot[m][1]; }
            }
            // start the next tile set's loads before the reduction
            ts += gridDim.x;
            have = ts < hi;
            if (have) {
                map_tileset<Q, EPI>(a, ts, g, tsp, &row0, &mat);
#pragma unroll
                for (int d = 0; d < D; ++d)
                    if (d < my_n) load_stage<Q, MT>(st[d], tsp, g0 + d * gstep, t);
            }
            __syncthreads();
            if (threadIdx.x < 16) {
                float v0 = 0.f, v1 = 0.f;
                for (int w = 0; w < nw; ++w) { v0 += red[w * 32 + threadIdx.x]; if (MT == 2) v1 += red[w * 32 + 16 + threadIdx.x]; }
                epilogue<EPI>(a, cur_row0, cur_mat, threadIdx.x, v0, v1);
            }
            __syncthreads();
        } else {
            if (t == 0) {
                epilogue<EPI>(a, cur_row0, cur_mat, g, tot[0][0], MT == 2 ? tot[MT - 1][0] : 0.f);
                epilogue<EPI>(a, cur_row0, cur_mat, g + 8, tot[0][1], MT == 2 ? tot[MT - 1][1] : 0.f);
            }
            int nxt = 0;
            if (lane == 0) nxt = atomicAdd(next_ts, 1);
            ts = __shfl_sync(0xffffffffu, nxt, 0);
            have = ts < hi;
            if (have) {
                map_tileset<Q, EPI>(a, ts, g, tsp, &row0, &mat);
#pragma unroll
                for (int d = 0; d < D; ++d)
                    if (d < my_n) load_stage<Q, MT>(st[d], tsp, g0 + d * gstep, t);
            }
        }
    }
}

// Shared-memory bytes the kernel needs for input length K.
inline size_t gemv_smem_bytes(int K) { return (size_t)K * 2 + (size_t)(K / kGroup) * 4 + 8 * 32 * 4 + 16; }

}  // namespace cq
