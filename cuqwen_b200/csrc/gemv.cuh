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
// Data path.  Every warp owns 16 output rows (x MT matrices) at a time and a
// private ring of shared-memory stages.  One lane issues a 2-D TMA tile copy
// (cp.async.bulk.tensor.2d: a box of 16 rows x up to 256 bytes of the row-major
// weight matrix, no cluster broadcast) per stage; the box lands in the ring and
// signals an mbarrier, so the HBM stream is decoupled from the register file
// and from the scoreboards: tens of KB per SM stay in flight while the warp
// computes.  Rows past the end of the matrix are zero-filled by the TMA unit.  Lane 4g+t then reads 16 bytes per
// row-group of rows g and g+8 from the stage, turns the integers into fp16 with
// a magic-exponent trick (two weights per LOP3/PRMT, no int->float converts) and
// feeds them as the A operand of mma.sync.m16n8k16; the activation vector sits
// in shared memory, pre-permuted so one LDS.128 yields the B operand of two MMA
// steps.  The fp16 magic adds a constant offset (72 for int4, 1152 for int8) to
// every weight; it is removed per group with offset * sum(x over the group),
// computed once per CTA.
//
// Every wait on an mbarrier is bounded (about two seconds of wall time); when
// it expires the kernel records a code in *err, stops waiting and finishes with
// meaningless numbers rather than hanging.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace cq {

enum Epi : int { EPI_F16 = 0, EPI_F32 = 1, EPI_RESID = 2, EPI_SWIGLU = 3, EPI_QKV = 4 };

struct alignas(64) GemvArgs {
    CUtensorMap tmap[3];      // one 2-D byte map per weight matrix: dims {row bytes, rows}, box {piece bytes, 16}
    const uint8_t* w[3];      // matrices: [0] generic / gate / q, [1] up / k, [2] v
    const __half* s[3];       // their group scales (null for fp16 weights)
    const __half* x;          // input vector [K]
    const __half* norm_w;     // non-null: x is RMS-normalised with this weight in the prologue
    float eps;
    int K;                    // input columns, multiple of 128
    int rows;                 // output rows of one matrix (QKV: unused)
    int nsets;                // number of 16-row tile sets
    int ksplit;               // 1: CTA per tile set, K split over its warps; 0: warp per tile set
    int pg;                   // 128-column groups per staged row piece
    int nst;                  // stages in each warp's ring
    unsigned* err;            // device word that receives a non-zero code when a bounded wait expires (may be null)
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

template <int EPI> struct EpiMT { static constexpr int MT = (EPI == EPI_SWIGLU || EPI == EPI_QKV) ? 2 : 1; };

// Shared-memory carve-up, computed the same way by the host (for the launch size) and the kernel.
struct GemvLayout {
    int piece_bytes, row_stride, stage_bytes, scale_tile_bytes;
    int off_corr, off_red, off_scales, off_stages, off_bars, total;
};
__host__ __device__ inline GemvLayout gemv_layout(int K, int group_bytes, int MT, int nw, int pg, int nst, int ksplit, bool quantised) {
    GemvLayout L;
    const int ng = K / kGroup;
    L.piece_bytes = pg * group_bytes;
    L.row_stride = L.piece_bytes;            // a TMA box is dense: [16 rows][piece bytes]
    L.stage_bytes = MT * 16 * L.row_stride;
    L.scale_tile_bytes = quantised ? MT * 16 * ng * 2 : 0;
    int o = K * 2;
    L.off_corr = o; o += (ng * 4 + 15) / 16 * 16;
    L.off_red = o; o += 8 * 32 * 4 + 16;
    o = (o + 127) / 128 * 128;
    L.off_scales = o; o += (ksplit ? 1 : nw) * 2 * L.scale_tile_bytes;
    o = (o + 127) / 128 * 128;               // TMA destinations are 128-byte aligned
    L.off_stages = o; o += nw * nst * L.stage_bytes;
    L.off_bars = o; o += nw * (nst + 2) * 8;
    L.total = o;
    return L;
}

// ---- async copy / mbarrier primitives -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
// Bounded wait: false when the phase did not complete within ~2 s.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > 2000000000ull) return false;
    }
}
// global -> shared bulk copy; completion is signalled on `bar` with the byte count.  dst, src and bytes are multiples of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 2-D tile copy: box of the tensor map at byte column x, row y.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_h(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}

__device__ __forceinline__ uint32_t dq4(uint32_t v) { return and_xor(v, 0x00f000f0u, 0x54805480u); }

// One 128-column group of all MT tiles: weights from the stage (wbase = this lane's row g of tile 0 at this group),
// x from xg, two alternating accumulator sets to halve the dependent-MMA chain.
template <int Q, int MT>
__device__ __forceinline__ void compute_group(uint32_t wbase, int row_stride, int t, const uint4* __restrict__ xg, float (&c)[MT][2][4]) {
    constexpr int NI = QT<Q>::NI;
    uint4 w[MT][2][NI];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < NI; ++i) w[m][h][i] = lds128(wbase + (m * 16 + h * 8) * row_stride + (i * 4 + t) * 16);
    if (Q == Q_I4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 xv = xg[j * 4 + t];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                uint32_t a = u4c(w[m][0][0], j), b = u4c(w[m][1][0], j);
                mma16816(c[m][0], dq4(a << 4), dq4(b << 4), dq4(a), dq4(b), xv.x, xv.y);
                mma16816(c[m][1], dq4(a >> 4), dq4(b >> 4), dq4(a >> 8), dq4(b >> 8), xv.z, xv.w);
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
                    uint32_t a0 = u4c(w[m][0][i], 2 * jj) ^ 0x80808080u, b0 = u4c(w[m][1][i], 2 * jj) ^ 0x80808080u;
                    uint32_t a1 = u4c(w[m][0][i], 2 * jj + 1) ^ 0x80808080u, b1 = u4c(w[m][1][i], 2 * jj + 1) ^ 0x80808080u;
                    const uint32_t M = 0x64646464u;
                    mma16816(c[m][0], prmt(a0, M, 0x4140), prmt(b0, M, 0x4140), prmt(a0, M, 0x4342), prmt(b0, M, 0x4342), xv.x, xv.y);
                    mma16816(c[m][1], prmt(a1, M, 0x4140), prmt(b1, M, 0x4140), prmt(a1, M, 0x4342), prmt(b1, M, 0x4342), xv.z, xv.w);
                }
            }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 xv = xg[i * 4 + t];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint4& a = w[m][0][i];
                const uint4& b = w[m][1][i];
                mma16816(c[m][0], a.x, b.x, a.y, b.y, xv.x, xv.y);
                mma16816(c[m][1], a.z, b.z, a.w, b.w, xv.z, xv.w);
            }
        }
    }
}

// Stage the activation vector into shared memory in the order the B operand wants, optionally RMS-normalising it
// first (reference src/kernels.cu:689-751: out = half(float(x) * inv_rms * float(w))), and compute the per-group
// offset corrections.
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

// Where the 16 x MT rows of tile set `ts` live.  base[m] / sbase[m]: first row of tile m; row0: first output row
// (generic) or the row inside its q / k / v matrix (QKV); valid: rows of the tile that exist.
template <int Q, int EPI>
struct TileMap {
    int mrow[EpiMT<EPI>::MT];            // first row of tile m inside its matrix
    int mmat[EpiMT<EPI>::MT];            // index of that matrix in GemvArgs::w / tmap
    const __half* sbase[EpiMT<EPI>::MT];
    int row0, mat, valid;
};
template <int Q, int EPI>
__device__ __forceinline__ TileMap<Q, EPI> map_tileset(const GemvArgs& a, int ts) {
    constexpr int MT = EpiMT<EPI>::MT;
    const int ng = a.K / kGroup;
    TileMap<Q, EPI> m;
    if (EPI == EPI_QKV) {
        const int spt = a.hd / 32;              // tile sets per head
        int hh = ts / spt, sub = ts % spt;
        int mat = hh < a.n_heads ? 0 : hh < a.n_heads + a.n_kv ? 1 : 2;
        int lh = mat == 0 ? hh : mat == 1 ? hh - a.n_heads : hh - a.n_heads - a.n_kv;
        m.row0 = lh * a.hd + sub * 16; m.mat = mat; m.valid = 16;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            size_t row = (size_t)m.row0 + mt * (a.hd / 2);
            m.mrow[mt] = (int)row; m.mmat[mt] = mat;
            m.sbase[mt] = a.s[mat] ? a.s[mat] + row * ng : nullptr;
        }
    } else {
        m.row0 = ts * 16; m.mat = 0;
        m.valid = a.rows - m.row0 < 16 ? a.rows - m.row0 : 16;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            m.mrow[mt] = m.row0; m.mmat[mt] = mt;
            m.sbase[mt] = a.s[mt] ? a.s[mt] + (size_t)m.row0 * ng : nullptr;
        }
    }
    return m;
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
__global__ void __launch_bounds__(256, 1) gemv_kernel(const __grid_constant__ GemvArgs a) {
    constexpr int MT = EpiMT<EPI>::MT;
    constexpr int GB = QT<Q>::GB;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    pdl_launch_dependents();    // let the next kernel's CTAs become resident and prefetch their weights while this one runs
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ngrp = a.K / kGroup, nst = a.nst, pg = a.pg;
    const GemvLayout L = gemv_layout(a.K, GB, MT, nw, pg, nst, a.ksplit, Q != Q_F16);
    uint4* xs = reinterpret_cast<uint4*>(smem_raw);
    float* corr = reinterpret_cast<float*>(smem_raw + L.off_corr);
    float* red = reinterpret_cast<float*>(smem_raw + L.off_red);
    const uint32_t sm0 = smem_u32(smem_raw);
    const uint32_t my_stages = sm0 + L.off_stages + warp * nst * L.stage_bytes;
    const uint32_t my_bars = sm0 + L.off_bars + warp * (nst + 2) * 8;          // nst stage barriers, then 2 scale barriers
    const int sowner = a.ksplit ? 0 : warp;                                      // warp whose scale buffers this warp reads
    const uint32_t sc_bufs = sm0 + L.off_scales + sowner * 2 * L.scale_tile_bytes;
    const uint32_t sc_bars = sm0 + L.off_bars + sowner * (nst + 2) * 8 + nst * 8;

    if (lane == 0) {
        for (int s = 0; s < nst + 2; ++s) mbar_init(my_bars + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // ---- this warp's work: n_ts tile sets, P row pieces of each ----
    const int rb = Q == Q_I4 ? a.K / 2 : Q == Q_I8 ? a.K : a.K * 2;            // bytes of one weight row
    const int PT = (rb + L.piece_bytes - 1) / L.piece_bytes;                   // pieces in a full row
    int ts0, ts_step, n_ts, c0, c_step, P;
    if (a.ksplit) {
        ts0 = blockIdx.x; ts_step = gridDim.x;
        n_ts = ts0 < a.nsets ? (a.nsets - ts0 + ts_step - 1) / ts_step : 0;
        c0 = warp; c_step = nw; P = warp < PT ? (PT - warp + nw - 1) / nw : 0;
    } else {
        const int lo = (int)((long long)a.nsets * blockIdx.x / gridDim.x), hi = (int)((long long)a.nsets * (blockIdx.x + 1) / gridDim.x);
        ts0 = lo + warp; ts_step = nw;
        n_ts = ts0 < hi ? (hi - ts0 + nw - 1) / nw : 0;
        c0 = 0; c_step = 1; P = PT;
    }
    const int T = n_ts * P;
    const bool scale_issuer = Q != Q_F16 && (a.ksplit ? warp == 0 : true);

    // issue item i = (tile set i / P, piece i % P) into stage i % nst
    auto issue = [&](int i) {
        const int j = i / P, p = i - j * P;
        const TileMap<Q, EPI> tm = map_tileset<Q, EPI>(a, ts0 + j * ts_step);
        const int c = c0 + p * c_step;
        const uint32_t bar = my_bars + (i % nst) * 8;
        const uint32_t dst = my_stages + (i % nst) * L.stage_bytes;
        if (lane == 0) {
            mbar_expect_tx(bar, (uint32_t)(L.stage_bytes));       // a box always delivers its full size (zero fill out of bounds)
#pragma unroll
            for (int m = 0; m < MT; ++m) tma_load_2d(dst + m * 16 * L.row_stride, &a.tmap[tm.mmat[m]], c * L.piece_bytes, tm.mrow[m], bar);
        }
    };
    auto issue_scales = [&](int j) {
        const TileMap<Q, EPI> tm = map_tileset<Q, EPI>(a, ts0 + j * ts_step);
        const uint32_t bar = my_bars + (nst + (j & 1)) * 8;
        const int boff = L.off_scales + warp * 2 * L.scale_tile_bytes + (j & 1) * L.scale_tile_bytes;
        const int tile_bytes = 16 * ngrp * 2;
        if (tm.valid == 16) {
            if (lane == 0) {
                mbar_expect_tx(bar, (uint32_t)(tile_bytes * MT));
#pragma unroll
                for (int m = 0; m < MT; ++m) bulk_g2s(sm0 + boff + m * tile_bytes, tm.sbase[m], tile_bytes, bar);
            }
        } else {
            // ragged last tile: its scale block is not a whole number of 16-byte units; copy it with plain loads
            __half* sb = reinterpret_cast<__half*>(smem_raw + boff);
            for (int idx = lane; idx < tm.valid * ngrp; idx += 32) sb[idx] = tm.sbase[0][idx];
            __syncwarp();
            if (lane == 0) mbar_expect_tx(bar, 0);
        }
        __syncwarp();
    };

    int issued = 0;          // items issued so far
    int sc_issued = 0;       // tile sets whose scales were issued
    // never run more than one tile set ahead of the consumer (the scale buffers are double-buffered), and never
    // more than nst items ahead
    auto pump = [&](int consumed, int j_cons) {
        if (scale_issuer) while (sc_issued < n_ts && sc_issued <= j_cons + 1) issue_scales(sc_issued++);
        if (P > 0) while (issued < T && issued < consumed + nst && issued / P <= j_cons + 1) issue(issued++);
    };
    pump(0, 0);

    pdl_wait();                 // everything above reads only weights
    stage_x<Q>(a, xs, corr, red);

    bool failed = false;
    int consumed = 0;
    for (int j = 0; j < n_ts; ++j) {
        const TileMap<Q, EPI> tm = map_tileset<Q, EPI>(a, ts0 + j * ts_step);
        float c[MT][2][4], tot[MT][2];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            tot[m][0] = tot[m][1] = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) c[m][0][q] = c[m][1][q] = 0.f;
        }
        uint32_t sbuf = 0;
        if (Q != Q_F16) {
            if (!failed && !mbar_wait(sc_bars + (j & 1) * 8, (j >> 1) & 1)) { failed = true; if (a.err) atomicExch(a.err, 2u); }
            sbuf = sc_bufs + (j & 1) * L.scale_tile_bytes;
        }
        for (int p = 0; p < P; ++p) {
            const int i = consumed;
            if (!failed && !mbar_wait(my_bars + (i % nst) * 8, (i / nst) & 1)) { failed = true; if (a.err) atomicExch(a.err, 1u); }
            const int cidx = c0 + p * c_step;
            const int grp0 = cidx * pg;
            const int ngp = ngrp - grp0 < pg ? ngrp - grp0 : pg;
            const uint32_t wrow = my_stages + (i % nst) * L.stage_bytes + g * L.row_stride;
            for (int gi = 0; gi < ngp; ++gi) {
                const int grp = grp0 + gi;
                compute_group<Q, MT>(wrow + gi * GB, L.row_stride, t, xs + grp * 16, c);
                if (Q != Q_F16) {
                    const float cr = corr[grp];
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float s0 = lds_h(sbuf + ((m * 16 + g) * ngrp + grp) * 2), s1 = lds_h(sbuf + ((m * 16 + g + 8) * ngrp + grp) * 2);
                        tot[m][0] = fmaf((c[m][0][0] + c[m][1][0]) - cr, s0, tot[m][0]);
                        tot[m][1] = fmaf((c[m][0][2] + c[m][1][2]) - cr, s1, tot[m][1]);
#pragma unroll
                        for (int q = 0; q < 4; ++q) c[m][0][q] = c[m][1][q] = 0.f;
                    }
                }
            }
            __syncwarp();
            fence_async_smem();        // the stage was read through the generic proxy; the refill writes through the async proxy
            ++consumed;
            pump(consumed, j);
        }
        if (Q == Q_F16) {
#pragma unroll
            for (int m = 0; m < MT; ++m) { tot[m][0] = c[m][0][0] + c[m][1][0]; tot[m][1] = c[m][0][2] + c[m][1][2]; }
        }
        if (a.ksplit) {
            if (t == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) { red[warp * 32 + m * 16 + g] = tot[m][0]; red[warp * 32 + m * 16 + g + 8] = tot[m][1]; }
            }
            __syncthreads();
            if (threadIdx.x < 16) {
                float v0 = 0.f, v1 = 0.f;
                for (int w = 0; w < nw; ++w) { v0 += red[w * 32 + threadIdx.x]; if (MT == 2) v1 += red[w * 32 + 16 + threadIdx.x]; }
                epilogue<EPI>(a, tm.row0, tm.mat, threadIdx.x, v0, v1);
            }
            __syncthreads();           // `red` and the scale buffer of tile set j are free again
        } else if (t == 0) {
            epilogue<EPI>(a, tm.row0, tm.mat, g, tot[0][0], MT == 2 ? tot[MT - 1][0] : 0.f);
            epilogue<EPI>(a, tm.row0, tm.mat, g + 8, tot[0][1], MT == 2 ? tot[MT - 1][1] : 0.f);
        }
        if (j + 1 < n_ts) pump(consumed, j + 1);
    }
    if (failed) {
        // give copies that may still be in flight a last bounded chance to land before the CTA's shared memory goes away
        for (int i = consumed; i < issued; ++i) mbar_wait(my_bars + (i % nst) * 8, (i / nst) & 1);
    }
}

// Shared-memory bytes the kernel needs.
inline size_t gemv_smem_bytes(int K, int quant, int MT, int nw, int pg, int nst, int ksplit) {
    const int gb = quant == Q_I4 ? 64 : quant == Q_I8 ? 128 : 256;
    return (size_t)gemv_layout(K, gb, MT, nw, pg, nst, ksplit, quant != Q_F16).total;
}

}  // namespace cq
