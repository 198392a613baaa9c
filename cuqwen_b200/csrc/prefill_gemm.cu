// The batched-token GEMM kernel and its launcher (see prefill_gemm.cuh for the design).
#include "prefill_gemm.cuh"
#include "tcgen05.cuh"

#include <mutex>
#include <vector>

namespace cq {

// Shared-memory matrix descriptor of a K-major tile in the 128-byte-swizzled canonical layout: rows of 128 bytes,
// eight-row groups 1024 bytes apart.  Fields: start address >> 4 [0,14), leading byte offset >> 4 [16,30) (unused by
// swizzled K-major tiles), stride byte offset >> 4 [32,46), descriptor version 1 [46,48), layout type 2 = 128-byte
// swizzle [61,64).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// W weights (32 or 16: one half or one quarter of a row's K block) -> W / 8 sixteen-byte chunks of fp16(q * scale),
// stored at the row's swizzled places.  raw: shared address of the part's bytes; brow: the row in the B tile; chunk0:
// the part's first chunk.
template <int Q, int W>
__device__ __forceinline__ void convert_part(uint32_t raw, uint32_t brow, int sw, int chunk0, __half2 sc2) {
    if (Q == Q_I4) {
        // two's-complement nibbles, element 2p in the low nibble of byte p: (n ^ 8) | 0x6400 is fp16(1024 + q + 8)
        const __half2 off = __floats2half2_rn(1032.f, 1032.f);
        uint32_t w4[4];
        if (W == 32) { const uint4 rw = lds128(raw); w4[0] = rw.x; w4[1] = rw.y; w4[2] = rw.z; w4[3] = rw.w; }
        else { asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w4[0]), "=r"(w4[1]) : "r"(raw)); w4[2] = w4[3] = 0u; }
#pragma unroll
        for (int i = 0; i < W / 8; ++i) {
            const uint32_t w = w4[i];
            uint32_t t[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t u = ((w >> (4 * j)) & 0x000f000fu) ^ 0x64086408u;          // (element j, element j + 4)
                const __half2 hv = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&u), off), sc2);
                t[j] = *reinterpret_cast<const uint32_t*>(&hv);
            }
            uint4 o;
            o.x = __byte_perm(t[0], t[1], 0x5410); o.y = __byte_perm(t[2], t[3], 0x5410);
            o.z = __byte_perm(t[0], t[1], 0x7632); o.w = __byte_perm(t[2], t[3], 0x7632);
            sts128(brow + (((chunk0 + i) ^ sw) << 4), o);
        }
    } else {
        // signed bytes: (b ^ 0x80) under a 0x64 exponent byte is fp16(1024 + b + 128)
        const __half2 off = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
        for (int h = 0; h < W / 16; ++h) {
            const uint4 rw = lds128(raw + h * 16);
            const uint32_t w4[4] = {rw.x, rw.y, rw.z, rw.w};
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                uint32_t t[4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t x = w4[2 * i + j] ^ 0x80808080u;
                    const uint32_t lo = __byte_perm(x, 0x64646464u, 0x4140), hi = __byte_perm(x, 0x64646464u, 0x4342);
                    const __half2 a = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&lo), off), sc2);
                    const __half2 b = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&hi), off), sc2);
                    t[2 * j] = *reinterpret_cast<const uint32_t*>(&a); t[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&b);
                }
                sts128(brow + (((chunk0 + h * 2 + i) ^ sw) << 4), make_uint4(t[0], t[1], t[2], t[3]));
            }
        }
    }
}

template <int Q, int NT>
__global__ void __launch_bounds__(kPfThreads, 1) prefill_gemm_kernel(const __grid_constant__ PfGemmArgs a) {
    extern __shared__ unsigned char pf_smem_raw[];
    const uint32_t base = (smem_u32(pf_smem_raw) + 1023u) & ~1023u;
    constexpr int NA = pf_na(Q), NB = pf_nb(Q), kRawBytes = pf_raw_bytes(Q, NT), kPfBBytes = NT * 128;
    constexpr uint32_t kPfIdesc = umma_idesc_f16(kPfM, NT, 0);
    constexpr int kASlot = kPfMH * kPfABytes;                  // X tiles of one slot
    const uint32_t ring_a = base, ring_raw = ring_a + NA * kASlot, ring_b = ring_raw + NA * kRawBytes;
    const uint32_t bars = ring_b + NB * kPfBBytes;
    const uint32_t bar_full = bars, bar_afree = bar_full + 8 * NA, bar_conv = bar_afree + 8 * NA, bar_bfree = bar_conv + 8 * NB, bar_done = bar_bfree + 8 * NB;
    const uint32_t tmem_slot = bar_done + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tm = blockIdx.x, tn = blockIdx.y, mh = a.mh;
    const bool swiglu = a.mode == PF_SWIGLU;
    const int rows_mat = swiglu ? NT / 2 : NT;                // rows of each matrix in this tile
    const int nmat = swiglu ? 2 : 1;
    int seg = 0, coff = 0, tseg = tn;                         // plain modes: which matrix this row tile belongs to, its first output column
    if (!swiglu)
        while (seg + 1 < a.nseg && tseg >= (a.seg_rows[seg] + NT - 1) / NT) { tseg -= (a.seg_rows[seg] + NT - 1) / NT; coff += a.seg_rows[seg]; ++seg; }
    const int row0 = tseg * rows_mat;                         // first row inside the matrix
    const int R = a.seg_rows[seg];
    const int nkb = a.K / kPfKB;
    constexpr int kRawKb = Q == Q_I4 ? 32 : 64;               // raw bytes of one row in one K block
    bool failed = false;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NA; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_afree + 8 * s, 1); }
        for (int s = 0; s < NB; ++s) { mbar_init(bar_conv + 8 * s, kPfConvWarps); mbar_init(bar_bfree + 8 * s, 1); }
        mbar_init(bar_done, 1);
        mbar_fence_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, (uint32_t)(mh * NT)); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = lds32(tmem_slot);

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t wbytes = Q == Q_F16 ? (uint32_t)kPfBBytes : (uint32_t)(NT * kRawKb);
            for (int kb = 0; kb < nkb && !failed; ++kb) {
                const int sa = kb % NA, sb = kb % NB; const uint32_t pa = (uint32_t)(kb / NA) & 1u;
                if (!mbar_wait(bar_afree + 8 * sa, pa ^ 1u)) { failed = true; break; }
                mbar_expect_tx(bar_full + 8 * sa, (uint32_t)(mh * kPfABytes) + wbytes);
                for (int h = 0; h < mh; ++h)        // a half that lies past the last token arrives as zeros
                    tma_load_2d(ring_a + sa * kASlot + h * kPfABytes, &a.tx, kb * kPfKB, (tm * mh + h) * kPfM, bar_full + 8 * sa);
                for (int m = 0; m < nmat; ++m) {
                    if (Q == Q_F16) tma_load_2d(ring_b + sb * kPfBBytes + m * rows_mat * 128, &a.tw[seg + m], kb * kPfKB, row0, bar_full + 8 * sa);    // NB == NA: freed together
                    else tma_load_2d(ring_raw + sa * kRawBytes + m * rows_mat * kRawKb, &a.tw[seg + m], kb * kRawKb, row0, bar_full + 8 * sa);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int kb = 0; kb < nkb && !failed; ++kb) {
                const int sa = kb % NA, sb = kb % NB; const uint32_t pa = (uint32_t)(kb / NA) & 1u, pb = (uint32_t)(kb / NB) & 1u;
                if (!mbar_wait(bar_full + 8 * sa, pa)) { failed = true; break; }
                if (Q != Q_F16 && !mbar_wait(bar_conv + 8 * sb, pb)) { failed = true; break; }
                tc_fence_after();
                const uint32_t at = ring_a + sa * kASlot, bt = ring_b + sb * kPfBBytes;
                for (int h = 0; h < mh; ++h)
#pragma unroll
                    for (int k4 = 0; k4 < kPfKB / 16; ++k4)
                        umma_f16(tmem + (uint32_t)(h * NT), umma_desc(at + h * kPfABytes + k4 * 32), umma_desc(bt + k4 * 32), kPfIdesc, (uint32_t)((kb | k4) != 0));
                umma_commit(bar_afree + 8 * sa);           // both slots may be refilled once these MMAs have read them
                if (Q != Q_F16) umma_commit(bar_bfree + 8 * sb);
            }
            umma_commit(bar_done);
        }
    } else {
        // a thread widens a whole row of the K block (as many rows as converter threads), or, with two or four times
        // as many threads as rows, a half or a quarter of one
        constexpr int kPerRow = kPfConvWarps * 32 / NT;       // threads per B row: 1, 2 or 4
        const int c = (threadIdx.x - 64) & (NT - 1);          // B row of this thread
        const int kpart = (threadIdx.x - 64) / NT;
        const int mat = swiglu ? c / rows_mat : 0, rin = swiglu ? c % rows_mat : c;
        const int grow = row0 + rin;
        const bool valid = grow < R;
        if (Q != Q_F16) {
            const int ngrp = a.K / kGroup;
            const __half* srow = a.s[seg + mat] + (size_t)(valid ? grow : 0) * ngrp;
            // the scales of the next two groups are already on their way while a group is widened (a load from L2 takes
            // longer than the MMAs of a K block)
            const __half zero = __float2half(0.f);
            __half sc = valid ? srow[0] : zero, sc1 = valid && ngrp > 1 ? srow[1] : zero, sc2 = valid && ngrp > 2 ? srow[2] : zero;
            for (int kb = 0; kb < nkb && !failed; ++kb) {
                const int sa = kb % NA, sb = kb % NB; const uint32_t pa = (uint32_t)(kb / NA) & 1u, pb = (uint32_t)(kb / NB) & 1u;
                const __half sc_use = sc;
                if (kb & 1) { sc = sc1; sc1 = sc2; const int g3 = (kb >> 1) + 3; sc2 = valid && g3 < ngrp ? srow[g3] : zero; }
                if (!mbar_wait(bar_full + 8 * sa, pa)) { failed = true; break; }
                if (!mbar_wait(bar_bfree + 8 * sb, pb ^ 1u)) { failed = true; break; }     // the MMAs of two K blocks ago have read this B slot
                {
                    constexpr int QQ = Q == Q_F16 ? Q_I8 : Q;
                    const uint32_t rawrow = ring_raw + sa * kRawBytes + c * kRawKb, brow = ring_b + sb * kPfBBytes + c * 128;
                    if (kPerRow == 4) convert_part<QQ, 16>(rawrow + kpart * (kRawKb / 4), brow, c & 7, kpart * 2, __half2half2(sc_use));
                    else {
#pragma unroll
                        for (int kh = kpart; kh < 2; kh += kPerRow)
                            convert_part<QQ, 32>(rawrow + kh * (kRawKb / 2), brow, c & 7, kh * 4, __half2half2(sc_use));
                    }
                }
                fence_async_smem();                            // the tensor core reads through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_conv + 8 * sb);
            }
        }
        // epilogue: TMEM lane = token, column = weight row of the tile
        if (!failed && !mbar_wait(bar_done, 0u)) failed = true;
        tc_fence_after();
        for (int h = 0; h < mh && !failed; ++h) {
            const int q = warp & 3, hh = (warp - 2) >> 2;        // TMEM lane quarter (fixed by the warp's number), column quarter
            const int token = (tm * mh + h) * kPfM + q * 32 + lane;
            const bool tv = token < a.T;
            const uint32_t tlane = tmem + (uint32_t)(h * NT) + ((uint32_t)(q * 32) << 16);
            if (!swiglu) {
#pragma unroll 1
                for (int ch = 0; ch < NT / 64; ++ch) {             // eight epilogue warps: two per TMEM lane quarter, half the columns each (32 columns a warp at the least)
                    const int col = hh * (NT / 2) + ch * 32;
                    float v[32];
                    tmem_ld32(tlane + (uint32_t)col, v);
                    const int r = row0 + col;
                    if (tv && r < R) {
                    if (a.mode == PF_OUT_F32) {
                        float* dst = a.out_f + (size_t)token * a.ldo + coff + r;
#pragma unroll
                        for (int i = 0; i < 32; i += 4) if (r + i < R) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                    } else {
                        __half* dst = a.out_h + (size_t)token * a.ldo + coff + r;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            if (r + i >= R) break;
                            float add[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                            if (a.mode == PF_RESID) {
                                const uint4 o = *reinterpret_cast<const uint4*>(dst + i);
                                const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
                                for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(oh[k]); add[2 * k] = f.x; add[2 * k + 1] = f.y; }
                            } else if (a.bias) {
                                const uint4 o = *reinterpret_cast<const uint4*>(a.bias + coff + r + i);
                                const __half2* oh = reinterpret_cast<const __half2*>(&o);
#pragma unroll
                                for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(oh[k]); add[2 * k] = f.x; add[2 * k + 1] = f.y; }
                            }
                            uint4 o;
                            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                            for (int k = 0; k < 4; ++k) oh[k] = __floats2half2_rn(add[2 * k] + v[i + 2 * k], add[2 * k + 1] + v[i + 2 * k + 1]);
                            *reinterpret_cast<uint4*>(dst + i) = o;
                        }
                    }
                    }
                    __syncwarp();
                }
            } else {
#pragma unroll 1
                for (int ch = 0; ch < (NT >= 128 ? NT / 128 : (hh == 0 ? 1 : 0)); ++ch) {       // 64-row tiles: 32 gate + 32 up columns, one warp per lane quarter takes them
                    const int col = NT >= 128 ? hh * (NT / 4) + ch * 32 : 0;
                    float g[32], u[32];
                    tmem_ld32(tlane + (uint32_t)col, g);
                    tmem_ld32(tlane + (uint32_t)(NT / 2 + col), u);
                    const int r = row0 + col;
                    __half* dst = a.out_h + (size_t)token * a.ldo + r;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (!tv || r + i >= R) break;
                        uint4 o;
                        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float g0 = g[i + 2 * k], g1 = g[i + 2 * k + 1];
                            const float s0 = __fdividef(1.0f, 1.0f + __expf(-g0)), s1 = __fdividef(1.0f, 1.0f + __expf(-g1));
                            oh[k] = __floats2half2_rn(g0 * s0 * u[i + 2 * k], g1 * s1 * u[i + 2 * k + 1]);
                        }
                        *reinterpret_cast<uint4*>(dst + i) = o;
                    }
                    __syncwarp();
                }
            }
        }
    }
    if (failed && a.err) atomicExch(a.err, 11u);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, (uint32_t)(mh * NT));
}

// ---- host side ------------------------------------------------------------------------------------------------------
typedef CUresult (*PfEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PfEncodeFn pf_encode() {
    static PfEncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return (PfEncodeFn)p;
    }();
    return fn;
}
// Row-major 2-D map: `cols` elements a row (row pitch = cols * elem bytes), box box_cols x box_rows.
static int pf_map(CUtensorMap* m, const void* p, CUtensorMapDataType dt, int elem, size_t rows, size_t cols, int box_cols, int box_rows, bool swizzle) {
    PfEncodeFn fn = pf_encode();
    if (!fn) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {cols, rows}, strides[1] = {cols * (size_t)elem};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows}, estr[2] = {1, 1};
    const CUresult r = fn(m, dt, 2, const_cast<void*>(p), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int Q, int NT>
static int pf_go(const PfGemmArgs& a, dim3 grid, cudaStream_t stream) {
    static bool once = false;
    if (!once) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_gemm_kernel<Q, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_smem_bytes(Q, NT));
        if (e != cudaSuccess) return (int)e;
        once = true;
    }
    prefill_gemm_kernel<Q, NT><<<grid, kPfThreads, pf_smem_bytes(Q, NT), stream>>>(a);
    return (int)cudaGetLastError();
}

int launch_prefill_gemm(int quant, PfGemmArgs& a, const void* x, const void* const* w, const int* rows, int nmat, cudaStream_t stream) {
    if (a.T <= 0 || a.K <= 0 || a.K % kGroup || a.ldo % 8 || quant < 0 || quant > 2 || nmat < 1 || nmat > 3) return (int)cudaErrorInvalidValue;
    const bool swiglu = a.mode == PF_SWIGLU;
    if (swiglu && (nmat != 2 || rows[0] != rows[1])) return (int)cudaErrorInvalidValue;
    // Tile width: 256 weight rows a CTA; 128 or 64 where the wide tiles would leave more than half / three quarters of
    // the SMs without a CTA (short prompts; the projections with few rows): more CTAs, each with less widening and MMA work.
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    a.mh = a.T > kPfM ? kPfMH : 1;
    const int mtiles = (a.T + kPfM * a.mh - 1) / (kPfM * a.mh);
    int wide = 0;
    for (int m = 0; m < (swiglu ? 1 : nmat); ++m) wide += (rows[m] + (swiglu ? kPfN / 2 : kPfN) - 1) / (swiglu ? kPfN / 2 : kPfN);
    const int nt = (sms > 0 && wide * mtiles * 4 <= sms) ? kPfN / 4 : (sms > 0 && wide * mtiles * 2 <= sms) ? kPfN / 2 : kPfN;
    const int rows_mat = swiglu ? nt / 2 : nt;
    if (int r = pf_map(&a.tx, x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (size_t)a.T, (size_t)a.K, kPfKB, kPfM, true)) return r;
    int tiles = 0;
    a.R = 0;
    for (int m = 0; m < nmat; ++m) {
        if (!w[m] || rows[m] <= 0 || rows[m] % 8) return (int)cudaErrorInvalidValue;
        int r;
        if (quant == Q_F16) r = pf_map(&a.tw[m], w[m], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (size_t)rows[m], (size_t)a.K, kPfKB, rows_mat, true);
        else {
            const size_t rb = quant == Q_I4 ? (size_t)a.K / 2 : (size_t)a.K;
            r = pf_map(&a.tw[m], w[m], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (size_t)rows[m], rb, quant == Q_I4 ? 32 : 64, rows_mat, false);
        }
        if (r) return r;
        a.seg_rows[m] = rows[m];
        if (!swiglu || m == 0) { tiles += (rows[m] + rows_mat - 1) / rows_mat; a.R += rows[m]; }
    }
    a.nseg = swiglu ? 1 : nmat;
    const dim3 grid(mtiles, tiles);
    if (nt == kPfN) {
        if (quant == Q_I4) return pf_go<Q_I4, kPfN>(a, grid, stream);
        if (quant == Q_I8) return pf_go<Q_I8, kPfN>(a, grid, stream);
        return pf_go<Q_F16, kPfN>(a, grid, stream);
    }
    if (nt == kPfN / 2) {
        if (quant == Q_I4) return pf_go<Q_I4, kPfN / 2>(a, grid, stream);
        if (quant == Q_I8) return pf_go<Q_I8, kPfN / 2>(a, grid, stream);
        return pf_go<Q_F16, kPfN / 2>(a, grid, stream);
    }
    if (quant == Q_I4) return pf_go<Q_I4, kPfN / 4>(a, grid, stream);
    if (quant == Q_I8) return pf_go<Q_I8, kPfN / 4>(a, grid, stream);
    return pf_go<Q_F16, kPfN / 4>(a, grid, stream);
}

}  // namespace cq
