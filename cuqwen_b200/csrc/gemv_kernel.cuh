// The GEMV data path: one producer warp keeps a CTA-wide ring of TMA stages full, eight consumer warps run the
// tensor-core inner product on it.  See gemv.cuh for the argument block and gemv_math.cuh for the arithmetic.
//
// Work split.  The consumer warps form rw row-warps x kw K-parts x gw group-parts (rw * kw * gw <= 8).  A CTA "block" is `brows`
// consecutive rows (at most 16 * rw: row-warp i takes rows 16 i .. 16 i + 15 of it; `brows` need not be a multiple of 16, the host picks it
// so that the blocks fill the SMs evenly); every ring step brings, for each K-part and matrix, one box of brows rows x piece_bytes.  K-part kp
// handles row pieces kp, kp+kw, ...; partial sums of the K-parts are merged in shared memory.  Blocks go to CTAs
// round-robin.
//
// gemv_produce / gemv_consume are the two halves; they keep their place in the ring in a RingCtx, so that a caller
// can run several matrices back to back through one ring (the producer then runs ahead into the next matrix while
// the consumers finish the current one).  gemv_kernel is the one-matrix-per-launch wrapper.
#pragma once
#include "gemv.cuh"
#include "gemv_stage.cuh"

namespace cq {

constexpr int kGemvThreads = (kConsumerWarps + 1) * 32;
constexpr int kConsumerThreads = kConsumerWarps * 32;

// Shared-memory map of a CTA plus this thread's position in the ring.  Layout: [x area at offset 0][corr][xscale]
// [red][two scale blocks][nslots ring slots][mbarriers: full[nslots], empty[nslots], scale full[2], scale empty[2]].
struct RingCtx {
    uint32_t sm0;                 // shared-window address of offset 0
    unsigned char* base;          // generic pointer to offset 0
    int off_corr, off_xscale, off_red, off_scales, scale_block_bytes, off_stages, slot_bytes, nslots;
    uint32_t bar_full, bar_empty, bar_sfull, bar_sempty;
    uint32_t bar_x, xpar;         // barrier of the bulk-copied activation vector and its parity
    int slot;                     // next ring slot
    uint32_t par;                 // its parity: number of completed laps, mod 2
    uint32_t sj;                  // scale blocks used so far
    uint32_t nsb;                 // scale blocks in shared memory (1 or 2): block j uses buffer j % nsb in phase (j / nsb) & 1
    unsigned* err;                // device word that receives a code when a bounded wait expires (may be null)
    bool failed;                  // a wait of this thread expired: stop waiting, finish with meaningless numbers

    __device__ __forceinline__ void advance() { if (++slot == nslots) { slot = 0; par ^= 1u; } }
    __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity, unsigned code) {
        if (!failed && !mbar_wait(bar, parity)) { failed = true; if (err) atomicExch(err, code); }
    }
};

__device__ __forceinline__ void ring_init_barriers(const RingCtx& R) {
    for (int s = 0; s < R.nslots; ++s) { mbar_init(R.bar_full + s * 8, 1); mbar_init(R.bar_empty + s * 8, kConsumerWarps); }
    for (int b = 0; b < 2; ++b) { mbar_init(R.bar_sfull + b * 8, 1); mbar_init(R.bar_sempty + b * 8, kConsumerWarps); }
    mbar_init(R.bar_x, 1);
    mbar_fence_init();
}

template <int Q, int EPI>
struct GemvGeom {
    static constexpr int MT = EpiMT<EPI>::MT;
    static constexpr int GB = QT<Q>::GB;
    int piece_bytes, box_rows, box_bytes, box_stride, stage_bytes, ngrp, PT, S, nblk;
    __device__ __forceinline__ GemvGeom(const GemvArgs& a) {
        piece_bytes = a.pg * GB; box_rows = EPI == EPI_QKV ? 16 : a.brows; box_bytes = box_rows * piece_bytes; box_stride = (box_bytes + 127) / 128 * 128; stage_bytes = a.kw * MT * box_stride;
        ngrp = a.K / kGroup;
        const int rb = Q == Q_I4 ? a.K / 2 : Q == Q_I8 ? a.K : a.K * 2;     // bytes of one weight row
        PT = (rb + piece_bytes - 1) / piece_bytes;                          // pieces in a full row
        S = (PT + a.kw - 1) / a.kw;                                         // ring steps per block
        nblk = EPI == EPI_QKV ? a.nsets : a.nblk;
    }
};

// Producer warp (all 32 lanes call): streams the weights and scales of CTA `cta`'s blocks.  Reads nothing that the
// step itself writes.
template <int Q, int EPI>
__device__ __forceinline__ void gemv_produce(const GemvArgs& a, RingCtx& R, int cta, int ncta) {
    constexpr int MT = EpiMT<EPI>::MT;
    constexpr bool kInt = Q != Q_F16;
    const GemvGeom<Q, EPI> G(a);
    const int lane = threadIdx.x & 31, kw = a.kw;
    const int n_b = cta < G.nblk ? (G.nblk - cta + ncta - 1) / ncta : 0;
    for (int j = 0; j < n_b; ++j) {
        const int blk = cta + j * ncta;
        const TileMap<EPI> tm = map_tile<EPI>(a, blk, 0);
        if (kInt) {
            const int sb = R.sj % R.nsb;
            R.wait(R.bar_sempty + sb * 8, ((R.sj / R.nsb) & 1) ^ 1, 3u);
            const int rows_here = min(G.box_rows, (EPI == EPI_QKV ? 16 : a.rows - tm.row0));
            const int bytes_m = rows_here * G.ngrp * 2;
            const uint32_t dst = R.sm0 + R.off_scales + sb * R.scale_block_bytes;
            bool aligned = (bytes_m & 15) == 0;                   // a bulk copy wants 16-byte sizes and addresses
#pragma unroll
            for (int m = 0; m < MT; ++m) aligned = aligned && (reinterpret_cast<uintptr_t>(tm.sbase[m]) & 15) == 0;
            if (aligned) {
                if (lane == 0) {
                    mbar_expect_tx(R.bar_sfull + sb * 8, (uint32_t)(bytes_m * MT));
#pragma unroll
                    for (int m = 0; m < MT; ++m) bulk_g2s(dst + m * G.box_rows * G.ngrp * 2, tm.sbase[m], bytes_m, R.bar_sfull + sb * 8);
                }
            } else {
                // a block whose scale rows are not whole, aligned 16-byte units (odd row counts, a ragged last block): plain loads
                __half* sbp = reinterpret_cast<__half*>(R.base + R.off_scales + sb * R.scale_block_bytes);
                for (int m = 0; m < MT; ++m)
                    for (int idx = lane; idx < rows_here * G.ngrp; idx += 32) sbp[m * G.box_rows * G.ngrp + idx] = tm.sbase[m][idx];
                __syncwarp();
                if (lane == 0) mbar_arrive(R.bar_sfull + sb * 8);
            }
            __syncwarp();
            ++R.sj;
        }
        for (int p = 0; p < G.S; ++p) {
            const int s = R.slot;
            R.wait(R.bar_empty + s * 8, R.par ^ 1u, 4u);
            int nparts = G.PT - p * kw; if (nparts > kw) nparts = kw;        // K-parts that still have a piece at this step
            if (lane == 0) mbar_expect_tx(R.bar_full + s * 8, (uint32_t)(nparts * MT * G.box_bytes));   // boxes deliver their full size
            __syncwarp();
            if (lane < nparts * MT) {
                const int kp = lane / MT, m = lane - kp * MT;
                tma_load_3d(R.sm0 + R.off_stages + s * R.slot_bytes + (kp * MT + m) * G.box_stride, &a.tmap[tm.mmat[m]],
                            0, tm.mrow[m], (kp + p * kw) * (G.piece_bytes / kChunkBytes), R.bar_full + s * 8);
            }
            R.advance();
        }
    }
}

// Consumer warps (the first kConsumerThreads threads call): stage x, run the blocks of CTA `cta`, write the outputs.
template <int Q, int EPI>
__device__ __forceinline__ void gemv_consume(const GemvArgs& a, RingCtx& R, int cta, int ncta) {
    constexpr int MT = EpiMT<EPI>::MT;
    constexpr int GB = QT<Q>::GB;
    constexpr bool kInt = Q != Q_F16;
    constexpr int NC = kConsumerThreads;
    const GemvGeom<Q, EPI> G(a);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rw = a.rw, kw = a.kw, gw = a.gw, pg = a.pg, ngrp = G.ngrp;
    const int rwi = warp % rw, kwi = (warp / rw) % kw, gwi = warp / (rw * kw);     // warp = rwi + rw * (kwi + kw * gwi)
    const int n_b = cta < G.nblk ? (G.nblk - cta + ncta - 1) / ncta : 0;
    uint4* xs = reinterpret_cast<uint4*>(R.base);
    int* corr = reinterpret_cast<int*>(R.base + R.off_corr);
    float* xscale = reinterpret_cast<float*>(R.base + R.off_xscale);
    float* red = reinterpret_cast<float*>(R.base + R.off_red);

    GatherSrc gs{a.gather, a.ngather, 0u, a.x_next, cta == 0, R.err, a.wait_cycles > 0 ? a.wait_cycles : kWaitCyclesDefault};
    if (a.ngather > 0) gs.seq = (unsigned)(*a.step_no) * kSeqPerStep + (unsigned)a.seq_index + 1u;     // tensor parallel: x plus the partials the ranks pushed
    if (kInt && a.xd_in) {
        // the vector arrives already staged (digit blocks, corrections, scales written by the kernel that produced it)
        const uint32_t cbytes = (uint32_t)((ngrp * 4 + 15) / 16 * 16);
        if (threadIdx.x == 0) {
            fence_async_smem();
            mbar_expect_tx(R.bar_x, (uint32_t)(a.K * 2) + 2u * cbytes);
            bulk_g2s(R.sm0, a.xd_in, (uint32_t)(a.K * 2), R.bar_x);
            bulk_g2s(R.sm0 + R.off_corr, a.corr_in, cbytes, R.bar_x);
            bulk_g2s(R.sm0 + R.off_xscale, a.xscale_in, cbytes, R.bar_x);
        }
        R.wait(R.bar_x, R.xpar, 9u);
        R.xpar ^= 1u;
    } else if (stage_x<Q>(a.x, a.norm_w, a.eps, a.K, R.base, R.off_corr, corr, xscale, red, NC, a.ngather > 0 ? &gs : nullptr, R.bar_x, R.xpar, a.trace)) R.xpar ^= 1u;
    // a SwiGLU kernel whose block is a whole 128-row group hands its outputs over in staged form as well
    const bool emit = EPI == EPI_SWIGLU && kInt && a.xd_out != nullptr && a.brows == 128 && rw == 8 && kw == 1 && gw == 1;
    __half* hbuf = reinterpret_cast<__half*>(red);
    if (threadIdx.x == 0) trace_last(a.trace, 3);

    for (int j = 0; j < n_b; ++j) {
        const int blk = cta + j * ncta;
        const TileMap<EPI> tm = map_tile<EPI>(a, blk, rwi);
        const bool live = tm.row0 < tm.row_end && gwi < gw;       // warps without rows (a short block, spare warps) only keep the barriers moving
        float tot[MT][2];
        float cf[MT][2][4];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            tot[m][0] = tot[m][1] = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) cf[m][0][q] = cf[m][1][q] = 0.f;
        }
        const bool merged = kw * gw > 1;                 // K-parts meet in shared memory; lanes 0-15 of the first part finish the rows
        float preA[2] = {0.f, 0.f}, preB[2] = {0.f, 0.f};
        if (merged) { if (kwi == 0 && gwi == 0 && lane < 16 && live) epilogue_fetch<EPI>(a, tm.row0, tm.row_end, tm.mat, lane, preA); }
        else if (t == 0 && live) { epilogue_fetch<EPI>(a, tm.row0, tm.row_end, tm.mat, g, preA); epilogue_fetch<EPI>(a, tm.row0, tm.row_end, tm.mat, g + 8, preB); }
        uint32_t sbuf = 0;
        const int sb = R.sj % R.nsb;
        if (kInt) {
            R.wait(R.bar_sfull + sb * 8, (R.sj / R.nsb) & 1, 2u);
            sbuf = R.sm0 + R.off_scales + sb * R.scale_block_bytes + (rwi * 16 + g) * ngrp * 2;     // this lane's row g of tile 0
        }
        for (int p = 0; p < G.S; ++p) {
            const int s = R.slot;
            R.wait(R.bar_full + s * 8, R.par, 1u);
            const int c = kwi + p * kw;
            if (live && c < G.PT) {
                const int grp0 = c * pg;
                const int ngp = ngrp - grp0 < pg ? ngrp - grp0 : pg;
                const int cstride = G.box_rows * kChunkBytes;        // chunk-major box: [chunk][row][64 bytes]
                const uint32_t wrow = R.sm0 + R.off_stages + s * R.slot_bytes + kwi * MT * G.box_stride + (rwi * 16 + g) * kChunkBytes + t * 16;
                if constexpr (kInt) {
                    constexpr int NI = QT<Q>::NI;
                    for (int gi = gwi; gi < ngp; gi += gw) {
                        const int grp = grp0 + gi;
                        uint4 w[MT][2][NI], xv[2];
                        load_group_w<Q, MT>(wrow + gi * (GB / kChunkBytes) * cstride, cstride, G.box_stride, w);
                        load_group_x(R.sm0 + grp * 256, g, t, xv);
                        const int cr = (int)lds32(R.sm0 + R.off_corr + grp * 4);
                        const float xsc = __uint_as_float(lds32(R.sm0 + R.off_xscale + grp * 4));
                        float sc[MT][2];
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            const uint32_t sa = sbuf + (m * G.box_rows * ngrp + grp) * 2;
                            sc[m][0] = lds_h(sa) * xsc; sc[m][1] = lds_h(sa + 8 * ngrp * 2) * xsc;
                        }
                        int ci[MT][2][4];
                        mma_group_int<Q, MT>(w, xv, ci);
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            // columns 0 and 1 (lanes with t == 0) hold sum q*d0 and sum q*d1
                            const int v0 = (ci[m][0][0] + ci[m][1][0]) + ((ci[m][0][1] + ci[m][1][1]) << 8) - cr;
                            const int v1 = (ci[m][0][2] + ci[m][1][2]) + ((ci[m][0][3] + ci[m][1][3]) << 8) - cr;
                            tot[m][0] = fmaf((float)v0, sc[m][0], tot[m][0]);
                            tot[m][1] = fmaf((float)v1, sc[m][1], tot[m][1]);
                        }
                    }
                } else {
                    for (int gi = gwi; gi < ngp; gi += gw)
                        compute_group_f16<MT>(wrow + gi * (GB / kChunkBytes) * cstride, cstride, G.box_stride, t, xs + (grp0 + gi) * 16, cf);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(R.bar_empty + s * 8);       // this warp is done with the stage
            R.advance();
        }
        if (kInt) { __syncwarp(); if (lane == 0) mbar_arrive(R.bar_sempty + sb * 8); ++R.sj; }
        if (threadIdx.x == 0 && j == n_b - 1) trace_last(a.trace, 4);
        if constexpr (!kInt) {
#pragma unroll
            for (int m = 0; m < MT; ++m) { tot[m][0] = cf[m][0][0] + cf[m][1][0]; tot[m][1] = cf[m][0][2] + cf[m][1][2]; }
        }
        if (merged) {
            if (t == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) { red[warp * 32 + m * 16 + g] = tot[m][0]; red[warp * 32 + m * 16 + g + 8] = tot[m][1]; }
            }
            consumer_sync(NC);
            if (kwi == 0 && gwi == 0 && lane < 16 && live) {
                float v0 = 0.f, v1 = 0.f;
                for (int kp = 0; kp < kw * gw; ++kp) { v0 += red[(kp * rw + rwi) * 32 + lane]; if (MT == 2) v1 += red[(kp * rw + rwi) * 32 + 16 + lane]; }
                epilogue<EPI>(a, tm.row0, tm.row_end, tm.mat, lane, v0, v1, preA);
            }
            consumer_sync(NC);         // `red` is free again
        } else if (t == 0 && live) {
            epilogue<EPI>(a, tm.row0, tm.row_end, tm.mat, g, tot[0][0], MT == 2 ? tot[MT - 1][0] : 0.f, preA, emit ? hbuf + rwi * 16 : nullptr);
            epilogue<EPI>(a, tm.row0, tm.row_end, tm.mat, g + 8, tot[0][1], MT == 2 ? tot[MT - 1][1] : 0.f, preB, emit ? hbuf + rwi * 16 : nullptr);
        }
        if constexpr (EPI == EPI_SWIGLU && kInt) {
            if (emit && (blk + 1) * 128 <= a.rows) {       // a whole 128-row group (uniform over the CTA)
                consumer_sync(NC);
                if (warp == 0) {
                    const int c = lane & 15;
                    const uint4 v = reinterpret_cast<const uint4*>(hbuf)[c];
                    digits_of_chunk<Q>(v, blk * 16 + c, lane < 16, a.xd_out, a.corr_out, a.xscale_out);
                }
                consumer_sync(NC);                         // hbuf is free for the next block
            }
        }
    }
}

// Ring context of a stand-alone launch: the layout gemv_layout computed for this matrix, an empty ring.
template <int Q, int EPI>
__device__ __forceinline__ RingCtx gemv_ring(const GemvArgs& a, unsigned char* smem) {
    const GemvLayout L = gemv_layout(a.K, QT<Q>::GB, EpiMT<EPI>::MT, EPI == EPI_QKV ? 16 : a.brows, a.kw, a.pg, a.nst, Q != Q_F16, a.nsb);
    RingCtx R;
    R.sm0 = smem_u32(smem); R.base = smem;
    R.off_corr = L.off_corr; R.off_xscale = L.off_xscale; R.off_red = L.off_red; R.off_scales = L.off_scales;
    R.scale_block_bytes = L.scale_block_bytes; R.off_stages = L.off_stages; R.slot_bytes = L.stage_bytes; R.nslots = a.nst;
    R.bar_full = R.sm0 + L.off_bars; R.bar_empty = R.bar_full + a.nst * 8; R.bar_sfull = R.bar_empty + a.nst * 8; R.bar_sempty = R.bar_sfull + 16;
    R.bar_x = R.bar_sempty + 16; R.xpar = 0u;
    R.slot = 0; R.par = 0; R.sj = 0; R.nsb = (uint32_t)a.nsb; R.err = a.err; R.failed = false;
    return R;
}

template <int Q, int EPI>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const __grid_constant__ GemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    pdl_launch_dependents();    // the next kernel in the stream may start its weight prefetch while this one runs
    RingCtx R = gemv_ring<Q, EPI>(a, smem_raw);
    if (threadIdx.x == 0) { trace_first(a.trace, 0); trace_last(a.trace, 1); trace_start(a.trace); ring_init_barriers(R); }
    __syncthreads();
    if ((threadIdx.x >> 5) == kConsumerWarps) {
        if (blockIdx.x == 0) {
#pragma unroll
            for (int i = 0; i < 3; ++i)
                for (int off = (threadIdx.x & 31) * 128; off < a.warm_bytes[i]; off += 32 * 128)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(a.warm[i]) + off));
        }
        gemv_produce<Q, EPI>(a, R, blockIdx.x, gridDim.x);
        return;
    }
    pdl_wait();                 // the activation vector comes from the previous kernel
    if (threadIdx.x == 0) trace_first(a.trace, 2);
    gemv_consume<Q, EPI>(a, R, blockIdx.x, gridDim.x);
    if (threadIdx.x == 0) trace_last(a.trace, 5);
}

}  // namespace cq
