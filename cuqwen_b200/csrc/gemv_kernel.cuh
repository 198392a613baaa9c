// The GEMV kernel: one producer warp keeps a CTA-wide ring of TMA stages full, eight consumer warps run the
// tensor-core inner product on it.  See gemv.cuh for the data path and gemv_math.cuh for the arithmetic.
//
// Work split.  The consumer warps form rw row-warps x kw K-parts (rw * kw = 8).  A CTA "block" is rw consecutive
// 16-row tile sets; every ring step brings, for each K-part and tile, one box of (16*rw rows) x piece_bytes.  K-part kp
// handles row pieces kp, kp+kw, ...; partial sums of the K-parts are merged in shared memory.  Blocks go to CTAs
// round-robin.
#pragma once
#include "gemv.cuh"
#include "gemv_stage.cuh"

namespace cq {

constexpr int kGemvThreads = (kConsumerWarps + 1) * 32;

template <int Q, int EPI>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const __grid_constant__ GemvArgs a) {
    constexpr int MT = EpiMT<EPI>::MT;
    constexpr int GB = QT<Q>::GB;
    constexpr bool kInt = Q != Q_F16;
    constexpr int NC = kConsumerWarps * 32;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    pdl_launch_dependents();    // the next kernel in the stream may start its weight prefetch while this one runs
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rw = a.rw, kw = a.kw, nst = a.nst, pg = a.pg;
    const int ngrp = a.K / kGroup;
    const GemvLayout L = gemv_layout(a.K, GB, MT, rw, kw, pg, nst, kInt);
    const uint32_t sm0 = smem_u32(smem_raw);
    const uint32_t bars = sm0 + L.off_bars;
    const uint32_t bar_full = bars, bar_empty = bars + nst * 8, bar_sfull = bars + 2 * nst * 8, bar_sempty = bars + (2 * nst + 2) * 8;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nst; ++s) { mbar_init(bar_full + s * 8, 1); mbar_init(bar_empty + s * 8, kConsumerWarps); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_sfull + b * 8, 1); mbar_init(bar_sempty + b * 8, kConsumerWarps); }
        mbar_fence_init();
    }
    __syncthreads();

    const int rb = Q == Q_I4 ? a.K / 2 : Q == Q_I8 ? a.K : a.K * 2;            // bytes of one weight row
    const int PT = (rb + L.piece_bytes - 1) / L.piece_bytes;                   // pieces in a full row
    const int S = (PT + kw - 1) / kw;                                          // ring steps per block
    const int nblk = (a.nsets + rw - 1) / rw;
    const int n_b = (int)blockIdx.x < nblk ? (nblk - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp == kConsumerWarps) {
        // ------------------------------- producer warp: reads only weights and scales -------------------------------
        bool failed = false;
        for (int j = 0; j < n_b; ++j) {
            const int blk = blockIdx.x + j * gridDim.x;
            const TileMap<EPI> tm = map_tileset<EPI>(a, blk * rw);
            if (kInt) {
                if (!failed && !mbar_wait(bar_sempty + (j & 1) * 8, ((j >> 1) & 1) ^ 1)) { failed = true; if (a.err) atomicExch(a.err, 3u); }
                const int rows_here = min(L.box_rows, (EPI == EPI_QKV ? 16 : a.rows - tm.row0));
                const int bytes_m = rows_here * ngrp * 2;
                const uint32_t dst = sm0 + L.off_scales + (j & 1) * L.scale_block_bytes;
                if ((bytes_m & 15) == 0) {
                    if (lane == 0) {
                        mbar_expect_tx(bar_sfull + (j & 1) * 8, (uint32_t)(bytes_m * MT));
#pragma unroll
                        for (int m = 0; m < MT; ++m) bulk_g2s(dst + m * L.box_rows * ngrp * 2, tm.sbase[m], bytes_m, bar_sfull + (j & 1) * 8);
                    }
                } else {
                    // ragged last block: its scale rows are not a whole number of 16-byte units; copy with plain loads
                    __half* sb = reinterpret_cast<__half*>(smem_raw + L.off_scales + (j & 1) * L.scale_block_bytes);
                    for (int m = 0; m < MT; ++m)
                        for (int idx = lane; idx < rows_here * ngrp; idx += 32) sb[m * L.box_rows * ngrp + idx] = tm.sbase[m][idx];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_sfull + (j & 1) * 8);
                }
                __syncwarp();
            }
            for (int p = 0; p < S; ++p) {
                const int i = j * S + p, s = i % nst;
                if (!failed && !mbar_wait(bar_empty + s * 8, ((i / nst) & 1) ^ 1)) { failed = true; if (a.err) atomicExch(a.err, 4u); }
                int nparts = PT - p * kw; if (nparts > kw) nparts = kw;        // K-parts that still have a piece at this step
                if (lane == 0) mbar_expect_tx(bar_full + s * 8, (uint32_t)(nparts * MT * L.box_bytes));   // boxes deliver their full size
                __syncwarp();
                if (lane < nparts * MT) {
                    const int kp = lane / MT, m = lane - kp * MT;
                    tma_load_2d(sm0 + L.off_stages + s * L.stage_bytes + (kp * MT + m) * L.box_bytes, &a.tmap[tm.mmat[m]],
                                (kp + p * kw) * L.piece_bytes, tm.mrow[m], bar_full + s * 8);
                }
            }
        }
        return;
    }

    // ------------------------------------------- consumer warps ---------------------------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int rwi = warp % rw, kwi = warp / rw;
    uint4* xs = reinterpret_cast<uint4*>(smem_raw);
    int* corr = reinterpret_cast<int*>(smem_raw + L.off_corr);
    float* xscale = reinterpret_cast<float*>(smem_raw + L.off_xscale);
    float* red = reinterpret_cast<float*>(smem_raw + L.off_red);

    pdl_wait();                 // the activation vector comes from the previous kernel
    if constexpr (kInt) stage_x_digits<Q>(a.x, a.norm_w, a.eps, a.K, smem_raw, corr, xscale, red, NC);
    else stage_x_f16(a.x, a.norm_w, a.eps, a.K, xs, red, NC);

    bool failed = false;
    for (int j = 0; j < n_b; ++j) {
        const int blk = blockIdx.x + j * gridDim.x;
        const int ts = blk * rw + rwi;
        const bool live = ts < a.nsets && kwi < kw;       // spare warps (rw * kw < 8) only keep the barriers moving
        const TileMap<EPI> tm = map_tileset<EPI>(a, live ? ts : 0);
        float tot[MT][2];
        float cf[MT][2][4];
        int ci[MT][2][4];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            tot[m][0] = tot[m][1] = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) { cf[m][0][q] = cf[m][1][q] = 0.f; ci[m][0][q] = ci[m][1][q] = 0; }
        }
        uint32_t sbuf = 0;
        if (kInt) {
            if (!failed && !mbar_wait(bar_sfull + (j & 1) * 8, (j >> 1) & 1)) { failed = true; if (a.err) atomicExch(a.err, 2u); }
            sbuf = sm0 + L.off_scales + (j & 1) * L.scale_block_bytes + (rwi * 16 + g) * ngrp * 2;     // this lane's row g of tile 0
        }
        for (int p = 0; p < S; ++p) {
            const int i = j * S + p, s = i % nst;
            if (!failed && !mbar_wait(bar_full + s * 8, (i / nst) & 1)) { failed = true; if (a.err) atomicExch(a.err, 1u); }
            const int c = kwi + p * kw;
            if (live && c < PT) {
                const int grp0 = c * pg;
                const int ngp = ngrp - grp0 < pg ? ngrp - grp0 : pg;
                const uint32_t wrow = sm0 + L.off_stages + s * L.stage_bytes + kwi * MT * L.box_bytes + (rwi * 16 + g) * L.piece_bytes;
                for (int gi = 0; gi < ngp; ++gi) {
                    const int grp = grp0 + gi;
                    if constexpr (kInt) {
                        compute_group_int<Q, MT>(wrow + gi * GB, L.piece_bytes, L.box_bytes, g, t, sm0 + grp * 256, ci);
                        const int cr = corr[grp];
                        const float xsc = xscale[grp];
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            const uint32_t sa = sbuf + (m * L.box_rows * ngrp + grp) * 2;
                            const float s0 = lds_h(sa) * xsc, s1 = lds_h(sa + 8 * ngrp * 2) * xsc;
                            // columns 0 and 1 (lanes with t == 0) hold sum q*d0 and sum q*d1
                            const int v0 = (ci[m][0][0] + ci[m][1][0]) + ((ci[m][0][1] + ci[m][1][1]) << 8) - cr;
                            const int v1 = (ci[m][0][2] + ci[m][1][2]) + ((ci[m][0][3] + ci[m][1][3]) << 8) - cr;
                            tot[m][0] = fmaf((float)v0, s0, tot[m][0]);
                            tot[m][1] = fmaf((float)v1, s1, tot[m][1]);
#pragma unroll
                            for (int q = 0; q < 4; ++q) ci[m][0][q] = ci[m][1][q] = 0;
                        }
                    } else {
                        compute_group_f16<MT>(wrow + gi * GB, L.piece_bytes, L.box_bytes, t, xs + grp * 16, cf);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + s * 8);       // this warp is done with the stage
        }
        if (kInt) { __syncwarp(); if (lane == 0) mbar_arrive(bar_sempty + (j & 1) * 8); }
        if constexpr (!kInt) {
#pragma unroll
            for (int m = 0; m < MT; ++m) { tot[m][0] = cf[m][0][0] + cf[m][1][0]; tot[m][1] = cf[m][0][2] + cf[m][1][2]; }
        }
        if (kw > 1) {
            if (t == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) { red[warp * 32 + m * 16 + g] = tot[m][0]; red[warp * 32 + m * 16 + g + 8] = tot[m][1]; }
            }
            consumer_sync(NC);
            if (kwi == 0 && lane < 16 && live) {
                float v0 = 0.f, v1 = 0.f;
                for (int kp = 0; kp < kw; ++kp) { v0 += red[(kp * rw + rwi) * 32 + lane]; if (MT == 2) v1 += red[(kp * rw + rwi) * 32 + 16 + lane]; }
                epilogue<EPI>(a, tm.row0, tm.mat, lane, v0, v1);
            }
            consumer_sync(NC);         // `red` is free again
        } else if (t == 0 && live) {
            epilogue<EPI>(a, tm.row0, tm.mat, g, tot[0][0], MT == 2 ? tot[MT - 1][0] : 0.f);
            epilogue<EPI>(a, tm.row0, tm.mat, g + 8, tot[0][1], MT == 2 ? tot[MT - 1][1] : 0.f);
        }
    }
}

}  // namespace cq
