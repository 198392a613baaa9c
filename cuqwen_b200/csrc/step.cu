// Host side of the persistent decode-step kernel (step_kernel.cuh): per-phase work split, shared-memory map, launch.
#include "step_kernel.cuh"

#include "launch.h"

namespace cq {

// Work split of one GEMV phase for `ncta` CTAs whose ring slots hold `slot_bytes`:
//   rw (16-row tile sets per block) minimises the tile sets on the busiest CTA, larger rw on ties (fewer blocks, fewer
//   merges); kw = 8 / rw K-parts, no more than a row has pieces; pg = the largest piece that lets a stage fit a slot.
int plan_step_gemv(int quant, int epi, GemvArgs& a, int ncta, int slot_bytes) {
    if (a.K <= 0 || a.K % kGroup != 0 || quant < 0 || quant > 2) return (int)cudaErrorInvalidValue;
    if (epi == EPI_QKV) {
        if (a.hd % 32 != 0) return (int)cudaErrorInvalidValue;
        a.nsets = (a.n_heads + 2 * a.n_kv) * (a.hd / 32);
    } else {
        if (a.rows <= 0) return (int)cudaErrorInvalidValue;
        a.nsets = (a.rows + 15) / 16;
    }
    const int MT = (epi == EPI_SWIGLU || epi == EPI_QKV) ? 2 : 1;
    const int ngrp = a.K / kGroup;
    const int gb = quant == Q_I4 ? 64 : quant == Q_I8 ? 128 : 256;
    int best_rw = 0, best_cost = 0;
    for (int rw = (epi == EPI_QKV ? 1 : 4); rw >= 1; rw /= 2) {
        const int nblk = (a.nsets + rw - 1) / rw;
        const int cost = (nblk + ncta - 1) / ncta * rw;
        if (!best_rw || cost < best_cost) { best_rw = rw; best_cost = cost; }
    }
    const int rw = best_rw;
    int kw = 0, pg = 0;
    for (int kcap = 8 / rw; kcap >= 1 && !pg; kcap /= 2)          // fp16 gate/up: fewer K-parts so that one piece still fits
        for (int q = 256 / gb; q >= 1; --q) {
            const int pt = (ngrp + q - 1) / q;
            int k = kcap; while (k > 1 && k > pt) k /= 2;
            if (k * MT * 16 * rw * q * gb <= slot_bytes) { kw = k; pg = q; break; }
        }
    if (!pg) return (int)cudaErrorInvalidValue;
    int gw = kConsumerWarps / (rw * kw);
    while (gw > 1 && gw > pg) gw /= 2;
    a.rw = rw; a.kw = kw; a.gw = gw; a.pg = pg; a.nst = 0;
    const size_t rbytes = quant == Q_I4 ? a.K / 2 : quant == Q_I8 ? a.K : (size_t)a.K * 2;
    const int nmat = epi == EPI_QKV ? 3 : epi == EPI_SWIGLU ? 2 : 1;
    for (int m = 0; m < nmat; ++m) {
        const size_t rows_m = epi == EPI_QKV ? (size_t)(m == 0 ? a.n_heads : a.n_kv) * a.hd : (size_t)a.rows;
        if (int r = make_weight_map(&a.tmap[m], a.w[m], rbytes, rows_m, pg * gb, 16 * rw)) return r;
    }
    return 0;
}

// Shared-memory map for a planned phase table.  Returns 0 and fills `sa`, or an error when not even three slots fit.
int plan_step_smem(StepArgs& sa, const StepPhase* ph, int n, int hd, int slot_bytes, int max_smem) {
    int kmax = 0, scale_block = 0, xnorm = 0;
    bool attn = false;
    for (int i = 0; i < n; ++i) {
        if (ph[i].kind != PH_GEMV) { attn = true; continue; }
        const GemvArgs& a = ph[i].g;
        const int MT = (ph[i].epi == EPI_SWIGLU || ph[i].epi == EPI_QKV) ? 2 : 1;
        if (a.K > kmax) kmax = a.K;
        if (a.norm_w && a.K <= 8192 && 4 * a.K > xnorm) xnorm = 4 * a.K;     // x and the norm weight side by side while staging
        if (ph[i].quant != Q_F16) { const int sb = MT * 16 * a.rw * (a.K / kGroup) * 2; if (sb > scale_block) scale_block = sb; }
    }
    int xarea = kmax * 2 > xnorm ? kmax * 2 : xnorm;
    if (attn) {
        const int need = kStepAttnWarps * kMaxGroup * hd * 4 + kStepAttnWarps * kMaxGroup * 2 * 4 + 16;    // also covers the fold phase's scratch
        if (need > xarea) xarea = need;
        if (2 * kStepAttnKeys * hd * 2 > slot_bytes) return (int)cudaErrorInvalidValue;
    }
    const int ng = kmax / kGroup;
    int o = (xarea + 15) / 16 * 16;
    sa.off_corr = o; o += (ng * 4 + 15) / 16 * 16;
    sa.off_xscale = o; o += (ng * 4 + 15) / 16 * 16;
    sa.off_red = o; o += kConsumerWarps * 32 * 4 + 16;
    o = (o + 127) / 128 * 128;
    scale_block = (scale_block + 127) / 128 * 128;
    sa.off_scales = o; sa.scale_block_bytes = scale_block; o += 2 * scale_block;
    o = (o + 127) / 128 * 128;
    sa.off_stages = o; sa.slot_bytes = slot_bytes;
    int nslots = (max_smem - o - 256) / slot_bytes;
    if (nslots > 12) nslots = 12;
    if (nslots < 3) return (int)cudaErrorInvalidValue;
    sa.nslots = nslots; o += nslots * slot_bytes;
    sa.off_bars = o; o += (2 * nslots + 5) * 8;
    sa.smem_bytes = o;
    sa.hd = hd;
    return 0;
}

template <int Q>
static int launch_step_q(const StepArgs& sa, int grid, const LaunchCfg& cfg) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel<Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, sa.smem_bytes);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid); lc.blockDim = dim3(kGemvThreads); lc.dynamicSmemBytes = sa.smem_bytes; lc.stream = cfg.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident at once: they wait for one another
    at[0].val.cooperative = 1;
    lc.attrs = at; lc.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&lc, decode_step_kernel<Q>, sa);
}

int launch_decode_step(int quant, const StepArgs& sa, int grid, const LaunchCfg& cfg) {
    if (grid < 1 || grid > cfg.sm_count) return (int)cudaErrorInvalidValue;
    if (quant == Q_I4) return launch_step_q<Q_I4>(sa, grid, cfg);
    if (quant == Q_I8) return launch_step_q<Q_I8>(sa, grid, cfg);
    if (quant == Q_F16) return launch_step_q<Q_F16>(sa, grid, cfg);
    return (int)cudaErrorInvalidValue;
}

}  // namespace cq
