// Split-KV FlashDecoding for one query token over the fp16 head-major KV cache [n_kv][max_seq][hd] (reference
// layout, include/model.cuh:25), all query heads of a KV head processed together so K and V are read once per group.
//
// Reference behaviour being replaced: src/kernels.cu:105-219 (stage 1, 64 fixed partitions, WMMA) and :222-288
// (stage 2 combine).  Here scores and the softmax stay in fp32 (the reference rounds scores to fp16).
//
// This header holds the argument block and the stage geometry.  The kernels are in attn_split.cuh (two launches:
// partials, then a per-head fold); the arithmetic of a key tile is in attn_tile.cuh.
//
// Scratch (sizes from attn_slots / attn_counters in attn_combine.cuh): part_o [slots][8][hd] fp32, part_ml
// [slots][8][2] fp32; slot [kvh][split] receives the partial of one key range.  `counters` is kept in the interface
// for callers that size it, and is left untouched (zero).
#pragma once
#include "attn_tile.cuh"
#include "tma.cuh"

namespace cq {

constexpr int kAttnStageKeys = 64;     // keys per ring stage (K half, then V half): four 16-key tiles

struct AttnArgs {
    const __half* q;        // [n_kv*grp][hd]
    const __half* kc;       // [n_kv][max_seq][hd]
    const __half* vc;
    __half* out;            // [n_kv*grp][hd]
    const int* d_pos;       // attends to keys [0, *d_pos]
    int n_kv, grp, max_seq, nsplit;
    float scale_log2;       // (1/sqrt(hd)) * log2(e)
    float* part_o;
    float* part_ml;
    unsigned* counters;
    unsigned* err;          // receives a non-zero code when a bounded wait expires (may be null)
    int stages;             // ring depth of the partial kernel (0 = its default)
    unsigned long long* trace;       // optional: timeline words of the partial launch and of the fold launch, else null
    // 8-bit cache (attn_partial_kernel<HD, true>): kc / vc point at int8 rows [n_kv][max_seq][hd], one fp32 scale per
    // cached row and KV head in kscale / vscale [n_kv][max_seq]; a row is  value = int8 * scale, scale = max|row| / 127.
    // The step's own key and value are not in the cache yet: they arrive in fp16 (k_cur / v_cur, [n_kv][hd]), are
    // attended to in fp16, and the kernel stores their 8-bit form into row *d_pos for the steps to come.
    float* kscale;
    float* vscale;
    const __half* k_cur;
    const __half* v_cur;
    // Hand-over to a quantised o_proj (head_dim 128 only: a head is then exactly one 128-column scale group): besides
    // the fp16 output the fold also writes it in the staged form a quantised GEMV's inner loop reads (digit blocks,
    // corrections, scales: gemv_stage.cuh), so that the o_proj CTAs fetch it with three bulk copies instead of each
    // converting the whole vector again.  quant_out: the consumer's weight format (Q_I4 / Q_I8); null = no hand-over.
    unsigned char* xd_out;
    int* corr_out;
    float* xscale_out;
    int quant_out;
};

}  // namespace cq
