// Tensor-parallel partition of one Qwen2.5 decoder across `size` GPUs of a box.
// Pure host arithmetic (no CUDA), shared by the loader and the step builder.
//
// Column-parallel (output rows split): q/k/v, gate/up, lm_head.  Row-parallel
// (input columns split, fp32 partial sums reduced across ranks): o_proj, down.
// Splits fall on whole query heads, whole 128-column scale groups and whole
// 16-row tiles, so no scale group is ever shared by two ranks; where the count
// does not divide evenly the shares differ by one unit.  With more ranks than KV
// heads, the ranks that share a KV head split its query heads between them and
// each keeps a full copy of that head's K/V rows.
#pragma once

namespace cq {

struct TpPlan {
    int qh0, qh1;      // global query-head range of this rank
    int kvh0, kvh1;    // global KV-head range stored (and attended) on this rank
    int grp;           // query heads per KV head on this rank
    int i0, i1;        // intermediate (MLP) channel range
    int v0, v1;        // vocabulary row range
};

// Returns 0 on success, non-zero when the model cannot be split this way.
inline int tp_plan(int n_heads, int n_kv, int head_dim, int inter, int vocab, int rank, int size, TpPlan* p) {
    if (size < 1 || rank < 0 || rank >= size || n_kv < 1 || n_heads % n_kv) return 1;
    const int grp = n_heads / n_kv;
    if (size <= n_kv) {
        if (n_kv % size) return 2;
        const int per = n_kv / size;
        p->kvh0 = rank * per; p->kvh1 = p->kvh0 + per;
        p->qh0 = p->kvh0 * grp; p->qh1 = p->kvh1 * grp;
        p->grp = grp;
    } else {
        if (size % n_kv) return 3;
        const int rp = size / n_kv, kv = rank / rp, sub = rank % rp;
        const int a = grp * sub / rp, b = grp * (sub + 1) / rp;
        if (b <= a) return 4;
        p->kvh0 = kv; p->kvh1 = kv + 1;
        p->qh0 = kv * grp + a; p->qh1 = kv * grp + b;
        p->grp = b - a;
    }
    if (((p->qh0 * head_dim) % 128) || ((p->qh1 * head_dim) % 128)) return 5;   // o_proj slice must hold whole scale groups
    if (inter % 128 || vocab % 16) return 6;
    const long long G = inter / 128, U = vocab / 16;
    p->i0 = (int)(G * rank / size) * 128; p->i1 = (int)(G * (rank + 1) / size) * 128;
    p->v0 = (int)(U * rank / size) * 16;  p->v1 = (int)(U * (rank + 1) / size) * 16;
    if (p->i1 <= p->i0 || p->v1 <= p->v0) return 7;
    return 0;
}

}  // namespace cq
