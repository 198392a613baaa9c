// Batched prefill: argument blocks and launchers of the attention and row-wise kernels (prefill_attn.cu); the GEMM is in
// prefill_gemm.cuh.  The reference prefills one token at a time through the decode path (src/main.cu:86-92).
#pragma once
#include "tma.cuh"

namespace cq {

struct PfAttnArgs {
    const __half* q;          // [T][ldq], post-RoPE; head h at columns [h * hd, h * hd + hd)
    const __half* kc;         // this layer's caches [n_kv][max_seq][hd]; rows pos0 .. pos0 + T - 1 already hold the tile's keys
    const __half* vc;
    __half* out;              // [T][ldq]
    int T, pos0, n_heads, grp, max_seq, ldq;      // grp = query heads per KV head
    float scale_log2;         // log2(e) / sqrt(hd)
};
int launch_prefill_attn(int head_dim, const PfAttnArgs& a, cudaStream_t stream);          // mma.sync, head_dim 64 / 128
// tcgen05 kernel, head_dim 64 / 128; kc / vc must be the caches' [n_kv][max_seq][head_dim] base.  *err receives a code when a bounded wait expires.
int launch_prefill_attn_tc(int head_dim, const PfAttnArgs& a, int n_kv, unsigned* err, cudaStream_t stream);

struct PfRopeArgs {
    const float* qkv;         // [T][q_dim + 2 kv_dim] fp32 sums
    const __half *bq, *bk, *bv;
    __half* q_out;            // [T][q_dim]
    __half *kcache, *vcache;  // this layer's [n_kv][max_seq][hd]
    int pos0, n_heads, n_kv, hd, q_dim, kv_dim, max_seq, rope_fast;
    float theta;
};
int launch_pf_embed(const __half* table, const int* d_tokens, __half* x, int T, int dim, cudaStream_t s);
int launch_pf_rmsnorm(const __half* x, const __half* w, __half* out, int T, int dim, float eps, cudaStream_t s);
int launch_pf_rope_kv(const PfRopeArgs& a, int T, cudaStream_t s);

}  // namespace cq
