// extern "C" shim around the UNMODIFIED CuQwen sources.  TEST / BASELINE
// INFRASTRUCTURE ONLY: it is compiled together with the reference's own
// src/kernels.cu, src/model.cu and src/load_weights.cpp (read where they lie,
// never copied) by oracle/build_ref.py, once per (model, quantisation) because
// the reference selects both at compile time.  The resulting library lets the
// GPU parity tests and the benchmark's reference arm call the reference's
// launch_* operators and its qwen_forward through plain C symbols.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <iostream>
#include <sstream>
#include <string>

#include "model.cuh"      // reference header (include path supplied by the build recipe)
#include "rng.cuh"        // this repository's counter-based N(0,1) fill, so both engines see identical KV data

struct RefModel {
    QwenWeights w;
    QwenState s;
    QwenConfig c;
    cudaEvent_t e0, e1;
};

extern "C" {

// dims of the compiled-in configuration: vocab, dim, inter, layers, heads, kv, hd, max_seq, quant, lm_head_quantised(-1 until loaded)
void ref_info(int* out10) {
    QwenConfig c;
    int v[10] = {c.vocab_size, c.dim, c.intermediate_size, c.n_layers, c.n_heads, c.n_kv_heads, c.head_dim, c.max_seq_len, c.quant_type, -1};
    for (int i = 0; i < 10; ++i) out10[i] = v[i];
}
int ref_sync(void) { return (int)cudaDeviceSynchronize(); }

// ---- operators ----
void ref_embedding(const void* table, const int* d_token, void* out, int dim) { launch_embedding_lookup((const half*)table, d_token, (half*)out, dim, 0); }
void ref_rmsnorm(const void* x, const void* w, void* out, int dim, float eps) { launch_rmsnorm((const half*)x, (const half*)w, (half*)out, dim, __float2half(eps), 0); }
void ref_qkv(const void* x, const void* wq, const void* wk, const void* wv, const void* sq, const void* sk, const void* sv,
             const void* bq, const void* bk, const void* bv, void* q, void* k, void* v, int dim, int n_heads, int n_kv, int hd,
             const int* d_pos, float theta) {
    launch_fused_attn_block((const half*)x, nullptr, (const qweight_t*)wq, (const qweight_t*)wk, (const qweight_t*)wv, (const half*)sq, (const half*)sk,
                            (const half*)sv, (const half*)bq, (const half*)bk, (const half*)bv, (half*)q, (half*)k, (half*)v, dim, n_heads * hd, n_kv * hd,
                            n_heads, n_kv, hd, d_pos, theta, __float2half(1e-6f), 0);
}
void ref_kv_store(const void* k, const void* v, void* kc, void* vc, const int* d_pos, int n_kv, int max_seq, int hd) {
    launch_kv_cache_store((const half*)k, (const half*)v, (half*)kc, (half*)vc, d_pos, n_kv, max_seq, hd, 0);
}
// partial buffers sized as src/model.cu:40-43 does: n_kv * 16 * 64 * (hd | 1 | 1) floats
void ref_attention(const void* q, const void* kc, const void* vc, void* out, const int* d_pos, int n_heads, int n_kv, int hd, int max_seq,
                   float* po, float* pm, float* ps) {
    launch_gqa_attention_decode((const half*)q, (const half*)kc, (const half*)vc, (half*)out, d_pos, n_heads, n_kv, hd, max_seq, po, pm, ps, 0);
}
void ref_gemv_add(const void* w, const void* s, const void* in, void* x, int rows, int cols) {
    launch_gemv_add_fp16((const qweight_t*)w, (const half*)s, (const half*)in, (half*)x, rows, cols, 0);
}
void ref_mlp1(const void* x, const void* wg, const void* wu, const void* sg, const void* su, void* out, int dim, int inter) {
    launch_fused_mlp_stage1((const half*)x, nullptr, (const qweight_t*)wg, (const qweight_t*)wu, (const half*)sg, (const half*)su, (half*)out, dim, inter,
                            __float2half(1e-6f), 0);
}
void ref_mlp2(void* x, const void* wd, const void* sd, const void* in, int dim, int inter) {
    launch_fused_mlp_stage2((half*)x, (const qweight_t*)wd, (const half*)sd, (const half*)in, dim, inter, 0);
}
void ref_logits(const void* xn, const void* w, void* logits, int vocab, int dim) { launch_compute_logits((const half*)xn, (const half*)w, (half*)logits, vocab, dim, 0); }
void ref_logits_int8(const void* xn, const void* w, const void* s, void* logits, int vocab, int dim) {
    launch_compute_logits_int8((const half*)xn, (const int8_t*)w, (const half*)s, (half*)logits, vocab, dim, 0);
}
void ref_penalty(void* logits, const int* hist, const int* d_len, int vocab, float pen) {
    launch_apply_repetition_penalty((half*)logits, hist, d_len, vocab, __float2half(pen), 0);
}
void ref_argmax(const void* logits, int* d_out, int vocab) { launch_argmax((const half*)logits, d_out, vocab, 0); }

// ---- timing loops in C (CUDA events around `iters` launches on the default stream), for the kernel-level baselines ----
// attention: rotates over n_copies (key, value) cache pairs so that the bytes come from HBM rather than L2
float ref_bench_attention(const void* q, void* const* kcs, void* const* vcs, int n_copies, void* out, const int* d_pos, int n_heads, int n_kv, int hd,
                          int max_seq, float* po, float* pm, float* ps, int iters) {
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < 3; ++i)
        launch_gqa_attention_decode((const half*)q, (const half*)kcs[i % n_copies], (const half*)vcs[i % n_copies], (half*)out, d_pos, n_heads, n_kv, hd, max_seq, po, pm, ps, 0);
    cudaEventRecord(e0, 0);
    for (int i = 0; i < iters; ++i)
        launch_gqa_attention_decode((const half*)q, (const half*)kcs[i % n_copies], (const half*)vcs[i % n_copies], (half*)out, d_pos, n_heads, n_kv, hd, max_seq, po, pm, ps, 0);
    cudaEventRecord(e1, 0); cudaEventSynchronize(e1);
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    return ms / iters;
}
// x += W . in over n_copies weight copies (a pure GEMV when x starts at zero: src/kernels.cu:674-687)
float ref_bench_gemv_add(void* const* ws, void* const* ss, int n_copies, const void* in, void* x, int rows, int cols, int iters) {
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < 3; ++i) launch_gemv_add_fp16((const qweight_t*)ws[i % n_copies], (const half*)ss[i % n_copies], (const half*)in, (half*)x, rows, cols, 0);
    cudaEventRecord(e0, 0);
    for (int i = 0; i < iters; ++i) launch_gemv_add_fp16((const qweight_t*)ws[i % n_copies], (const half*)ss[i % n_copies], (const half*)in, (half*)x, rows, cols, 0);
    cudaEventRecord(e1, 0); cudaEventSynchronize(e1);
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    return ms / iters;
}

// ---- whole model ----
void* ref_model_load(const char* path) {
    std::ostringstream sink;
    std::streambuf* old = std::cout.rdbuf(sink.rdbuf());     // the loader narrates on stdout
    RefModel* m = new RefModel();
    m->c = load_weights(std::string(path), m->w);
    malloc_qwen_state(m->c, m->s);
    std::cout.rdbuf(old);
    cudaEventCreate(&m->e0); cudaEventCreate(&m->e1);
    return m;
}
int ref_lm_head_quantized(void* h) { return ((RefModel*)h)->w.lm_head_quantized ? 1 : 0; }
int ref_forward(void* h, int token, int pos, const int* hist, int hist_len) {
    RefModel* m = (RefModel*)h;
    return qwen_forward(token, pos, m->c, m->s, m->w, hist, hist_len, 0);
}
// n greedy steps, each through qwen_forward (the reference has no other way to decode); returns elapsed ms
float ref_decode_n(void* h, int first_token, int start_pos, int n, int* out_tokens) {
    RefModel* m = (RefModel*)h;
    int tok = first_token;
    cudaEventRecord(m->e0, m->s.stream);
    for (int i = 0; i < n; ++i) { tok = qwen_forward(tok, start_pos + i, m->c, m->s, m->w, nullptr, 0, 0); if (out_tokens) out_tokens[i] = tok; }
    cudaEventRecord(m->e1, m->s.stream);
    cudaEventSynchronize(m->e1);
    float ms = 0; cudaEventElapsedTime(&ms, m->e0, m->e1);
    return ms;
}
void ref_kv_fill_normal(void* h, int ctx_len, unsigned long long seed) {
    RefModel* m = (RefModel*)h;
    const size_t head_stride = (size_t)m->c.max_seq_len * m->c.head_dim;
    for (int l = 0; l < m->c.n_layers; ++l)
        for (int hh = 0; hh < m->c.n_kv_heads; ++hh) {
            const size_t off = ((size_t)l * m->c.n_kv_heads + hh) * head_stride, n = (size_t)ctx_len * m->c.head_dim;
            int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192); if (blocks < 1) blocks = 1;
            cq::fill_normal_kernel<<<blocks, 256>>>(m->s.key_cache + off, n, seed * 2 + 0, off);
            cq::fill_normal_kernel<<<blocks, 256>>>(m->s.value_cache + off, n, seed * 2 + 1, off);
        }
    cudaDeviceSynchronize();
}
// 0 logits, 1 key_cache, 2 value_cache, 3 x, 4 q, 5 k, 6 v, 7 xb (attention output), 8 gate
void* ref_state_ptr(void* h, int which) {
    RefModel* m = (RefModel*)h;
    switch (which) {
        case 0: return m->s.logits; case 1: return m->s.key_cache; case 2: return m->s.value_cache; case 3: return m->s.x;
        case 4: return m->s.q; case 5: return m->s.k; case 6: return m->s.v; case 7: return m->s.xb; case 8: return m->s.gate;
    }
    return nullptr;
}
void ref_model_free(void* h) {
    RefModel* m = (RefModel*)h;
    free_qwen_state(m->s); free_weights(m->w, m->c);
    delete m;
}

}  // extern "C"
