// Source-level compatibility layer: CuQwen's C++ host API (include/config.h:52-127, include/load_weights.h:17-60,
// include/model.cuh:9-60, include/kernels.cuh:19-160 of that project) expressed on top of the C ABI of
// libcuqwen_b200.so.  A program written against CuQwen's headers (its main.cu, its benchmarks) compiles against this
// one header instead and links -lcuqwen_b200; model and quantisation are still chosen with -DQWEN_MODEL_* / -DQUANT_*.
//
// What is kept: type, field, macro and function names and argument meaning; print-and-exit error behaviour.
// What differs: the engine owns every device buffer, so the structs hold BORROWED pointers (free_* release the engine,
// not individual tensors); the engine has its own stream and CUDA graph: qwen_forward is synchronous and ignores its
// `stream` argument, the launch_* wrappers order their work against the stream they are given (StreamScope); the knobs
// that tuned the reference kernels (ATTN_PARTITIONS, ...) exist as constants for harnesses that print them but tune nothing.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "cuqwen_b200.h"

constexpr int QUANT_GROUP_SIZE = 128;
#if defined(QUANT_INT8)
using qweight_t = int8_t;
#define QUANT_TAG "int8"
#define QUANT_TYPE_ID 1
#define QUANT_ENABLED
#define WEIGHT_ROW_STRIDE(cols) (cols)
#elif defined(QUANT_INT4)
using qweight_t = int8_t;           // two 4-bit weights per byte, low nibble = even column
#define QUANT_TAG "int4"
#define QUANT_TYPE_ID 2
#define QUANT_ENABLED
#define WEIGHT_ROW_STRIDE(cols) ((cols) / 2)
#else
using qweight_t = half;
#define QUANT_TAG "fp16"
#define QUANT_TYPE_ID 0
#define WEIGHT_ROW_STRIDE(cols) (cols)
#endif

#define CUDA_CHECK(call)                                                                                   \
    do {                                                                                                   \
        cudaError_t cuqwen_e_ = (call);                                                                    \
        if (cuqwen_e_ != cudaSuccess) {                                                                    \
            fprintf(stderr, "CUDA Error at %s:%d - %s\n", __FILE__, __LINE__, cudaGetErrorString(cuqwen_e_)); \
            exit(EXIT_FAILURE);                                                                            \
        }                                                                                                  \
    } while (0)

// model table: id in the C ABI, tag, display name, vocab, dim, intermediate, layers, heads, kv heads, head dim
#if defined(QWEN_MODEL_0_5B)
#define CUQWEN_ROW(X) X(CUQWEN_MODEL_0_5B, "0_5b", "0.5B", 151936, 896, 4864, 24, 14, 2, 64)
#elif defined(QWEN_MODEL_1_5B)
#define CUQWEN_ROW(X) X(CUQWEN_MODEL_1_5B, "1_5b", "1.5B", 151936, 1536, 8960, 28, 12, 2, 128)
#elif defined(QWEN_MODEL_3B)
#define CUQWEN_ROW(X) X(CUQWEN_MODEL_3B, "3b", "3B", 151936, 2048, 11008, 36, 16, 2, 128)
#elif defined(QWEN_MODEL_14B)
#define CUQWEN_ROW(X) X(CUQWEN_MODEL_14B, "14b", "14B", 152064, 5120, 13824, 48, 40, 8, 128)
#else   // QWEN_MODEL_7B, also the default
#define CUQWEN_ROW(X) X(CUQWEN_MODEL_7B, "7b", "7B", 152064, 3584, 18944, 28, 28, 4, 128)
#endif
#define CUQWEN_TAG_OF(id, tag, name, v, d, i, l, h, kv, hd) tag
#define MODEL_TAG CUQWEN_ROW(CUQWEN_TAG_OF)

struct QwenConfig {
    static constexpr int32_t magic = 0x5157454E;
#define CUQWEN_FIELDS(id, tag, name, v, d, i, l, h, kv, hd)                                                       \
    static constexpr int model_id = id;                                                                            \
    static constexpr const char* model_name = name;                                                               \
    static constexpr int32_t vocab_size = v, dim = d, intermediate_size = i, n_layers = l, n_heads = h, n_kv_heads = kv, head_dim = hd;
    CUQWEN_ROW(CUQWEN_FIELDS)
#undef CUQWEN_FIELDS
    static constexpr int32_t max_seq_len = 32768;
    static constexpr const char* bin_path = "weights/model_" QUANT_TAG "_" MODEL_TAG ".bin";
    static constexpr int32_t quant_type = QUANT_TYPE_ID;
    static constexpr float norm_eps = 1e-6f, rope_theta = 1000000.0f, repetition_penalty = 1.1f;
};

// tuning constants of the reference kernels (include/config.h:140-186), kept as names with the reference's values so
// that programs which size buffers or print them compile; this library's kernels choose their own launch shapes
constexpr int ATTN_PARTITIONS = 64, KSPLIT_WARPS = 8, PARTIAL_HEAD_SLOTS = 16, ARGMAX_BLOCKS = 128, ARGMAX_THREADS = 256;
constexpr int ATTN_KEYS_CAP = (((QwenConfig::max_seq_len + ATTN_PARTITIONS - 1) / ATTN_PARTITIONS) + 15) / 16 * 16;
constexpr int GEMV_WARPS_PER_BLOCK = 8;
constexpr int GEMV_WIDE_WARPS_PER_BLOCK = (QwenConfig::dim >= 4096) ? 32 : (QwenConfig::dim >= 3072) ? 16 : 8;

struct LayerWeights {
    half* input_layernorm_weight;
    qweight_t* q_proj_weight; half* q_proj_bias;
    qweight_t* k_proj_weight; half* k_proj_bias;
    qweight_t* v_proj_weight; half* v_proj_bias;
    qweight_t* o_proj_weight;
    half* post_attention_layernorm_weight;
    qweight_t *gate_proj_weight, *up_proj_weight, *down_proj_weight;
    half *q_proj_scale, *k_proj_scale, *v_proj_scale, *o_proj_scale, *gate_proj_scale, *up_proj_scale, *down_proj_scale;
};
struct QwenWeights {
    half* embed_tokens;
    std::vector<LayerWeights> layers;
    half* norm_weight;
    half* lm_head_weight;
    bool lm_head_quantized = false;
    int8_t* lm_head_q = nullptr;
    half* lm_head_scale = nullptr;
    cuqwen_engine* backend = nullptr;       // not in the reference: the engine that owns everything above
};
struct QwenState {
    half *x, *xb, *q, *k, *v, *att, *gate, *up, *mlp_out, *logits;
    int* d_sampled_token;
    int* d_history;
    half *key_cache, *value_cache;          // head-major [n_layers][n_kv_heads][max_seq_len][head_dim]
    float *d_partial_out, *d_partial_max, *d_partial_sum;
    int *d_token, *d_pos, *d_history_len;
    cudaStream_t stream;
    cudaGraph_t graph;
    cudaGraphExec_t graph_exec;
    bool graph_created;
    cuqwen_engine* backend;                 // not in the reference
};

namespace cuqwen_compat {
[[noreturn]] inline void die(const char* what) {
    fprintf(stderr, "%s: %s\n", what, cuqwen_last_error());
    exit(EXIT_FAILURE);
}
inline void* ptr_of(cuqwen_engine* e, int which, int layer = 0) {
    void* p = nullptr;
    size_t n = 0;
    if (cuqwen_get_ptr(e, which, layer, &p, &n)) die("cuqwen_get_ptr");
    return p;
}
inline cuqwen_engine*& current() { static cuqwen_engine* e = nullptr; return e; }
}  // namespace cuqwen_compat

inline QwenConfig load_weights(const std::string& bin_path, QwenWeights& w) {
    using namespace cuqwen_compat;
    cuqwen_params p;
    cuqwen_engine* e = nullptr;
    if (cuqwen_model_params(QwenConfig::model_id, QUANT_TYPE_ID, &p) || cuqwen_create(&p, &e)) die("Error");
    if (cuqwen_load(e, bin_path.c_str())) die("Error");                 // the message is the loader's own text
    w.backend = e; current() = e;
    w.embed_tokens = (half*)ptr_of(e, CUQWEN_PTR_EMBED);
    w.norm_weight = (half*)ptr_of(e, CUQWEN_PTR_NORM);
    const int kind = cuqwen_lm_head_kind(e);
    w.lm_head_quantized = kind == 1;
    w.lm_head_q = kind == 1 ? (int8_t*)ptr_of(e, CUQWEN_PTR_LM_HEAD) : nullptr;
    w.lm_head_scale = kind == 1 ? (half*)ptr_of(e, CUQWEN_PTR_LM_HEAD_SCALE) : nullptr;
    w.lm_head_weight = kind == 1 ? nullptr : (half*)ptr_of(e, CUQWEN_PTR_LM_HEAD);
    w.layers.resize(QwenConfig::n_layers);
    for (int l = 0; l < QwenConfig::n_layers; ++l) {
        LayerWeights& L = w.layers[l];
        L.input_layernorm_weight = (half*)ptr_of(e, CUQWEN_PTR_IN_NORM, l);
        L.q_proj_weight = (qweight_t*)ptr_of(e, CUQWEN_PTR_WQ, l); L.q_proj_scale = (half*)ptr_of(e, CUQWEN_PTR_SQ, l); L.q_proj_bias = (half*)ptr_of(e, CUQWEN_PTR_BQ, l);
        L.k_proj_weight = (qweight_t*)ptr_of(e, CUQWEN_PTR_WK, l); L.k_proj_scale = (half*)ptr_of(e, CUQWEN_PTR_SK, l); L.k_proj_bias = (half*)ptr_of(e, CUQWEN_PTR_BK, l);
        L.v_proj_weight = (qweight_t*)ptr_of(e, CUQWEN_PTR_WV, l); L.v_proj_scale = (half*)ptr_of(e, CUQWEN_PTR_SV, l); L.v_proj_bias = (half*)ptr_of(e, CUQWEN_PTR_BV, l);
        L.o_proj_weight = (qweight_t*)ptr_of(e, CUQWEN_PTR_WO, l); L.o_proj_scale = (half*)ptr_of(e, CUQWEN_PTR_SO, l);
        L.post_attention_layernorm_weight = (half*)ptr_of(e, CUQWEN_PTR_POST_NORM, l);
        L.gate_proj_weight = (qweight_t*)ptr_of(e, CUQWEN_PTR_WGATE, l); L.gate_proj_scale = (half*)ptr_of(e, CUQWEN_PTR_SGATE, l);
        L.up_proj_weight = (qweight_t*)ptr_of(e, CUQWEN_PTR_WUP, l); L.up_proj_scale = (half*)ptr_of(e, CUQWEN_PTR_SUP, l);
        L.down_proj_weight = (qweight_t*)ptr_of(e, CUQWEN_PTR_WDOWN, l); L.down_proj_scale = (half*)ptr_of(e, CUQWEN_PTR_SDOWN, l);
    }
    return QwenConfig{};
}
// The tensors belong to the engine; it is released with the state (free_qwen_state) or here when no state was made.
inline void free_weights(QwenWeights& w, const QwenConfig&) {
    if (w.backend && cuqwen_compat::current() == w.backend) { cuqwen_destroy(w.backend); cuqwen_compat::current() = nullptr; }
    w = QwenWeights{};
}

inline void malloc_qwen_state(const QwenConfig&, QwenState& s) {
    using namespace cuqwen_compat;
    cuqwen_engine* e = current();
    if (!e) { fprintf(stderr, "malloc_qwen_state: load_weights must come first\n"); exit(EXIT_FAILURE); }
    s = QwenState{};
    s.backend = e;
    s.x = (half*)ptr_of(e, CUQWEN_PTR_X); s.att = (half*)ptr_of(e, CUQWEN_PTR_XN); s.xb = (half*)ptr_of(e, CUQWEN_PTR_ATT);
    s.q = (half*)ptr_of(e, CUQWEN_PTR_Q); s.k = (half*)ptr_of(e, CUQWEN_PTR_K); s.v = (half*)ptr_of(e, CUQWEN_PTR_V);
    s.gate = (half*)ptr_of(e, CUQWEN_PTR_GATE); s.logits = (half*)ptr_of(e, CUQWEN_PTR_LOGITS);
    s.key_cache = (half*)ptr_of(e, CUQWEN_PTR_KEY_CACHE); s.value_cache = (half*)ptr_of(e, CUQWEN_PTR_VALUE_CACHE);
    s.d_history = (int*)ptr_of(e, CUQWEN_PTR_HISTORY);
    // the device ints of the step, the split-KV scratch and the two buffers the reference allocates without using them
    // (src/model.cu:18-20): all point at engine-owned memory, so a harness that pokes them finds valid addresses
    s.d_token = (int*)ptr_of(e, CUQWEN_PTR_TOKEN); s.d_pos = (int*)ptr_of(e, CUQWEN_PTR_POS);
    s.d_history_len = (int*)ptr_of(e, CUQWEN_PTR_HISTORY_LEN); s.d_sampled_token = (int*)ptr_of(e, CUQWEN_PTR_SAMPLED);
    s.d_partial_out = (float*)ptr_of(e, CUQWEN_PTR_PARTIAL_O);
    s.d_partial_max = (float*)ptr_of(e, CUQWEN_PTR_PARTIAL_ML); s.d_partial_sum = s.d_partial_max;   // (max, sum) pairs live in one buffer here
    s.up = (half*)ptr_of(e, CUQWEN_PTR_UP); s.mlp_out = (half*)ptr_of(e, CUQWEN_PTR_MLP_OUT);
    s.stream = (cudaStream_t)ptr_of(e, CUQWEN_PTR_STREAM);
}
inline void free_qwen_state(QwenState& s) {
    if (s.backend && cuqwen_compat::current() == s.backend) { cuqwen_destroy(s.backend); cuqwen_compat::current() = nullptr; }
    s = QwenState{};
}

// The reference runs the step on `stream` (or on state.stream when it is 0) and waits for it (src/model.cu:193-222).
// Here the step runs on the engine's own stream; work the caller queued on `stream` before the call is waited for
// first, and the call returns with the step complete, so the ordering a caller can observe is the same.
inline int qwen_forward(int token, int pos, const QwenConfig&, QwenState& s, const QwenWeights&, const int* h_history = nullptr,
                        int history_len = 0, cudaStream_t stream = 0) {
    int next = -1;
    if (stream != 0 && stream != s.stream && cudaStreamSynchronize(stream) != cudaSuccess) { fprintf(stderr, "qwen_forward: the caller's stream failed\n"); exit(EXIT_FAILURE); }
    if (cuqwen_step(s.backend, token, pos, h_history, history_len, &next)) cuqwen_compat::die("qwen_forward");
    return next;
}

// Not in the reference (its chat loop calls qwen_forward once per prompt token, src/main.cu:86-92): the cache rows
// [pos0, pos0 + n) of n prompt tokens in one batched pass.  Returns nothing to sample from - call qwen_forward on the
// prompt's last token afterwards (prefill the tokens before it).
inline void qwen_prefill(const int* tokens, int n, int pos0, const QwenConfig&, QwenState& s, const QwenWeights&) {
    if (n > 0 && cuqwen_prefill(s.backend, tokens, n, pos0)) cuqwen_compat::die("qwen_prefill");
}

// ---- the launch_* operators (device pointers in the reference's layouts; work is queued on the library's stream of
// device 0, cuqwen_dev_sync(0) waits for it; `stream` arguments are ignored) ----
#define CUQWEN_K(call) do { if (call) cuqwen_compat::die(#call); } while (0)
// The reference's launch_* are ordered on the stream they are given.  The library queues on a stream of its own, so
// every wrapper below brackets its call: on entry the library's stream waits for what the caller's stream holds, on
// exit the caller's stream waits for the work just queued (cuqwen_dev_join).  Events, copies and synchronisation on
// the caller's stream then mean what they mean with the reference.
namespace cuqwen_compat {
struct StreamScope {
    cudaStream_t s;
    explicit StreamScope(cudaStream_t st) : s(st) { if (cuqwen_dev_join(0, (void*)s, 0)) die("cuqwen_dev_join"); }
    ~StreamScope() { cuqwen_dev_join(0, (void*)s, 1); }
};
}  // namespace cuqwen_compat
inline void launch_embedding_lookup(const half* table, const int* d_token_id, half* out, int dim, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_embedding(0, table, d_token_id, out, dim));
}
inline void launch_rmsnorm(const half* x, const half* norm_weight, half* out, int dim, half eps, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_rmsnorm(0, x, norm_weight, out, dim, __half2float(eps)));
}
inline void launch_kv_cache_store(const half* k, const half* v, half* kcache, half* vcache, const int* d_pos, int n_kv_heads, int max_seq, int head_dim,
                                  cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_kv_store(0, k, v, kcache, vcache, d_pos, n_kv_heads, max_seq, head_dim));
}
inline void launch_gemv_add_fp16(const qweight_t* w, const half* scale, const half* in, half* x_inout, int rows, int cols, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_gemv_add(0, QUANT_TYPE_ID, w, scale, in, x_inout, rows, cols));
}
inline void launch_fused_mlp_stage2(half* x, const qweight_t* down_weight, const half* down_scale, const half* intermediate_in, int dim, int inter_dim,
                                    cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_gemv_add(0, QUANT_TYPE_ID, down_weight, down_scale, intermediate_in, x, dim, inter_dim));
}
// norm_weight / eps are accepted and, as in the reference (src/kernels.cu:578), ignored: x arrives normalised
inline void launch_fused_mlp_stage1(const half* x, const half* /*norm_weight*/, const qweight_t* gate_weight, const qweight_t* up_weight, const half* gate_scale,
                                    const half* up_scale, half* intermediate_out, int dim, int inter_dim, half /*eps*/, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_mlp1(0, QUANT_TYPE_ID, x, nullptr, 0.f, gate_weight, up_weight, gate_scale, up_scale, intermediate_out, dim, inter_dim));
}
// q/k/v projections + bias + RoPE; norm_weight / eps ignored as in the reference (src/kernels.cu:502)
inline void launch_fused_attn_block(const half* x, const half* /*norm_weight*/, const qweight_t* W_q, const qweight_t* W_k, const qweight_t* W_v,
                                    const half* W_q_scale, const half* W_k_scale, const half* W_v_scale, const half* b_q, const half* b_k, const half* b_v,
                                    half* q_out, half* k_out, half* v_out, int dim, int /*q_dim*/, int /*kv_dim*/, int n_heads, int n_kv_heads, int head_dim,
                                    const int* d_pos, float rope_theta, half /*eps*/, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_qkv(0, QUANT_TYPE_ID, x, nullptr, 0.f, W_q, W_k, W_v, W_q_scale, W_k_scale, W_v_scale, b_q, b_k, b_v, q_out, k_out, v_out, nullptr, nullptr,
                          dim, n_heads, n_kv_heads, head_dim, QwenConfig::max_seq_len, d_pos, rope_theta, 1));
}
// The partial buffers of the reference are not used: this library keeps its own scratch per (device, shape).
inline void launch_gqa_attention_decode(const half* q, const half* key_cache, const half* value_cache, half* attn_out, const int* d_pos, int n_heads,
                                        int n_kv_heads, int head_dim, int max_seq_len, float* /*d_partial_out*/, float* /*d_partial_max*/,
                                        float* /*d_partial_sum*/, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    static void *so = nullptr, *sml = nullptr, *cnt = nullptr;
    static size_t have[3] = {0, 0, 0};
    static int sms = 0;
    if (!sms && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0) != cudaSuccess) sms = 128;
    const int splits = sms / n_kv_heads > 128 ? 128 : sms / n_kv_heads < 1 ? 1 : sms / n_kv_heads;
    size_t need[3];
    CUQWEN_K(cuqwen_attn_scratch_bytes(n_kv_heads, head_dim, splits, &need[0], &need[1], &need[2]));
    if (need[0] > have[0] || need[1] > have[1] || need[2] > have[2]) {
        if (so) { cuqwen_dev_free(0, so); cuqwen_dev_free(0, sml); cuqwen_dev_free(0, cnt); }
        CUQWEN_K(cuqwen_dev_alloc(0, need[0], &so)); CUQWEN_K(cuqwen_dev_alloc(0, need[1], &sml)); CUQWEN_K(cuqwen_dev_alloc(0, need[2], &cnt));
        CUQWEN_K(cuqwen_dev_memset(0, cnt, 0, need[2]));
        have[0] = need[0]; have[1] = need[1]; have[2] = need[2];
    }
    CUQWEN_K(cuqwen_k_attention(0, q, key_cache, value_cache, attn_out, d_pos, n_heads, n_kv_heads, head_dim, max_seq_len, splits, so, sml, cnt));
}
inline void launch_apply_repetition_penalty(half* logits, const int* d_history, const int* d_history_len, int vocab_size, half penalty, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    static void* bitmap = nullptr;
    static int have = 0;
    if (vocab_size > have) {
        if (bitmap) cuqwen_dev_free(0, bitmap);
        CUQWEN_K(cuqwen_dev_alloc(0, (size_t)(vocab_size + 31) / 32 * 4, &bitmap));
        CUQWEN_K(cuqwen_dev_memset(0, bitmap, 0, (size_t)(vocab_size + 31) / 32 * 4));
        have = vocab_size;
    }
    CUQWEN_K(cuqwen_k_penalty(0, logits, d_history, d_history_len, vocab_size, __half2float(penalty), bitmap));
}
inline void launch_argmax(const half* logits, int* d_sampled_token, int vocab_size, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    static void* scratch = nullptr;
    if (!scratch) { CUQWEN_K(cuqwen_dev_alloc(0, 16, &scratch)); CUQWEN_K(cuqwen_dev_memset(0, scratch, 0, 16)); }
    CUQWEN_K(cuqwen_k_argmax(0, logits, d_sampled_token, vocab_size, scratch));
}
inline void launch_compute_logits(const half* x_normed, const half* lm_head_weight, half* logits, int vocab_size, int dim, cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_gemv(0, CUQWEN_FP16, lm_head_weight, nullptr, x_normed, nullptr, 0.f, logits, vocab_size, dim));
}
inline void launch_compute_logits_int8(const half* x_normed, const int8_t* lm_head_w, const half* lm_head_scale, half* logits, int vocab_size, int dim,
                                       cudaStream_t stream = 0) {
    cuqwen_compat::StreamScope scope_(stream);
    CUQWEN_K(cuqwen_k_gemv(0, CUQWEN_INT8, lm_head_w, lm_head_scale, x_normed, nullptr, 0.f, logits, vocab_size, dim));
}
#undef CUQWEN_K
