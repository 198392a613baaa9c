/*
 * C ABI of libcuqwen_b200.so: a B200 (sm_100a) batch-1 decode engine for the
 * Qwen2.5 family that is a drop-in for CuQwen's weight file format, model
 * table and host API.  Plain pointers and sizes only; every function returns a
 * status code (0 = ok) instead of exiting the process, and a message for the
 * last failure of the calling thread is available from cuqwen_last_error().
 *
 * Each entry point names the CuQwen interface it stands in for
 * (file:line within that project).  Device pointers are marked "dev".
 */
#ifndef CUQWEN_B200_H
#define CUQWEN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cuqwen_engine cuqwen_engine;

enum {
    CUQWEN_OK = 0,
    CUQWEN_ERR_ARG = 1,       /* bad argument / unsupported shape */
    CUQWEN_ERR_IO = 2,        /* file cannot be opened / short read / truncated tensor data */
    CUQWEN_ERR_MAGIC = 3,     /* header magic is not 0x5157454E */
    CUQWEN_ERR_DIMS = 4,      /* header dims differ from the engine's configuration */
    CUQWEN_ERR_QUANT = 5,     /* header quantisation differs from the engine's configuration */
    CUQWEN_ERR_CUDA = 6,
    CUQWEN_ERR_NCCL = 7,
    CUQWEN_ERR_STATE = 8,     /* call made in the wrong order (e.g. step before load) */
    CUQWEN_ERR_TIMEOUT = 9    /* a bounded device-side wait expired */
};

enum { CUQWEN_FP16 = 0, CUQWEN_INT8 = 1, CUQWEN_INT4 = 2 };          /* include/config.h:18-32 QUANT_TYPE_ID */

/* Rows of the model table, include/config.h:55-113. */
enum { CUQWEN_MODEL_0_5B = 0, CUQWEN_MODEL_1_5B = 1, CUQWEN_MODEL_3B = 2, CUQWEN_MODEL_7B = 3, CUQWEN_MODEL_14B = 4, CUQWEN_MODEL_CUSTOM = -1 };

enum {
    CUQWEN_FLAG_ACCURATE_ROPE = 1,  /* accurate pow/sin/cos instead of the fast-math forms the reference build uses */
    CUQWEN_FLAG_NO_PDL = 2,         /* plain stream order between kernels (no programmatic dependent launch) */
    CUQWEN_FLAG_NO_GRAPH = 4,       /* launch the step kernel by kernel instead of replaying a CUDA graph */
    /* 8 is unused (it selected a persistent one-launch step kernel that was removed: it never beat the launch chain) */
    CUQWEN_FLAG_STEP_TRACE = 16,    /* profiling: every GEMV / attention launch of a step stamps its timeline (CUQWEN_PTR_STEP_TRACE) */
    CUQWEN_FLAG_TP_NCCL = 32,       /* tensor parallel: sum the row-parallel partials with NCCL all-reduce calls instead of peer stores */
    CUQWEN_FLAG_NO_HANDOVER = 64,   /* o_proj and the down projection convert their input themselves instead of taking it staged from the attention fold / the SwiGLU kernel */
    CUQWEN_FLAG_PREFILL_ATTN_MMA = 512, /* cuqwen_prefill: attention on the mma.sync kernel also where head_dim is 128 (comparison variant) */
    CUQWEN_FLAG_TP_SUM_IN_GEMV = 256, /* tensor parallel, peer-store exchange: no separate sum kernel; every CTA of the GEMV that consumes the
                                     * vector adds the ranks' partials while it stages its input (comparison variant, measured slower) */
    CUQWEN_FLAG_KV_INT8 = 128       /* opt-in, outside the parity contract (the reference keeps fp16, its roadmap names this: README.md:147):
                                     * the KV cache holds int8 rows with one fp32 scale per token and KV head (scale = max|row| / 127), which
                                     * halves the bytes attention streams; the step's own key and value are still attended to in fp16 */
};

/* Mirrors QwenConfig (include/config.h:52-127) as run-time data. */
typedef struct cuqwen_params {
    int32_t model_id;        /* CUQWEN_MODEL_*; CUSTOM uses the explicit dims below */
    int32_t vocab_size, dim, intermediate_size, n_layers, n_heads, n_kv_heads, head_dim;
    int32_t max_seq_len;     /* KV rows per head; 0 = 32768 (include/config.h:65) */
    int32_t quant;           /* CUQWEN_FP16 / INT8 / INT4 */
    int32_t device;          /* CUDA device ordinal */
    int32_t tp_rank, tp_size;/* tensor-parallel position; tp_size 0 or 1 = single GPU */
    int32_t attn_splits;     /* split-KV CTAs per KV head; 0 = choose from the SM count */
    uint32_t flags;
    float norm_eps, rope_theta, repetition_penalty;   /* 0 = 1e-6, 1e6, 1.1 (include/config.h:124-126) */
} cuqwen_params;

/* Fill `p` from the model table.  Replaces the -Dmodel/-Dquant compile-time selection (CMakeLists.txt:18-82). */
int cuqwen_model_params(int model_id, int quant, cuqwen_params* p);

/* malloc_qwen_state (src/model.cu:5-44): activations, KV cache, scratch, stream. */
int cuqwen_create(const cuqwen_params* p, cuqwen_engine** out);
/* free_qwen_state + free_weights (src/model.cu:46-74, src/load_weights.cpp:167-200). */
void cuqwen_destroy(cuqwen_engine* e);

/* load_weights (src/load_weights.cpp:36-165): same file format, same validation; returns a code instead of exit(). */
int cuqwen_load(cuqwen_engine* e, const char* bin_path);

/* qwen_forward (src/model.cu:183-223): one decode step; host token in, host token out, synchronous.  Token and
 * position travel through a pinned host mailbox that the step's kernels read and write themselves (no copy call, no
 * stream synchronisation; the reference pays three copies and a synchronisation per token, src/model.cu:193-222). */
int cuqwen_step(cuqwen_engine* e, int token, int pos, const int* history, int history_len, int* out_token);

/* The reference's host loop (src/main.cu:95-112) as one call: n times cuqwen_step with history_len 0, every sampled
 * token returning to the host before it is fed to the next step (unlike cuqwen_decode_n below). */
int cuqwen_step_loop(cuqwen_engine* e, int first_token, int start_pos, int n, int* out_tokens);

/* n greedy steps with the sampled token fed back on the device (no counterpart in the reference, which pays
 * a host round trip per token, src/main.cu:95-112).  out_tokens receives n ids.  history_len = 0 semantics. */
int cuqwen_decode_n(cuqwen_engine* e, int first_token, int start_pos, int n, int* out_tokens);
/* Batched prefill (no counterpart in the reference: src/main.cu:86-92 calls qwen_forward once per prompt token and
 * throws the logits away; README.md:145 lists the batched form as future work).  Runs n_tokens prompt tokens
 * (host array) through every layer as 128-token tiles - tcgen05 GEMMs over the quantised weights, causal attention
 * over the cache - and leaves their keys and values in cache rows [pos0, pos0 + n_tokens), as n_tokens calls of
 * cuqwen_step at positions pos0.. would.  Produces no logits: feed the prompt's last token to cuqwen_step
 * afterwards (prefill the tokens before it).  One GPU, fp16 KV cache, head_dim 64 or 128.  The device time is
 * readable through cuqwen_last_decode_ms. */
int cuqwen_prefill(cuqwen_engine* e, const int* tokens, int n_tokens, int pos0);
/* Milliseconds the device spent in the last cuqwen_decode_n (CUDA events around the n graph launches). */
float cuqwen_last_decode_ms(const cuqwen_engine* e);

/* Benchmark / test hook: fill K and V of every layer for positions [0, ctx_len) with N(0,1) fp16 values that
 * depend only on (seed, layer, global kv head, position, d).  Stands in for the prefill the reference benchmark
 * skips (benchmark/cuqwen_benchmark.cu:57-62). */
int cuqwen_kv_fill_normal(cuqwen_engine* e, int ctx_len, uint64_t seed);

/* Tensor-parallel set-up.  nccl_unique_id: the 128 bytes of an ncclUniqueId created by rank 0 and broadcast by
 * the host program.  Must be called on every rank after cuqwen_create. */
int cuqwen_tp_init(cuqwen_engine* e, const void* nccl_unique_id, size_t id_bytes);
int cuqwen_nccl_unique_id(void* out, size_t cap);
/* The partition cuqwen_create applies for (tp_rank, tp_size): out9 = {q_head0, q_head1, kv_head0, kv_head1,
 * q_heads_per_kv_head, inter0, inter1, vocab0, vocab1} (half-open global ranges).  Pure host arithmetic. */
int cuqwen_tp_plan(int n_heads, int n_kv_heads, int head_dim, int intermediate_size, int vocab_size, int rank, int size, int* out9);

/* Device pointers of engine-owned buffers, for harnesses that poke state directly the way the reference's do
 * (QwenState / QwenWeights fields, include/model.cuh:9-46, include/load_weights.h:17-54). */
enum {
    CUQWEN_PTR_X = 0, CUQWEN_PTR_XN, CUQWEN_PTR_Q, CUQWEN_PTR_K, CUQWEN_PTR_V, CUQWEN_PTR_ATT, CUQWEN_PTR_GATE,
    CUQWEN_PTR_LOGITS, CUQWEN_PTR_KEY_CACHE, CUQWEN_PTR_VALUE_CACHE, CUQWEN_PTR_HISTORY,
    CUQWEN_PTR_STEP_TRACE,          /* u64 [launch][8] nanosecond stamps merged over CTAs with atomic max, launch = position in the step (0 = the
                                     * embedding copy, then 6 per layer, then the lm_head): ~first CTA start, last CTA start, ~first dependency
                                     * wait returned, last input staged, last main loop done, last exit, 2 spare ("~" = stored complemented).
                                     * Stamps accumulate: zero the block between steps. */
    CUQWEN_PTR_TOKEN, CUQWEN_PTR_POS, CUQWEN_PTR_HISTORY_LEN, CUQWEN_PTR_SAMPLED,   /* the four device ints a step reads / writes (QwenState::d_token, d_pos, d_history_len, d_sampled_token) */
    CUQWEN_PTR_PARTIAL_O, CUQWEN_PTR_PARTIAL_ML,   /* split-KV scratch: fp32 partial outputs, (max, sum) pairs */
    CUQWEN_PTR_UP, CUQWEN_PTR_MLP_OUT,              /* QwenState::up / mlp_out: allocated for harnesses that write them, unused by the step (as in the reference, src/model.cu:18-20) */
    CUQWEN_PTR_STREAM,                              /* not a buffer: the cudaStream_t the engine queues its steps on (bytes = 0) */
    CUQWEN_PTR_KEY_SCALE, CUQWEN_PTR_VALUE_SCALE,   /* CUQWEN_FLAG_KV_INT8: fp32 [n_layers][n_kv_heads][max_seq_len] row scales; the caches are then int8 in the same layout */
    CUQWEN_PTR_EMBED = 32, CUQWEN_PTR_NORM, CUQWEN_PTR_LM_HEAD, CUQWEN_PTR_LM_HEAD_SCALE,
    CUQWEN_PTR_IN_NORM = 64, CUQWEN_PTR_WQ, CUQWEN_PTR_SQ, CUQWEN_PTR_BQ, CUQWEN_PTR_WK, CUQWEN_PTR_SK, CUQWEN_PTR_BK,
    CUQWEN_PTR_WV, CUQWEN_PTR_SV, CUQWEN_PTR_BV, CUQWEN_PTR_WO, CUQWEN_PTR_SO, CUQWEN_PTR_POST_NORM,
    CUQWEN_PTR_WGATE, CUQWEN_PTR_SGATE, CUQWEN_PTR_WUP, CUQWEN_PTR_SUP, CUQWEN_PTR_WDOWN, CUQWEN_PTR_SDOWN
};
int cuqwen_get_ptr(cuqwen_engine* e, int which, int layer, void** dev_ptr, size_t* bytes);
/* 1 when the loaded file carries an INT8 lm_head (QwenWeights::lm_head_quantized), 0 fp16, 2 fp16 tied to the embedding. */
int cuqwen_lm_head_kind(const cuqwen_engine* e);
int cuqwen_get_params(const cuqwen_engine* e, cuqwen_params* out);
/* Algorithmic bytes one decode step reads at context length ctx on this rank: all weights, scales, biases,
 * norms, one embedding row, and K+V rows [0, ctx) of every layer. */
uint64_t cuqwen_step_bytes(const cuqwen_engine* e, int ctx);
/* Kernel launches in one decode step. */
int cuqwen_step_launches(const cuqwen_engine* e);
/* Tracing aid (no counterpart in the reference, whose benchmark/kernel_profile.cu times kernels in isolation): run ONE
 * step launch by launch with a CUDA event after every launch and return the microseconds between consecutive events,
 * in launch order (embedding, then per layer qkv / attention / o_proj / gate-up / down, lm_head, penalty, sampler;
 * tensor-parallel runs add their exchange launches).  Times include launch gaps.  Every rank must call it together. */
int cuqwen_step_profile(cuqwen_engine* e, int token, int pos, float* us, int cap, int* n_out);

/* ---- raw device memory helpers (so a host language needs no CUDA binding of its own) ---- */
int cuqwen_dev_alloc(int device, size_t bytes, void** dev_ptr);
/* Number of SMs of the device (what benchmark/kernel_profile.cu's callers would read from cudaGetDeviceProperties):
 * split counts and grid sizes are chosen from it. */
int cuqwen_dev_sm_count(int device, int* sm_count);
int cuqwen_dev_free(int device, void* dev_ptr);
int cuqwen_dev_upload(int device, void* dev_dst, const void* host_src, size_t bytes);
int cuqwen_dev_download(int device, void* host_dst, const void* dev_src, size_t bytes);
int cuqwen_dev_memset(int device, void* dev_ptr, int value, size_t bytes);
int cuqwen_dev_sync(int device);
/* Stream ordering between a caller's CUDA stream (a cudaStream_t; NULL = the legacy default stream) and the
 * library's per-device stream that the cuqwen_k_* calls queue on.  leave == 0: later cuqwen_k_* work waits for what
 * the caller's stream holds now; leave != 0: later work on the caller's stream waits for the cuqwen_k_* work queued
 * so far.  The reference's launch_* take the stream as an argument (include/kernels.cuh:19-160); a binding that
 * wraps each call in join(0) ... join(1) keeps that meaning. */
int cuqwen_dev_join(int device, void* caller_stream, int leave);
/* Kernel timing without the calling language in the measurement (benchmark/kernel_profile.cu times its launches from
 * C++; a host that calls through a binding would otherwise time its own call overhead): between cuqwen_capture_begin
 * and cuqwen_capture_replay the cuqwen_k_* calls on `device` are recorded into a CUDA graph instead of running;
 * cuqwen_capture_replay replays it `replays` times between two events and returns the milliseconds per replay.
 * Every kernel must have run once before the capture starts. */
int cuqwen_capture_begin(int device);
int cuqwen_capture_replay(int device, int replays, float* ms_per_replay);
/* CUDA events on the library's per-device stream, to time a sequence of cuqwen_k_* calls from a host language. */
int cuqwen_bench_begin(int device);
int cuqwen_bench_end(int device, float* ms);

/* ---- per-kernel entry points: the launch_* functions of include/kernels.cuh:19-160 with run-time dims.
 * All pointers are device pointers; work is queued on the device's default stream of this library
 * (cuqwen_dev_sync waits for it). ---- */

/* launch_embedding_lookup (kernels.cuh:19) */
int cuqwen_k_embedding(int device, const void* embed_table, const int* d_token, void* out, int dim);
/* launch_rmsnorm (kernels.cuh:132-139); eps as the fp16-rounded value the reference passes. */
int cuqwen_k_rmsnorm(int device, const void* x, const void* weight, void* out, int dim, float eps);
/* launch_fused_attn_block (kernels.cuh:69-94): q/k/v = W.x + b, then RoPE on q and k.  norm_weight non-null
 * fuses the RMSNorm of x; kcache/vcache non-null also stores k, v at row *d_pos (launch_kv_cache_store, :37-47).
 * x, the three weights, the three biases and d_pos are required (and the scales when quant != 0); q_out / k_out / v_out
 * and the caches may be null one by one.  Like every cuqwen_k_* entry, a null required pointer is CUQWEN_ERR_ARG. */
int cuqwen_k_qkv(int device, int quant, const void* x, const void* norm_weight, float eps,
                 const void* wq, const void* wk, const void* wv, const void* sq, const void* sk, const void* sv,
                 const void* bq, const void* bk, const void* bv, void* q_out, void* k_out, void* v_out,
                 void* kcache, void* vcache, int dim, int n_heads, int n_kv_heads, int head_dim, int max_seq_len,
                 const int* d_pos, float rope_theta, int rope_fast);
/* apply_rope_kernel alone (src/kernels.cu:370-398) */
int cuqwen_k_rope(int device, void* q, void* k, int n_heads, int n_kv_heads, int head_dim, const int* d_pos, float rope_theta, int rope_fast);
/* launch_kv_cache_store (kernels.cuh:37-47) */
int cuqwen_k_kv_store(int device, const void* k, const void* v, void* kcache, void* vcache, const int* d_pos, int n_kv_heads, int max_seq_len, int head_dim);
/* launch_gqa_attention_decode (kernels.cuh:21-36).  scratch_o / scratch_ml / counters sized by
 * cuqwen_attn_scratch_bytes; `counters` is kept in the signature for callers that size it and is never touched. */
int cuqwen_k_attention(int device, const void* q, const void* kcache, const void* vcache, void* out, const int* d_pos,
                       int n_heads, int n_kv_heads, int head_dim, int max_seq_len, int n_splits,
                       void* scratch_o, void* scratch_ml, void* counters);
/* No counterpart in the reference (8-bit KV cache, its roadmap README.md:147).  cuqwen_k_attention over int8 caches
 * [n_kv_heads][max_seq_len][head_dim] with fp32 row scales [n_kv_heads][max_seq_len]: attends to cache rows [0, *d_pos)
 * plus the step's own key / value given in fp16 (k_cur, v_cur: [n_kv_heads][head_dim]), and stores their 8-bit form
 * into row *d_pos of the caches and scale arrays.  The scale arrays need three entries of room past max_seq_len. */
int cuqwen_k_attention_kv8(int device, const void* q, void* kcache8, void* vcache8, float* kscale, float* vscale, const void* k_cur, const void* v_cur,
                           void* out, const int* d_pos, int n_heads, int n_kv_heads, int head_dim, int max_seq_len, int n_splits,
                           void* scratch_o, void* scratch_ml);
/* No counterpart in the reference, which prefills one token at a time through the decode kernels (src/main.cu:86-92;
 * batched prefill is on its roadmap, README.md:145).  Batched-token GEMM on the tcgen05 tensor cores:
 * out[t][r] = sum_k x[t][k] * W[r][k] for n_tokens rows of x ([n_tokens][cols] fp16) and a weight matrix in the model
 * file's format (quant 0 fp16 / 1 int8 / 2 int4, scales [rows][cols / 128] fp16).  mode 0: fp16 output (+ bias[r]);
 * 1: fp32 output; 2: out (fp16) += result, the residual add; 3: SwiGLU of two matrices, out = silu(W0 x) * (W1 x).
 * out_stride = elements between consecutive tokens of out.  rows and out_stride are multiples of 8, cols of 128. */
int cuqwen_k_prefill_gemm(int device, int quant, int mode, const void* x, const void* w0, const void* s0, const void* w1, const void* s1,
                          const void* bias, void* out, int n_tokens, int rows, int cols, int out_stride);
/* No counterpart in the reference (see cuqwen_prefill).  Causal attention of n_tokens prompt queries at cache positions
 * pos0 .. pos0 + n_tokens - 1 over the head-major fp16 caches [n_kv_heads][max_seq_len][head_dim], whose rows for those
 * positions must already hold the queries' own keys and values.  q / out: [n_tokens][q_stride] fp16, head h at columns
 * h * head_dim.  impl 0: tcgen05 kernel, impl 1: mma.sync kernel; head_dim 64 or 128. */
int cuqwen_k_prefill_attention(int device, int impl, const void* q, const void* kcache, const void* vcache, void* out, int n_tokens, int pos0,
                               int n_heads, int n_kv_heads, int head_dim, int max_seq_len, int q_stride);
int cuqwen_attn_scratch_bytes(int n_kv_heads, int head_dim, int n_splits, size_t* bytes_o, size_t* bytes_ml, size_t* bytes_counters);
/* No counterpart in the reference.  Same computation as cuqwen_k_attention for hosts that may not allocate device
 * memory any more (fixed memory budget, or code that must not stall the device's other streams on cudaMalloc):
 * the scratch is a fixed 1.6 MB array inside this library, one per device, so the call allocates nothing.
 * Limit: n_kv_heads * (n_splits + ceil(n_splits / 8)) <= 384 and n_kv_heads * (ceil(n_splits / 8) + 1) <= 256, else
 * CUQWEN_ERR_ARG.  `stream` is a cudaStream_t (NULL = the CUDA default stream); the caller synchronises it.  The
 * first call per device does one-time set-up (address look-up of the array) and should come before any stream
 * capture.  Calls that can overlap on one device (different unordered streams) race on the single scratch block. */
int cuqwen_k_attention_static(int device, void* stream, const void* q, const void* kcache, const void* vcache, void* out,
                              const int* d_pos, int n_heads, int n_kv_heads, int head_dim, int max_seq_len, int n_splits);
/* No counterpart in the reference.  How a caller of cuqwen_k_attention_static learns that a bounded wait inside its
 * kernels ran out (the output is then meaningless): the kernels leave a code in a status word of the fixed array, which
 * no call clears.  This query waits for `stream`, copies the word into *code_out (the caller's own variable; nothing is
 * allocated), clears it, and returns CUQWEN_ERR_TIMEOUT when it was non-zero, CUQWEN_OK otherwise. */
int cuqwen_k_attention_static_status(int device, void* stream, unsigned* code_out);
/* launch_gemv_add_fp16 / launch_fused_mlp_stage2 (kernels.cuh:122-130, :110-120): x_inout += W . input */
int cuqwen_k_gemv_add(int device, int quant, const void* w, const void* scale, const void* input, void* x_inout, int rows, int cols);
/* Plain GEMV y = W . x (fp16 out), optional fused RMSNorm of x.  launch_compute_logits(_int8) (kernels.cuh:141-160). */
int cuqwen_k_gemv(int device, int quant, const void* w, const void* scale, const void* x, const void* norm_weight, float eps, void* y, int rows, int cols);
/* Same with fp32 output (row-parallel partial sums under tensor parallelism). */
int cuqwen_k_gemv_f32(int device, int quant, const void* w, const void* scale, const void* x, float* y, int rows, int cols);
/* launch_fused_mlp_stage1 (kernels.cuh:96-108): h = silu(Wg.x) * (Wu.x), optional fused RMSNorm of x. */
int cuqwen_k_mlp1(int device, int quant, const void* x, const void* norm_weight, float eps, const void* wg, const void* wu,
                  const void* sg, const void* su, void* out, int dim, int inter);
/* launch_apply_repetition_penalty (kernels.cuh:49-56); bitmap: ceil(vocab/32) zeroed u32, left zeroed. */
int cuqwen_k_penalty(int device, void* logits, const int* d_history, const int* d_history_len, int vocab, float penalty, void* bitmap);
/* launch_argmax (kernels.cuh:58-67); scratch: 16 zeroed bytes, left zeroed. */
int cuqwen_k_argmax(int device, const void* logits, int* d_token_out, int vocab, void* scratch16);
/* Dequantised fp16 weights half(float(q) * float(scale)) (the value dot8 multiplies by, src/kernels.cu:27-42). */
int cuqwen_k_dequant(int device, int quant, const void* w, const void* scale, void* out_fp16, long rows, long cols);

/* No counterpart in the reference (it is single-GPU).  The residual update after a row-parallel matrix under tensor
 * parallelism, stand-alone: x_next = half(float(x) + sum over n_ranks receive slots), slots = [n_ranks][dim] 8-byte words
 * {fp32 partial, sequence number}.  The kernel re-reads a word until it carries  *d_step_no * 512 + seq_index + 1, for
 * at most wait_cycles SM cycles (0 = the default of about 4e9); when the wait runs out it returns with whatever the
 * slots hold and the next cuqwen_dev_sync reports CUQWEN_ERR_TIMEOUT. */
int cuqwen_k_tp_sum(int device, const void* x, void* x_next, const void* slots, int n_ranks, int dim, const int* d_step_no, int seq_index,
                    long long wait_cycles);

const char* cuqwen_strerror(int code);
const char* cuqwen_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
