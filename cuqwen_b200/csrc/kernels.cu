// Small kernels of the decode step (embedding row, stand-alone RMSNorm / RoPE /
// KV store, repetition penalty, greedy sampler, tensor-parallel helpers) and
// the launch wrappers for the attention kernel.
#include "attn_split.cuh"
#include "gemv.cuh"
#include "gemv_math.cuh"
#include "gemv_stage.cuh"
#include "launch.h"
#include "rng.cuh"

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <vector>

namespace cq {

template <typename... KArgs, typename... Args>
static int launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, const LaunchCfg& cfg, Args... args) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid; lc.blockDim = block; lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = cfg.pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&lc, kern, KArgs(args)...);
}

// ---- embedding row copy (reference src/kernels.cu:85-96) -------------------
__global__ void embed_kernel(const __half* __restrict__ table, const int* __restrict__ d_token, __half* __restrict__ out, int dim) {
    pdl_launch_dependents(); pdl_wait();
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(*d_token) * dim);
    uint4* dst = reinterpret_cast<uint4*>(out);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim / 8; i += gridDim.x * blockDim.x) dst[i] = src[i];
}
int launch_embed(const __half* table, const int* d_token, __half* out, int dim, const LaunchCfg& cfg) {
    return launch_k(embed_kernel, dim3((dim / 8 + 255) / 256), dim3(256), 0, cfg, table, d_token, out, dim);
}

// The same as the first launch of a decode step.  One CTA: thread 0 first takes over what the host left in the mailbox
// (one 16-byte read of mapped host memory), the others wait for it, and only then are the dependent launches released -
// a later kernel may read ctl->pos before its own dependency wait.
__global__ void embed_step_kernel(const __half* __restrict__ table, StepCtl* ctl, __half* __restrict__ out, int dim) {
    if (threadIdx.x == 0 && ctl->hio && !ctl->auto_advance) {
        int sq, tk, ps, hl;
        asm volatile("ld.volatile.global.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(sq), "=r"(tk), "=r"(ps), "=r"(hl) : "l"(ctl->hio) : "memory");
        if (sq != ctl->io_seq) { ctl->token = tk; ctl->pos = ps; ctl->hist_len = hl; ctl->io_seq = sq; }
        __threadfence();
    }
    __syncthreads();
    pdl_launch_dependents();
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(*(volatile int*)&ctl->token) * dim);
    uint4* dst = reinterpret_cast<uint4*>(out);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = src[i];
}
int launch_embed_step(const __half* table, StepCtl* ctl, __half* out, int dim, const LaunchCfg& cfg) {
    return launch_k(embed_step_kernel, dim3(1), dim3(256), 0, cfg, table, ctl, out, dim);
}

// ---- stand-alone RMSNorm (reference src/kernels.cu:689-751) ----------------
__global__ void rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ w, __half* __restrict__ out, int dim, float eps) {
    __shared__ float red[40];
    pdl_launch_dependents(); pdl_wait();
    const float inv = block_inv_rms(x, dim, eps, red);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        out[i] = __float2half(__half2float(x[i]) * inv * __half2float(w[i]));
}
int launch_rmsnorm(const __half* x, const __half* w, __half* out, int dim, float eps, const LaunchCfg& cfg) {
    return launch_k(rmsnorm_kernel, dim3(1), dim3(256), 0, cfg, x, w, out, dim, eps);
}

// ---- stand-alone RoPE (reference src/kernels.cu:370-398) -------------------
__global__ void rope_kernel(__half* q, __half* k, int n_heads, int n_kv, int hd, const int* d_pos, float theta, int fast) {
    pdl_launch_dependents(); pdl_wait();
    const int half_hd = hd / 2, tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= (n_heads + n_kv) * half_hd) return;
    const bool is_q = tid < n_heads * half_hd;
    const int lt = is_q ? tid : tid - n_heads * half_hd;
    const int head = lt / half_hd, i = lt % half_hd;
    float c, s;
    rope_cs(i, hd, *d_pos, theta, fast, &c, &s);
    __half* buf = is_q ? q : k;
    const int b = head * hd + i;
    const float v0 = __half2float(buf[b]), v1 = __half2float(buf[b + half_hd]);
    buf[b] = __float2half(v0 * c - v1 * s);
    buf[b + half_hd] = __float2half(v1 * c + v0 * s);
}
int launch_rope(__half* q, __half* k, int n_heads, int n_kv, int hd, const int* d_pos, float theta, int fast, const LaunchCfg& cfg) {
    int n = (n_heads + n_kv) * (hd / 2);
    return launch_k(rope_kernel, dim3((n + 255) / 256), dim3(256), 0, cfg, q, k, n_heads, n_kv, hd, d_pos, theta, fast);
}

// ---- stand-alone KV store (reference src/kernels.cu:326-347) ---------------
__global__ void kv_store_kernel(const __half* __restrict__ k, const __half* __restrict__ v, __half* __restrict__ kc, __half* __restrict__ vc,
                                const int* __restrict__ d_pos, int n_kv, int max_seq, int hd) {
    pdl_launch_dependents(); pdl_wait();
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= n_kv * hd) return;
    const int h = tid / hd, d = tid % hd;
    const size_t dst = ((size_t)h * max_seq + *d_pos) * hd + d;
    kc[dst] = k[tid]; vc[dst] = v[tid];
}
int launch_kv_store(const __half* k, const __half* v, __half* kc, __half* vc, const int* d_pos, int n_kv, int max_seq, int hd, const LaunchCfg& cfg) {
    return launch_k(kv_store_kernel, dim3((n_kv * hd + 255) / 256), dim3(256), 0, cfg, k, v, kc, vc, d_pos, n_kv, max_seq, hd);
}

// ---- repetition penalty (reference src/kernels.cu:873-891) -----------------
// The reference visits the first min(hist_len, 4096) history entries and rescales once per
// occurrence, racing on duplicates.  Here the first thread to set the id's bit in `bitmap`
// applies the penalty, so every distinct id is penalised exactly once.
__global__ void penalty_kernel(__half* logits, const int* __restrict__ hist, const int* __restrict__ d_hist_len,
                               int vocab, int vocab_base, float pen, unsigned* bitmap) {
    pdl_launch_dependents(); pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= *d_hist_len) return;
    const int id = hist[idx] - vocab_base;
    if (id < 0 || id >= vocab) return;
    const unsigned bit = 1u << (id & 31);
    if (atomicOr(bitmap + (id >> 5), bit) & bit) return;
    const float l = __half2float(logits[id]);
    logits[id] = __float2half(l < 0.f ? l * pen : l / pen);
}
__global__ void clear_bitmap_kernel(const int* __restrict__ hist, const int* __restrict__ d_hist_len, int vocab, int vocab_base, unsigned* bitmap) {
    pdl_launch_dependents(); pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= *d_hist_len) return;
    const int id = hist[idx] - vocab_base;
    if (id >= 0 && id < vocab) bitmap[id >> 5] = 0u;
}
int launch_penalty(__half* logits, const int* hist, const int* d_hist_len, int vocab, int vocab_base, float penalty, unsigned* bitmap, const LaunchCfg& cfg) {
    return launch_k(penalty_kernel, dim3(16), dim3(256), 0, cfg, logits, hist, d_hist_len, vocab, vocab_base, penalty, bitmap);
}
int launch_clear_bitmap(const int* hist, const int* d_hist_len, int vocab, int vocab_base, unsigned* bitmap, const LaunchCfg& cfg) {
    return launch_k(clear_bitmap_kernel, dim3(16), dim3(256), 0, cfg, hist, d_hist_len, vocab, vocab_base, bitmap);
}

// ---- greedy sampler (reference src/kernels.cu:907-950) ---------------------
__device__ __forceinline__ unsigned long long argmax_pack(float v, int idx) {
    unsigned fu = __float_as_uint(v);
    unsigned key = (fu & 0x80000000u) ? ~fu : (fu | 0x80000000u);
    return ((unsigned long long)key << 32) | (unsigned)(~idx);
}
__device__ __forceinline__ void finish_step(StepCtl* ctl, int token, int* out_ring, int ring_cap) {
    ctl->sampled = token;
    ctl->pad[1] += 1;                  // steps completed: sequence numbers of the tensor-parallel exchanges derive from it
    if (ctl->auto_advance) {
        ctl->token = token;
        ctl->pos += 1;
        const int o = ctl->out_idx;
        if (out_ring && o < ring_cap) out_ring[o] = token;
        ctl->out_idx = o + 1;
    } else if (ctl->hio) {             // host-fed step: the result goes to the mailbox, its sequence number last
        HostIo* h = ctl->hio;
        h->sampled = token; h->err = ctl->pad[0];
        __threadfence_system();
        h->seq_out = ctl->io_seq;
    }
}
// Tensor parallel: where a rank's best (value, index) goes.  Every rank stores ONE 64-bit word into every rank's key
// slots (plain peer stores, like the partial sums of the row-parallel matrices): bits 63..32 the order-preserving key
// of the fp32 value, 31..14 the complemented global index (vocabularies below 2^18 entries), 13..0 the step's number.
// Slots are double-buffered by step parity; a reader knows a word is this step's by its low 14 bits.
struct KeyPush {
    unsigned long long* slot[8];   // rank d's receive words [2][n]: slot[d] points at word [0][this rank]
    int n;                         // ranks (0 = no push)
};
__device__ __forceinline__ unsigned long long key_word(unsigned long long packed, unsigned step) {
    const unsigned long long hi = packed >> 32, nidx = packed & 0x3ffffull;      // ~index keeps its low 18 bits
    return (hi << 32) | (nidx << 14) | (unsigned long long)((step + 1u) & 0x3fffu);
}

__global__ void argmax_kernel(const __half* __restrict__ logits, int vocab, int vocab_base, StepCtl* ctl, int* out_ring, int ring_cap,
                              const int* __restrict__ hist, unsigned* bitmap, unsigned long long* best, unsigned* ticket,
                              unsigned long long* key_out, int* token_out, const KeyPush kp) {
    __shared__ unsigned long long sbest[8];
    pdl_launch_dependents(); pdl_wait();
    // undo the penalty pass's marks (idempotent stores of zero)
    if (hist && bitmap) {
        const int idx = blockIdx.x * blockDim.x + threadIdx.x;
        if (idx < min(ctl->hist_len, 4096)) {
            const int id = hist[idx] - vocab_base;
            if (id >= 0 && id < vocab) bitmap[id >> 5] = 0u;
        }
    }
    unsigned long long b = 0ull;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        unsigned long long p = argmax_pack(__half2float(logits[i]), i + vocab_base);
        b = p > b ? p : b;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { unsigned long long y = __shfl_xor_sync(0xffffffffu, b, o); b = y > b ? y : b; }
    if ((threadIdx.x & 31) == 0) sbest[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) b = sbest[w] > b ? sbest[w] : b;
        atomicMax(best, b);
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            __threadfence();
            const unsigned long long fin = atomicExch(best, 0ull);
            *ticket = 0u;
            const int token = (int)(~((unsigned)(fin & 0xffffffffu)));
            if (kp.n > 0) {
                const unsigned step = (unsigned)ctl->pad[1];
                const unsigned long long w = key_word(fin, step);
                for (int d = 0; d < kp.n; ++d)
                    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(kp.slot[d] + (size_t)(step & 1u) * kp.n), "l"(w) : "memory");
            } else if (key_out) *key_out = fin;
            else if (ctl) finish_step(ctl, token, out_ring, ring_cap);
            if (token_out) *token_out = token;
        }
    }
}
int launch_argmax(const __half* logits, int vocab, int vocab_base, StepCtl* ctl, int* out_ring, int ring_cap, const int* hist, unsigned* bitmap,
                  unsigned long long* best, unsigned* ticket, unsigned long long* key_out, int* token_out, const LaunchCfg& cfg,
                  unsigned long long* const* push_slots, int n_push) {
    int blocks = cfg.sm_count > 16 ? cfg.sm_count : 16;   // >= 16 blocks x 256 threads cover the 4096 history slots
    KeyPush kp{};
    if (push_slots && n_push > 0) {
        if (n_push > 8 || vocab_base + vocab > (1 << 18) || !ctl) return (int)cudaErrorInvalidValue;
        kp.n = n_push;
        for (int d = 0; d < n_push; ++d) kp.slot[d] = push_slots[d];
    }
    return launch_k(argmax_kernel, dim3(blocks), dim3(256), 0, cfg, logits, vocab, vocab_base, ctl, out_ring, ring_cap, hist, bitmap, best, ticket, key_out, token_out, kp);
}
// Tensor parallel: waits (bounded) until the n key words of this step have arrived in this rank's slots, takes their
// maximum and finishes the step like the single-GPU sampler does.  One warp; lane r watches rank r's word.
__global__ void merge_pushed_keys_kernel(const unsigned long long* slots, int n, StepCtl* ctl, int* out_ring, int ring_cap, unsigned* err, long long limit) {
    pdl_launch_dependents(); pdl_wait();
    const int lane = threadIdx.x;
    const unsigned step = (unsigned)ctl->pad[1];
    const unsigned want = (step + 1u) & 0x3fffu;
    unsigned long long w = 0ull;
    if (lane < n) {
        const unsigned long long* p = slots + (size_t)(step & 1u) * n + lane;
        unsigned long long t0 = 0ull;
        for (;;) {
            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
            if ((unsigned)(w & 0x3fffull) == want) break;
            const unsigned long long now = (unsigned long long)sm_cycles();
            if (t0 == 0ull) t0 = now | 1ull;
            else if (now - t0 > (unsigned long long)limit) { if (err) atomicExch(err, 10u); break; }
        }
        w >>= 14;                                           // (value key, ~index): larger value first, then smaller index
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const unsigned long long y = __shfl_xor_sync(0xffffffffu, w, o); w = y > w ? y : w; }
    if (lane == 0) finish_step(ctl, (int)(~(unsigned)(w & 0x3ffffull) & 0x3ffffu), out_ring, ring_cap);
}
int launch_merge_pushed_keys(const unsigned long long* slots, int n, StepCtl* ctl, int* out_ring, int ring_cap, unsigned* err, long long wait_cycles, const LaunchCfg& cfg) {
    return launch_k(merge_pushed_keys_kernel, dim3(1), dim3(32), 0, cfg, slots, n, ctl, out_ring, ring_cap, err, wait_cycles > 0 ? wait_cycles : kWaitCyclesDefault);
}
__global__ void merge_keys_kernel(const unsigned long long* __restrict__ keys, int n, StepCtl* ctl, int* out_ring, int ring_cap) {
    pdl_launch_dependents(); pdl_wait();
    if (threadIdx.x != 0) return;
    unsigned long long b = 0ull;
    for (int i = 0; i < n; ++i) b = keys[i] > b ? keys[i] : b;
    finish_step(ctl, (int)(~((unsigned)(b & 0xffffffffu))), out_ring, ring_cap);
}
int launch_merge_keys(const unsigned long long* keys, int n, StepCtl* ctl, int* out_ring, int ring_cap, const LaunchCfg& cfg) {
    return launch_k(merge_keys_kernel, dim3(1), dim3(32), 0, cfg, keys, n, ctl, out_ring, ring_cap);
}

// ---- tensor-parallel residual from pushed slots: x_next = half(float(x) + sum_r slot_r), one thread per 8 columns ----
// Used instead of the gather inside the consuming GEMV when there are many ranks: there every CTA would read all
// ranks' slots again; here they are read once.  Same words, same bounded re-read, same rank order as park_gather.
__global__ void tp_sum_kernel(const __half* __restrict__ x, __half* __restrict__ x_next, const uint2* slots, int n, int K, const int* step_no, int seq_index,
                              unsigned* err, long long limit) {
    pdl_launch_dependents(); pdl_wait();
    const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c8 >= K / 8) return;
    const unsigned seq = (unsigned)(*step_no) * kSeqPerStep + (unsigned)seq_index + 1u;
    const uint4 xo = __ldcg(reinterpret_cast<const uint4*>(x) + c8);
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool gave_up = false;
    for (int r0 = 0; r0 < n; r0 += 4) {
        unsigned long long q[4][8];
        unsigned long long t0 = 0ull;
        for (;;) {
            bool ok = true;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (r0 + j < n) {
                    const uint2* p = slots + (size_t)(r0 + j) * K + (size_t)c8 * 8;
#pragma unroll
                    for (int i = 0; i < 4; ++i) ld_pair2(p + 2 * i, q[j][2 * i], q[j][2 * i + 1]);
                }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (r0 + j < n) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) ok = ok && pair_seq(q[j][i]) == seq;
                }
            if (ok || gave_up) break;
            const unsigned long long now = (unsigned long long)sm_cycles();      // the SM's cycle counter: cheap to read
            if (t0 == 0ull) t0 = now | 1ull;
            else if (now - t0 > (unsigned long long)limit) { gave_up = true; if (err) atomicExch(err, 8u); break; }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (r0 + j < n) {
#pragma unroll
                for (int i = 0; i < 8; ++i) s[i] += pair_val(q[j][i]);
            }
    }
    uint4 xn;
    const __half2* h = reinterpret_cast<const __half2*>(&xo);
    __half2* o = reinterpret_cast<__half2*>(&xn);
#pragma unroll
    for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h[k]); o[k] = __floats2half2_rn(f.x + s[2 * k], f.y + s[2 * k + 1]); }
    reinterpret_cast<uint4*>(x_next)[c8] = xn;
}
int launch_tp_sum(const __half* x, __half* x_next, const void* slots, int n, int K, const int* step_no, int seq_index, unsigned* err, long long wait_cycles,
                  const LaunchCfg& cfg) {
    return launch_k(tp_sum_kernel, dim3((K / 8 + 31) / 32), dim3(32), 0, cfg, x, x_next, (const uint2*)slots, n, K, step_no, seq_index, err,
                    wait_cycles > 0 ? wait_cycles : kWaitCyclesDefault);
}

// ---- tensor-parallel residual: x = half(float(x) + sum_r partial_r) --------
__global__ void resid_sum_kernel(__half* x, const float* __restrict__ partial, int n_parts, size_t stride, int dim) {
    pdl_launch_dependents(); pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dim) return;
    float s = 0.f;
    for (int r = 0; r < n_parts; ++r) s += partial[(size_t)r * stride + i];
    x[i] = __float2half(__half2float(x[i]) + s);
}
int launch_resid_sum(__half* x, const float* partial, int n_parts, size_t part_stride, int dim, const LaunchCfg& cfg) {
    return launch_k(resid_sum_kernel, dim3((dim + 255) / 256), dim3(256), 0, cfg, x, partial, n_parts, part_stride, dim);
}

// ---- dequantised fp16 weights: half(float(q) * float(scale)) ---------------
__global__ void dequant_kernel(int quant, const uint8_t* __restrict__ w, const __half* __restrict__ s, __half* __restrict__ out, long rows, long cols) {
    const long n = rows * cols, ng = cols / kGroup;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const long r = i / cols, c = i % cols;
        int q;
        if (quant == Q_I4) {
            const unsigned b = w[r * (cols / 2) + c / 2];
            const unsigned nib = (c & 1) ? (b >> 4) : (b & 0xF);
            q = (int)(nib ^ 8u) - 8;
        } else {
            q = (int)reinterpret_cast<const int8_t*>(w)[i];
        }
        out[i] = __float2half((float)q * __half2float(s[r * ng + c / kGroup]));
    }
}
int launch_dequant(int quant, const void* w, const __half* s, __half* out, long rows, long cols, const LaunchCfg& cfg) {
    long n = rows * cols;
    int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    return launch_k(dequant_kernel, dim3(blocks), dim3(256), 0, cfg, quant, (const uint8_t*)w, s, out, rows, cols);
}

// The same N(0,1) values as fill_normal_kernel, stored as 8-bit cache rows: one warp per row of `hd` values.
__global__ void fill_normal_q8_kernel(signed char* dst, float* scales, size_t rows, int hd, uint64_t seed, uint64_t base) {
    const int lane = threadIdx.x & 31, n = hd / 32;
    for (size_t r = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += (size_t)gridDim.x * (blockDim.x >> 5)) {
        float v[4], m = 0.f;
        for (int i = 0; i < n; ++i) { v[i] = __half2float(__float2half(normal_at(seed, base + r * hd + lane * n + i))); m = fmaxf(m, fabsf(v[i])); }
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float inv = m > 0.f ? 127.0f / m : 0.f;
        for (int i = 0; i < n; ++i) dst[r * hd + lane * n + i] = (signed char)__float2int_rn(v[i] * inv);
        if (lane == 0) scales[r] = m / 127.0f;
    }
}
int launch_fill_normal_q8(void* dst, float* scales, size_t rows, int hd, uint64_t seed, uint64_t base, const LaunchCfg& cfg) {
    if (hd != 64 && hd != 128) return (int)cudaErrorInvalidValue;
    int blocks = (int)((rows + 7) / 8 < 8192 ? (rows + 7) / 8 : 8192);
    if (blocks < 1) blocks = 1;
    return launch_k(fill_normal_q8_kernel, dim3(blocks), dim3(256), 0, cfg, (signed char*)dst, scales, rows, hd, seed, base);
}

int launch_fill_normal(__half* dst, size_t n, uint64_t seed, uint64_t base, const LaunchCfg& cfg) {
    int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    if (blocks < 1) blocks = 1;
    return launch_k(fill_normal_kernel, dim3(blocks), dim3(256), 0, cfg, dst, n, seed, base);
}

// ---- attention -------------------------------------------------------------
size_t attn_scratch_floats_o(int n_kv, int nsplit, int head_dim) { return attn_slots(n_kv, nsplit) * kMaxGroup * head_dim; }
size_t attn_scratch_floats_ml(int n_kv, int nsplit) { return attn_slots(n_kv, nsplit) * kMaxGroup * 2; }
size_t attn_scratch_counters(int n_kv, int nsplit) { return attn_counters(n_kv, nsplit); }

// Two launches: partials, then the fold (attn_split.cuh).  Returns the first error.  a.kscale != null selects the
// kernel for the 8-bit cache.
template <int HD, bool KV8>
static int launch_attn_split(const AttnArgs& a, const LaunchCfg& cfg) {
    AttnArgs b = a;
    b.stages = kSplitStages;
    const size_t smem = attn_split_smem_bytes(HD, b.stages, KV8);
    static bool once = false;
    if (!once) {
        cudaError_t e = cudaFuncSetAttribute(attn_partial_kernel<HD, KV8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_partial_kernel<HD, KV8>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_fold_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        once = true;
    }
    if (int r = launch_k(attn_partial_kernel<HD, KV8>, dim3(b.n_kv, b.nsplit), dim3(kSplitThreads), smem, cfg, b)) return r;
    return launch_k(attn_fold_kernel<HD>, dim3(b.n_kv * b.grp), dim3(kFoldWarps * 32), 0, cfg, b);
}
int launch_attn(int head_dim, const AttnArgs& a, const LaunchCfg& cfg) {
    if (a.grp < 1 || a.grp > kMaxGroup || a.nsplit < 1 || a.nsplit > kMaxSplit) return (int)cudaErrorInvalidValue;
    const bool kv8 = a.kscale != nullptr;
    if (kv8 && (!a.vscale || !a.k_cur || !a.v_cur)) return (int)cudaErrorInvalidValue;
    if (head_dim == 128) return kv8 ? launch_attn_split<128, true>(a, cfg) : launch_attn_split<128, false>(a, cfg);
    if (head_dim == 64) return kv8 ? launch_attn_split<64, true>(a, cfg) : launch_attn_split<64, false>(a, cfg);
    return (int)cudaErrorInvalidValue;
}

// ---- GEMV dispatch ---------------------------------------------------------
int launch_gemv_i4(int epi, const GemvArgs& a, dim3 grid, dim3 block, size_t smem, const LaunchCfg& cfg);
int launch_gemv_i8(int epi, const GemvArgs& a, dim3 grid, dim3 block, size_t smem, const LaunchCfg& cfg);
int launch_gemv_f16(int epi, const GemvArgs& a, dim3 grid, dim3 block, size_t smem, const LaunchCfg& cfg);

// cuTensorMapEncodeTiled through the runtime's driver-entry-point lookup (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}
// Byte-typed 3-D map of a row-major matrix seen as [rows][64-byte chunks]: dims {64, rows, row_bytes / 64}, box
// {64, box_rows, piece_bytes / 64}, zero fill out of bounds.  A box therefore lands in shared memory chunk-major,
// [chunk][row][64 bytes]: consecutive rows of one chunk are 64 bytes apart, so the 16-byte fragment loads of an MMA
// operand (eight rows x four 16-byte columns per quarter-warp) touch every bank once.  In a row-major box the rows
// would be piece_bytes (a multiple of 128) apart and pairs of rows would collide on the same banks.
// Encoding a map is a driver call of a microsecond or so; a caller that launches the same matrix again and again (the
// stand-alone entry points, the microbenchmarks) gets it from a small table instead.  A map depends on nothing but the
// arguments below, so an entry can never go stale.
namespace {
struct MapKey { const void* w; size_t row_bytes, rows; int piece_bytes, box_rows; };
struct MapEntry { MapKey k; CUtensorMap m; };
std::mutex g_map_mu;
std::vector<MapEntry> g_maps;
}  // namespace
static int encode_weight_map(CUtensorMap* m, const void* w, size_t row_bytes, size_t rows, int piece_bytes, int box_rows);
int make_weight_map(CUtensorMap* m, const void* w, size_t row_bytes, size_t rows, int piece_bytes, int box_rows) {
    std::lock_guard<std::mutex> lk(g_map_mu);
    for (const MapEntry& e : g_maps)
        if (e.k.w == w && e.k.row_bytes == row_bytes && e.k.rows == rows && e.k.piece_bytes == piece_bytes && e.k.box_rows == box_rows) { *m = e.m; return 0; }
    if (int r = encode_weight_map(m, w, row_bytes, rows, piece_bytes, box_rows)) return r;
    if (g_maps.size() >= 4096) g_maps.clear();
    g_maps.push_back(MapEntry{MapKey{w, row_bytes, rows, piece_bytes, box_rows}, *m});
    return 0;
}
static int encode_weight_map(CUtensorMap* m, const void* w, size_t row_bytes, size_t rows, int piece_bytes, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return (int)cudaErrorNotSupported;
    if (row_bytes % kChunkBytes || piece_bytes % kChunkBytes) return (int)cudaErrorInvalidValue;
    const cuuint64_t dims[3] = {kChunkBytes, rows, row_bytes / kChunkBytes}, strides[2] = {row_bytes, kChunkBytes};
    const cuuint32_t box[3] = {kChunkBytes, (cuuint32_t)box_rows, (cuuint32_t)(piece_bytes / kChunkBytes)}, estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

constexpr int kGemvThreadsHost = (kConsumerWarps + 1) * 32;

// Rows per CTA block: whole 16-row tiles, as many per block (1, 2, 4 or 8) as keep at least one block per SM.
// (The kernel takes any row count per block.  Cutting the matrix into SM-count nearly equal blocks instead - 26 rows
// for the 3584-row projections of the 7B model, 138 blocks in one round where whole tiles give 224 - measured slower:
// down projection 11.8 against 10.4 us in the step, o_proj 5.9 against 5.1.  The 224 blocks of 16 rows run two to an
// SM, sixteen consumer warps per SM, and the SMs with one block leave their share of the bandwidth to the others.)
int gemv_block_rows(int rows, int K, int sm_count, int epi) {
    (void)K;
    if (epi == EPI_QKV) return 16;
    const int nsets = (rows + 15) / 16;
    int rw = 1;
    while (rw < 8 && nsets / (rw * 2) >= sm_count) rw *= 2;
    return 16 * rw;
}

// Picks the work split (rw row-warps x kw K-parts), the staged piece size and the ring depth for one GEMV launch.
//   many tile sets: blocks of up to 8 tile sets (128 rows), every consumer warp walks the whole K of its 16 rows;
//   few tile sets: one tile set per CTA, its K split over the eight consumer warps.
int launch_gemv(int quant, int epi, GemvArgs& a, const LaunchCfg& cfg) {
    if (a.K <= 0 || a.K % kGroup != 0 || a.K > 24576) return (int)cudaErrorInvalidValue;
    if (quant < 0 || quant > 2) return (int)cudaErrorInvalidValue;
    if (epi == EPI_QKV) {
        if (a.hd % 32 != 0) return (int)cudaErrorInvalidValue;
        a.nsets = (a.n_heads + 2 * a.n_kv) * (a.hd / 32);
        a.brows = 16; a.nblk = a.nsets;
    } else {
        if (a.rows <= 0) return (int)cudaErrorInvalidValue;
        a.nsets = (a.rows + 15) / 16;
        a.brows = gemv_block_rows(a.rows, a.K, cfg.sm_count, epi);
        a.nblk = (a.rows + a.brows - 1) / a.brows;
    }
    const int MT = (epi == EPI_SWIGLU || epi == EPI_QKV) ? 2 : 1;
    const int ngrp = a.K / kGroup;
    const int gb = quant == Q_I4 ? 64 : quant == Q_I8 ? 128 : 256;
    const int pg_max = 256 / gb;                     // row pieces of at most 256 bytes (TMA box limit for byte elements)
    const int kMaxSmem = 225 * 1024;
    int rw = 1;
    while (16 * rw < a.brows) rw *= 2;               // row-warps: enough 16-row tiles to cover a block (1, 2, 4 or 8)
    int kw = 8 / rw;                                 // rw * kw may end up below 8 when a row has few pieces: the spare warps idle
    const int nblk = a.nblk;
    // Shared-memory budget of a CTA.  int4 weights with more blocks than SMs: 110 KB, two CTAs to an SM (at the 96
    // registers of the one-matrix kernels two CTAs fit), so that one streams while the other is in its prologue or
    // epilogue.  int8 / fp16 weights move two to four times the bytes per row piece, and a ring cut to 110 KB is too
    // shallow for them (measured on the 14B int8 matrices: gate/up 37.5 us at 110 KB against 28.2 us at 220 KB,
    // lm_head 139 against 119 us): they take the whole SM.
    // (CTAs of two consecutive kernels of the step do not share an SM at these register counts.  Capped at 80
    // registers they do, and the step was slower - 574 against 703 tok/s on the 7B int4 model: the early weight
    // copies of the next kernel compete with the loads the running kernel is waiting for.)
    const int cap_kb = (nblk > cfg.sm_count && quant == Q_I4) ? 110 : 220;
    const int per_sm = cap_kb == 110 ? 2 : 1;
    const int grid = nblk < per_sm * cfg.sm_count ? nblk : per_sm * cfg.sm_count;
    const int nsb = nblk <= grid ? 1 : 2;            // a second scale block only when some CTA has a second block
    int cap = cap_kb * 1024;
    int pg = 0, nst = 0;
    for (int pass = 0; pass < 2 && !nst; ++pass) {
        for (int q = pg_max; q >= 1; --q) {
            const int pt = (ngrp + q - 1) / q;
            int kwq = kw; while (kwq > 1 && kwq > pt) kwq /= 2;                   // no more K-parts than pieces
            const int steps = (pt + kwq - 1) / kwq;
            int want = rw == 8 ? 6 : steps < 6 ? steps : 6;
            int n = want;
            while (n > 1 && gemv_smem_bytes(a.K, quant, MT, a.brows, kwq, q, n, nsb) > (size_t)cap) --n;
            if (gemv_smem_bytes(a.K, quant, MT, a.brows, kwq, q, n, nsb) > (size_t)cap) continue;
            if (n >= (want < 3 ? want : 3) || q == 1) { pg = q; nst = n; kw = kwq; break; }
            if (!nst || n > nst) { pg = q; nst = n; kw = kwq; }
            if (q == 1) break;
            nst = 0;
        }
        if (!nst) cap = kMaxSmem;
    }
    if (!nst) return (int)cudaErrorInvalidValue;
    if (epi == EPI_QKV && rw != 1) return (int)cudaErrorInvalidValue;
    int gw = kConsumerWarps / (rw * kw);              // warps left over share cells, group by group
    while (gw > 1 && gw > pg) gw /= 2;
    a.rw = rw; a.kw = kw; a.gw = gw; a.pg = pg; a.nst = nst; a.nsb = nsb;
    const size_t smem = gemv_smem_bytes(a.K, quant, MT, a.brows, kw, pg, nst, nsb);
    {
        const size_t rbytes = quant == Q_I4 ? a.K / 2 : quant == Q_I8 ? a.K : (size_t)a.K * 2;
        const int nmat = epi == EPI_QKV ? 3 : epi == EPI_SWIGLU ? 2 : 1;
        for (int m = 0; m < nmat; ++m) {
            const size_t rows_m = epi == EPI_QKV ? (size_t)(m == 0 ? a.n_heads : a.n_kv) * a.hd : (size_t)a.rows;
            if (int r = make_weight_map(&a.tmap[m], a.w[m], rbytes, rows_m, pg * gb, a.brows)) return r;
        }
    }
    const dim3 gridd(grid), block(kGemvThreadsHost);
    if (quant == Q_I4) return launch_gemv_i4(epi, a, gridd, block, smem, cfg);
    if (quant == Q_I8) return launch_gemv_i8(epi, a, gridd, block, smem, cfg);
    return launch_gemv_f16(epi, a, gridd, block, smem, cfg);
}

}  // namespace cq
