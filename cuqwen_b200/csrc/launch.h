// Host-side launch interface shared by the engine and the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cq {

struct GemvArgs;
struct AttnArgs;

// Device-resident control block of one decode step.  The graph reads token /
// pos / hist_len from here; with auto_advance set the sampler feeds its result
// back so consecutive graph launches need no host round trip.
// Host-visible mailbox of a step (pinned, mapped host memory): the host writes the inputs of cuqwen_step here and the
// step's first kernel fetches them; the step's last kernel leaves the result here and the host polls for it.  No copy
// call and no stream synchronisation lie between a token going in and the next one coming out.  Two 64-byte lines.
struct HostIo {
    int seq_in, token, pos, hist_len;      // one 16-byte unit: read by the device with a single load; seq_in is written last
    int rsv_in[12];
    volatile int seq_out;                  // = the seq_in this result belongs to, written after the two words below
    volatile int sampled, err;
    int rsv_out[13];
};
struct StepCtl {
    int token;
    int pos;
    int hist_len;
    int auto_advance;
    int out_idx;      // next slot of the output ring (auto_advance only)
    int sampled;      // result of the last step
    int pad[2];       // [0] a bounded wait expired (code), [1] steps completed
    int io_seq;       // seq_in of the last mailbox message taken over
    int rsv;
    HostIo* hio;      // the mailbox, or null
};

struct LaunchCfg {
    cudaStream_t stream;
    int sm_count;
    bool pdl;         // launch with programmatic stream serialization
};

// GEMV family.  quant: 0 fp16, 1 int8, 2 int4.  epi: cq::Epi.  Chooses the work split (rw, kw, gw), the staged piece
// size and the ring depth, builds the tensor maps and launches.  Returns a cudaError_t value.
int launch_gemv(int quant, int epi, GemvArgs& a, const LaunchCfg& cfg);
// Rows per CTA block that launch_gemv will choose for a matrix of `rows` rows and K input columns.
int gemv_block_rows(int rows, int K, int sm_count, int epi);

// Byte-typed 3-D tensor map of a row-major matrix seen as [rows][64-byte chunks]: a box of box_rows rows x piece_bytes
// lands in shared memory chunk-major, [chunk][row][64 bytes].
int make_weight_map(CUtensorMap* m, const void* w, size_t row_bytes, size_t rows, int piece_bytes, int box_rows);

int launch_attn(int head_dim, const AttnArgs& a, const LaunchCfg& cfg);
size_t attn_scratch_floats_o(int n_kv, int nsplit, int head_dim);
size_t attn_scratch_floats_ml(int n_kv, int nsplit);
size_t attn_scratch_counters(int n_kv, int nsplit);   // u32 tickets

int launch_embed(const __half* table, const int* d_token, __half* out, int dim, const LaunchCfg& cfg);
// First launch of a decode step: takes over a new mailbox message (unless the step feeds itself), then copies the token's row.
int launch_embed_step(const __half* table, StepCtl* ctl, __half* out, int dim, const LaunchCfg& cfg);
int launch_rmsnorm(const __half* x, const __half* w, __half* out, int dim, float eps, const LaunchCfg& cfg);
int launch_rope(__half* q, __half* k, int n_heads, int n_kv, int hd, const int* d_pos, float theta, int fast, const LaunchCfg& cfg);
int launch_kv_store(const __half* k, const __half* v, __half* kc, __half* vc, const int* d_pos, int n_kv, int max_seq, int hd, const LaunchCfg& cfg);
// Repetition penalty, once per distinct id among the first min(hist_len, 4096) entries.
// `bitmap` holds ceil(vocab/32) zeroed words; the sampler (or clear_bitmap) zeroes it again.
int launch_penalty(__half* logits, const int* hist, const int* d_hist_len, int vocab, int vocab_base, float penalty, unsigned* bitmap, const LaunchCfg& cfg);
int launch_clear_bitmap(const int* hist, const int* d_hist_len, int vocab, int vocab_base, unsigned* bitmap, const LaunchCfg& cfg);
// Greedy sampler.  best/ticket: one u64 and one u32 of zeroed scratch.  Writes ctl->sampled and, when
// ctl->auto_advance is set, feeds the token back (token, pos+1, out_ring).  When key_out is non-null the packed
// (order key << 32 | ~global index) is stored there instead (tensor-parallel ranks merge them later).
// push_slots / n_push (tensor parallel without a collective call): the packed key, tagged with the step's number, is
// stored into one 64-bit word per rank instead (kernels.cu: KeyPush); launch_merge_pushed_keys reads them.
int launch_argmax(const __half* logits, int vocab, int vocab_base, StepCtl* ctl, int* out_ring, int ring_cap,
                  const int* hist, unsigned* bitmap, unsigned long long* best, unsigned* ticket,
                  unsigned long long* key_out, int* token_out, const LaunchCfg& cfg,
                  unsigned long long* const* push_slots = nullptr, int n_push = 0);
int launch_merge_pushed_keys(const unsigned long long* slots, int n, StepCtl* ctl, int* out_ring, int ring_cap, unsigned* err, long long wait_cycles,
                             const LaunchCfg& cfg);
// Merge n packed keys (one per rank) and finish the step like launch_argmax does.
int launch_merge_keys(const unsigned long long* keys, int n, StepCtl* ctl, int* out_ring, int ring_cap, const LaunchCfg& cfg);
// x = half(float(x) + sum_r partial[r][:])   (row-parallel layers under tensor parallelism)
int launch_resid_sum(__half* x, const float* partial, int n_parts, size_t part_stride, int dim, const LaunchCfg& cfg);
// Tensor parallel, many ranks: x_next = half(float(x) + sum over n ranks of the pushed {value, sequence} slots [n][K]).
// wait_cycles: bound of the re-read loop in SM cycles (0 = the default of about two to four seconds).
int launch_tp_sum(const __half* x, __half* x_next, const void* slots, int n, int K, const int* step_no, int seq_index, unsigned* err, long long wait_cycles,
                  const LaunchCfg& cfg);
// out = half(float(q) * float(scale)) for every weight; quant 1 or 2.
int launch_dequant(int quant, const void* w, const __half* s, __half* out, long rows, long cols, const LaunchCfg& cfg);
// The same values as 8-bit cache rows (one fp32 scale per row of hd values): rows * hd values starting at element `base`.
int launch_fill_normal_q8(void* dst, float* scales, size_t rows, int hd, uint64_t seed, uint64_t base, const LaunchCfg& cfg);
// Deterministic N(0,1) fp16 fill: element i gets a value that depends only on (seed, base + i).
int launch_fill_normal(__half* dst, size_t n, uint64_t seed, uint64_t base, const LaunchCfg& cfg);

}  // namespace cq
