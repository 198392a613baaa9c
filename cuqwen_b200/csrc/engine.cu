// Host side of the decode engine: model table, weight loader, state, the
// per-step launch sequence and its CUDA graph, tensor-parallel plumbing, and
// the extern "C" boundary declared in include/cuqwen_b200.h.
#include <dlfcn.h>
#include <fcntl.h>
#include <nccl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/cuqwen_b200.h"
#include "attn.cuh"
#include "errors.h"
#include "gemv.cuh"
#include "launch.h"
#include "prefill.cuh"
#include "prefill_gemm.cuh"
#include "tp_plan.h"

using namespace cq;

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";
static int fail(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof g_err, fmt, ap); va_end(ap);
    return code;
}
int cq::report_error(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof g_err, fmt, ap); va_end(ap);
    return code;
}
#define CK(call) do { cudaError_t e_ = (cudaError_t)(call); if (e_ != cudaSuccess) return fail(CUQWEN_ERR_CUDA, "%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); } while (0)

extern "C" const char* cuqwen_last_error(void) { return g_err; }
extern "C" const char* cuqwen_strerror(int code) {
    switch (code) {
        case CUQWEN_OK: return "ok";
        case CUQWEN_ERR_ARG: return "bad argument or unsupported shape";
        case CUQWEN_ERR_IO: return "weight file cannot be read";
        case CUQWEN_ERR_MAGIC: return "weight file magic mismatch";
        case CUQWEN_ERR_DIMS: return "weight file dimensions do not match the engine";
        case CUQWEN_ERR_QUANT: return "weight file quantisation does not match the engine";
        case CUQWEN_ERR_CUDA: return "CUDA error";
        case CUQWEN_ERR_NCCL: return "NCCL error";
        case CUQWEN_ERR_STATE: return "call made in the wrong state";
        case CUQWEN_ERR_TIMEOUT: return "device-side wait timed out";
    }
    return "unknown error";
}

// ---------------------------------------------------------------------------
// model table (reference include/config.h:55-113)
// ---------------------------------------------------------------------------
struct ModelRow { int vocab, dim, inter, layers, heads, kv, hd; };
static const ModelRow kModels[5] = {
    {151936, 896, 4864, 24, 14, 2, 64},     // 0.5B
    {151936, 1536, 8960, 28, 12, 2, 128},   // 1.5B
    {151936, 2048, 11008, 36, 16, 2, 128},  // 3B
    {152064, 3584, 18944, 28, 28, 4, 128},  // 7B
    {152064, 5120, 13824, 48, 40, 8, 128},  // 14B
};

extern "C" int cuqwen_model_params(int model_id, int quant, cuqwen_params* p) {
    if (!p || model_id < 0 || model_id > 4 || quant < 0 || quant > 2) return fail(CUQWEN_ERR_ARG, "model_id %d / quant %d out of range", model_id, quant);
    memset(p, 0, sizeof *p);
    const ModelRow& m = kModels[model_id];
    p->model_id = model_id; p->vocab_size = m.vocab; p->dim = m.dim; p->intermediate_size = m.inter; p->n_layers = m.layers;
    p->n_heads = m.heads; p->n_kv_heads = m.kv; p->head_dim = m.hd; p->max_seq_len = 32768; p->quant = quant;
    p->tp_size = 1; p->norm_eps = 1e-6f; p->rope_theta = 1000000.0f; p->repetition_penalty = 1.1f;
    return CUQWEN_OK;
}

// ---------------------------------------------------------------------------
// per-device context for the stand-alone kernel entry points
// ---------------------------------------------------------------------------
struct DevCtx { bool init = false; cudaStream_t stream = nullptr; int sms = 0; cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev_join = nullptr; unsigned* err = nullptr; unsigned* h_err = nullptr; };
// device word that kernels launched by the calling thread report an expired bounded wait to
static thread_local unsigned* t_err = nullptr;
static DevCtx g_dev[64];
static std::mutex g_dev_mu;
static int dev_ctx(int device, DevCtx** out) {
    if (device < 0 || device >= 64) return fail(CUQWEN_ERR_ARG, "device %d out of range", device);
    std::lock_guard<std::mutex> lk(g_dev_mu);
    CK(cudaSetDevice(device));
    DevCtx& d = g_dev[device];
    if (!d.init) {
        CK(cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking));
        CK(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device));
        CK(cudaEventCreate(&d.ev0)); CK(cudaEventCreate(&d.ev1));
        CK(cudaEventCreateWithFlags(&d.ev_join, cudaEventDisableTiming));
        CK(cudaMalloc((void**)&d.err, 4)); CK(cudaMemset(d.err, 0, 4)); CK(cudaMallocHost((void**)&d.h_err, 4));
        d.init = true;
    }
    *out = &d;
    return CUQWEN_OK;
}
// The per-kernel entry points launch the way the engine's graph does: with programmatic dependent launch, so that a
// kernel's prologue may overlap the tail of the call before it (every kernel waits for its predecessor before it
// touches data).
#define DEV(device) DevCtx* dc; { int r_ = dev_ctx(device, &dc); if (r_) return r_; } t_err = dc->err; LaunchCfg cfg{dc->stream, dc->sms, true}

// ---------------------------------------------------------------------------
// NCCL through dlopen (no link-time dependency; single-GPU use never loads it)
// ---------------------------------------------------------------------------
struct Nccl {
    void* lib = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
};
static Nccl g_nccl;
static int nccl_load() {
    static std::mutex mu; std::lock_guard<std::mutex> lk(mu);
    if (g_nccl.lib) return CUQWEN_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(CUQWEN_ERR_NCCL, "dlopen libnccl.so.2: %s", dlerror());
#define SYM(n) g_nccl.n = (decltype(g_nccl.n))dlsym(h, "nccl" #n); if (!g_nccl.n) return fail(CUQWEN_ERR_NCCL, "nccl" #n " missing")
    SYM(GetUniqueId); SYM(CommInitRank); SYM(AllReduce); SYM(AllGather); SYM(CommDestroy); SYM(GetErrorString);
#undef SYM
    g_nccl.lib = h;
    return CUQWEN_OK;
}
#define NK(call) do { ncclResult_t r_ = (call); if (r_ != ncclSuccess) return fail(CUQWEN_ERR_NCCL, "%s: %s", #call, g_nccl.GetErrorString(r_)); } while (0)

// ---------------------------------------------------------------------------
// engine
// ---------------------------------------------------------------------------
struct Mat { uint8_t* w = nullptr; __half* s = nullptr; int rows = 0, cols = 0; };
struct Layer {
    __half *in_norm = nullptr, *post_norm = nullptr, *bq = nullptr, *bk = nullptr, *bv = nullptr;
    Mat q, k, v, o, gate, up, down;
};

struct cuqwen_engine {
    cuqwen_params p{};
    int sms = 0;
    cudaStream_t stream = nullptr;
    TpPlan plan{};
    int tp = 1, rank = 0;
    // local sizes
    int n_heads_l = 0, n_kv_l = 0, q_dim_l = 0, kv_dim_l = 0, inter_l = 0, vocab_l = 0, nsplit = 0;
    // weights
    uint8_t* warena = nullptr; size_t warena_bytes = 0;
    std::vector<Layer> layers;
    __half *embed = nullptr, *norm = nullptr;
    Mat lm; int lm_quant = 0; int lm_kind = 0;   // kind: 0 fp16 separate, 1 int8, 2 tied
    bool loaded = false;
    uint64_t weight_bytes = 0;                   // algorithmic bytes of all tensors a step reads (this rank)
    // state
    __half *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *gate = nullptr, *logits = nullptr;
    __half *kc = nullptr, *vc = nullptr;                  // CUQWEN_FLAG_KV_INT8: int8 rows behind these pointers, scales below
    float *kscale = nullptr, *vscale = nullptr; bool kv8 = false;
    __half *spare_up = nullptr, *spare_out = nullptr;     // QwenState::up / mlp_out of the source-compatible layer (never read by the step)
    float *part_o = nullptr, *part_ml = nullptr; unsigned* counters = nullptr;
    StepCtl* ctl = nullptr; StepCtl* h_ctl = nullptr;
    HostIo* hio = nullptr; HostIo* hio_dev = nullptr; int io_seq = 0; bool ctl_dirty = true;   // mailbox of cuqwen_step (launch.h); ctl_dirty: the device block must be rewritten first
    int* d_hist = nullptr; unsigned* bitmap = nullptr; unsigned long long* best = nullptr; unsigned* ticket = nullptr;
    int* out_ring = nullptr; int ring_cap = 65536; int* h_out = nullptr;   // h_out holds ring_cap + 1 ints
    float* tp_partial = nullptr; unsigned long long* tp_keys = nullptr;
    // peer exchange (tensor parallel without collective calls): one receive block per rank, mapped into every peer
    unsigned char* tp_rx = nullptr; size_t tp_rx_bytes = 0; unsigned char* peer_rx[8] = {}; bool tp_peer = false;
    __half* x2 = nullptr; bool tp_sum_separate = false;
    unsigned char* gate_xd = nullptr; int* gate_corr = nullptr; float* gate_xscale = nullptr;    // SwiGLU output in staged form (see GemvArgs::xd_out)
    unsigned char* att_xd = nullptr; int* att_corr = nullptr; float* att_xscale = nullptr;       // attention output in staged form (see AttnArgs::xd_out)
    // batched prefill workspace (cuqwen_prefill), allocated at the first call for kPrefillChunk tokens
    __half *pf_x = nullptr, *pf_xn = nullptr, *pf_q = nullptr, *pf_att = nullptr, *pf_g = nullptr; float* pf_qkv = nullptr; int* pf_tok = nullptr;
    int steps_done = 0;                          // mirrors the device-side step counter (StepCtl::pad[1])
    std::vector<cudaEvent_t>* prof = nullptr;    // cuqwen_step_profile: an event is recorded after every launch of the step
    unsigned long long* step_trace = nullptr; size_t step_trace_bytes = 0;     // CUQWEN_FLAG_STEP_TRACE: eight timeline words per launch (tma.cuh)
    // graph
    cudaGraph_t graph = nullptr; cudaGraphExec_t gexec = nullptr; bool graph_ready = false;
    int launches = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr; float last_ms = 0.f;
    // nccl
    ncclComm_t comm = nullptr;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static size_t elem_bytes2(int quant, size_t rows, size_t cols) { return quant == 2 ? rows * cols / 2 : quant == 1 ? rows * cols : rows * cols * 2; }

extern "C" int cuqwen_create(const cuqwen_params* pin, cuqwen_engine** out) {
    if (!pin || !out) return fail(CUQWEN_ERR_ARG, "null argument");
    cuqwen_params p = *pin;
    if (p.model_id >= 0) {
        if (p.model_id > 4) return fail(CUQWEN_ERR_ARG, "model_id %d out of range", p.model_id);
        const ModelRow& m = kModels[p.model_id];
        p.vocab_size = m.vocab; p.dim = m.dim; p.intermediate_size = m.inter; p.n_layers = m.layers; p.n_heads = m.heads; p.n_kv_heads = m.kv; p.head_dim = m.hd;
    }
    if (p.max_seq_len <= 0) p.max_seq_len = 32768;
    if (p.tp_size <= 0) p.tp_size = 1;
    if (p.norm_eps == 0.f) p.norm_eps = 1e-6f;
    if (p.rope_theta == 0.f) p.rope_theta = 1000000.0f;
    if (p.repetition_penalty == 0.f) p.repetition_penalty = 1.1f;
    if (p.quant < 0 || p.quant > 2) return fail(CUQWEN_ERR_ARG, "quant %d out of range", p.quant);
    if (p.dim <= 0 || p.dim % 128 || p.intermediate_size <= 0 || p.intermediate_size % 128 || p.vocab_size <= 0 || p.vocab_size % 16 ||
        p.n_layers <= 0 || p.n_heads <= 0 || p.n_kv_heads <= 0 || p.n_heads % p.n_kv_heads || (p.head_dim != 64 && p.head_dim != 128) ||
        (p.n_heads * p.head_dim) % 128 || p.n_heads / p.n_kv_heads > kMaxGroup)
        return fail(CUQWEN_ERR_ARG, "unsupported dims: dim %d inter %d vocab %d layers %d heads %d/%d hd %d", p.dim, p.intermediate_size, p.vocab_size,
                    p.n_layers, p.n_heads, p.n_kv_heads, p.head_dim);
    if ((p.flags & CUQWEN_FLAG_KV_INT8) && p.max_seq_len % 4)
        return fail(CUQWEN_ERR_ARG, "the 8-bit KV cache needs max_seq_len to be a multiple of 4 (its row scales travel in 16-byte units); got %d", p.max_seq_len);
    // exchanges of a step are numbered 0 .. 2 * n_layers + 1 inside a window of kSeqPerStep numbers (common.cuh)
    if (p.tp_size > 1 && 2 * p.n_layers + 2 > (int)kSeqPerStep)
        return fail(CUQWEN_ERR_ARG, "tensor parallelism supports at most %d layers (this model has %d)", (int)kSeqPerStep / 2 - 1, p.n_layers);
    TpPlan plan;
    if (int r = tp_plan(p.n_heads, p.n_kv_heads, p.head_dim, p.intermediate_size, p.vocab_size, p.tp_rank, p.tp_size, &plan))
        return fail(CUQWEN_ERR_ARG, "model cannot be split over tp_size %d (rule %d)", p.tp_size, r);

    CK(cudaSetDevice(p.device));
    cuqwen_engine* e = new cuqwen_engine();
    e->p = p; e->plan = plan; e->tp = p.tp_size; e->rank = p.tp_rank;
    e->n_heads_l = plan.qh1 - plan.qh0; e->n_kv_l = plan.kvh1 - plan.kvh0;
    e->q_dim_l = e->n_heads_l * p.head_dim; e->kv_dim_l = e->n_kv_l * p.head_dim;
    e->inter_l = plan.i1 - plan.i0; e->vocab_l = plan.v1 - plan.v0;
    CK(cudaDeviceGetAttribute(&e->sms, cudaDevAttrMultiProcessorCount, p.device));
    // one CTA per SM and not one more: the partial kernel takes a whole SM's shared memory, so a 149th CTA would wait for
    // a second wave (measured at 40/8 heads, 32K keys: 19 splits 40.7 us, 16 splits 26.9 us)
    e->nsplit = p.attn_splits > 0 ? p.attn_splits : (e->sms / e->n_kv_l > 0 ? e->sms / e->n_kv_l : 1);
    if (e->nsplit > kMaxSplit) e->nsplit = kMaxSplit;
    CK(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    CK(cudaEventCreate(&e->ev0)); CK(cudaEventCreate(&e->ev1));

    auto dalloc = [&](void** ptr, size_t bytes) -> cudaError_t { cudaError_t r = cudaMalloc(ptr, bytes); if (r == cudaSuccess) r = cudaMemset(*ptr, 0, bytes); return r; };
    const size_t kvn = (size_t)p.n_layers * e->n_kv_l * p.max_seq_len * p.head_dim;
    CK(dalloc((void**)&e->x, p.dim * 2)); CK(dalloc((void**)&e->xn, p.dim * 2));
    CK(dalloc((void**)&e->q, e->q_dim_l * 2)); CK(dalloc((void**)&e->k, e->kv_dim_l * 2)); CK(dalloc((void**)&e->v, e->kv_dim_l * 2));
    CK(dalloc((void**)&e->att, e->q_dim_l * 2)); CK(dalloc((void**)&e->gate, e->inter_l * 2));
    { const size_t cb = ((size_t)(e->inter_l / kGroup) * 4 + 15) / 16 * 16; CK(dalloc((void**)&e->gate_xd, (size_t)e->inter_l * 2)); CK(dalloc((void**)&e->gate_corr, cb)); CK(dalloc((void**)&e->gate_xscale, cb)); } CK(dalloc((void**)&e->logits, e->vocab_l * 2));
    { const size_t cb = ((size_t)(e->q_dim_l / kGroup) * 4 + 15) / 16 * 16; CK(dalloc((void**)&e->att_xd, (size_t)e->q_dim_l * 2)); CK(dalloc((void**)&e->att_corr, cb)); CK(dalloc((void**)&e->att_xscale, cb)); }
    CK(dalloc((void**)&e->spare_up, (size_t)e->inter_l * 2)); CK(dalloc((void**)&e->spare_out, (size_t)p.dim * 2));
    e->kv8 = (p.flags & CUQWEN_FLAG_KV_INT8) != 0;
    if (e->kv8) {
        const size_t ns = (size_t)p.n_layers * e->n_kv_l * p.max_seq_len + 16;       // room for the bulk copies' 16-byte rounding past the last row
        CK(dalloc((void**)&e->kc, kvn)); CK(dalloc((void**)&e->vc, kvn));
        CK(dalloc((void**)&e->kscale, ns * 4)); CK(dalloc((void**)&e->vscale, ns * 4));
    } else {
        CK(dalloc((void**)&e->kc, kvn * 2)); CK(dalloc((void**)&e->vc, kvn * 2));     // zeroed like src/model.cu:37-38
    }
    CK(dalloc((void**)&e->part_o, attn_scratch_floats_o(e->n_kv_l, e->nsplit, p.head_dim) * 4));
    CK(dalloc((void**)&e->part_ml, attn_scratch_floats_ml(e->n_kv_l, e->nsplit) * 4));
    CK(dalloc((void**)&e->counters, attn_scratch_counters(e->n_kv_l, e->nsplit) * 4));
    CK(dalloc((void**)&e->ctl, sizeof(StepCtl))); CK(cudaMallocHost((void**)&e->h_ctl, sizeof(StepCtl)));
    CK(cudaHostAlloc((void**)&e->hio, sizeof(HostIo), cudaHostAllocMapped));
    memset(e->hio, 0, sizeof(HostIo));
    CK(cudaHostGetDevicePointer((void**)&e->hio_dev, e->hio, 0));
    CK(dalloc((void**)&e->d_hist, (size_t)p.max_seq_len * 4));
    CK(dalloc((void**)&e->bitmap, ((size_t)e->vocab_l + 31) / 32 * 4));
    CK(dalloc((void**)&e->best, 8)); CK(dalloc((void**)&e->ticket, 4));
    CK(dalloc((void**)&e->out_ring, (size_t)e->ring_cap * 4)); CK(cudaMallocHost((void**)&e->h_out, ((size_t)e->ring_cap + 1) * 4));
    if (e->tp > 1) { CK(dalloc((void**)&e->tp_partial, (size_t)p.dim * 4)); CK(dalloc((void**)&e->tp_keys, (size_t)(e->tp + 1) * 8)); }
    *out = e;
    return CUQWEN_OK;
}

extern "C" void cuqwen_destroy(cuqwen_engine* e) {
    if (!e) return;
    cudaSetDevice(e->p.device);
    cudaStreamSynchronize(e->stream);
    if (e->gexec) cudaGraphExecDestroy(e->gexec);
    if (e->graph) cudaGraphDestroy(e->graph);
    for (int r = 0; r < 8; ++r) if (e->peer_rx[r] && e->peer_rx[r] != e->tp_rx) cudaIpcCloseMemHandle(e->peer_rx[r]);
    if (e->tp_rx) cudaFree(e->tp_rx);
    if (e->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(e->comm);
    void* bufs[] = {e->x, e->xn, e->q, e->k, e->v, e->att, e->gate, e->logits, e->kc, e->vc, e->part_o, e->part_ml, e->counters, e->ctl, e->d_hist,
                    e->bitmap, e->best, e->ticket, e->out_ring, e->tp_partial, e->tp_keys, e->warena, e->step_trace, e->spare_up, e->spare_out, e->kscale, e->vscale, e->x2, e->gate_xd, e->gate_corr, e->gate_xscale, e->att_xd, e->att_corr, e->att_xscale,
                    e->pf_x, e->pf_xn, e->pf_q, e->pf_att, e->pf_g, e->pf_qkv, e->pf_tok};
    for (void* b : bufs) if (b) cudaFree(b);
    if (e->h_ctl) cudaFreeHost(e->h_ctl);
    if (e->hio) cudaFreeHost(e->hio);
    if (e->h_out) cudaFreeHost(e->h_out);
    cudaEventDestroy(e->ev0); cudaEventDestroy(e->ev1);
    cudaStreamDestroy(e->stream);
    delete e;
}

// ---------------------------------------------------------------------------
// loader (file layout: export_weights.py:267-323; validation: src/load_weights.cpp:46-84)
// ---------------------------------------------------------------------------
namespace {
struct Slice { size_t r0, r1, c0, c1; };   // rows [r0,r1), cols [c0,c1) of a [rows, cols] matrix
struct Cursor {
    const uint8_t* base; size_t size, off;
    bool take(size_t n, const uint8_t** ptr) { if (off + n > size) return false; *ptr = base + off; off += n; return true; }
};
struct Arena {
    uint8_t* base = nullptr; size_t used = 0; bool dry = true;
    void* get(size_t bytes) { size_t o = used; used = align_up(used + bytes, 256); return dry ? (void*)(uintptr_t)(o + 256) : base + o; }
};
}  // namespace

// Copies the slice of a projection (weights + scales) from the file image into the arena.
static int load_proj(Cursor& cur, Arena& ar, int quant, size_t rows, size_t cols, const Slice& sl, Mat* m, uint64_t* bytes) {
    const uint8_t* wsrc; const uint8_t* ssrc = nullptr;
    if (!cur.take(elem_bytes2(quant, rows, cols), &wsrc)) return CUQWEN_ERR_IO;
    if (quant && !cur.take(rows * (cols / kGroup) * 2, &ssrc)) return CUQWEN_ERR_IO;
    const size_t nr = sl.r1 - sl.r0, nc = sl.c1 - sl.c0;
    const size_t src_pitch = elem_bytes2(quant, 1, cols), dst_pitch = elem_bytes2(quant, 1, nc), c0b = elem_bytes2(quant, 1, sl.c0);
    m->rows = (int)nr; m->cols = (int)nc;
    m->w = (uint8_t*)ar.get(nr * dst_pitch);
    m->s = quant ? (__half*)ar.get(nr * (nc / kGroup) * 2) : nullptr;
    *bytes += nr * dst_pitch + (quant ? nr * (nc / kGroup) * 2 : 0);
    if (ar.dry) return CUQWEN_OK;
    if (cudaMemcpy2D(m->w, dst_pitch, wsrc + sl.r0 * src_pitch + c0b, src_pitch, dst_pitch, nr, cudaMemcpyHostToDevice) != cudaSuccess) return CUQWEN_ERR_CUDA;
    if (quant) {
        const size_t sp = (cols / kGroup) * 2, dp = (nc / kGroup) * 2;
        if (cudaMemcpy2D(m->s, dp, ssrc + sl.r0 * sp + (sl.c0 / kGroup) * 2, sp, dp, nr, cudaMemcpyHostToDevice) != cudaSuccess) return CUQWEN_ERR_CUDA;
    }
    return CUQWEN_OK;
}
static int load_vec(Cursor& cur, Arena& ar, size_t n, size_t e0, size_t e1, __half** dst, uint64_t* bytes) {
    const uint8_t* src;
    if (!cur.take(n * 2, &src)) return CUQWEN_ERR_IO;
    *dst = (__half*)ar.get((e1 - e0) * 2);
    *bytes += (e1 - e0) * 2;
    if (ar.dry) return CUQWEN_OK;
    return cudaMemcpy(*dst, src + e0 * 2, (e1 - e0) * 2, cudaMemcpyHostToDevice) == cudaSuccess ? CUQWEN_OK : CUQWEN_ERR_CUDA;
}

// One walk over the file; dry = size the arena only.
static int walk_file(cuqwen_engine* e, Cursor cur, Arena& ar, int lm_fmt) {
    const cuqwen_params& p = e->p; const TpPlan& pl = e->plan;
    const size_t d = p.dim, hd = p.head_dim, qd = (size_t)p.n_heads * hd, kd = (size_t)p.n_kv_heads * hd, I = p.intermediate_size, V = p.vocab_size;
    const int Q = p.quant;
    uint64_t wb = 0, dummy = 0;
    int r;
#define TRY(x) do { r = (x); if (r) return r; } while (0)
    TRY(load_vec(cur, ar, V * d, 0, V * d, &e->embed, &dummy));
    e->layers.resize(p.n_layers);
    for (int l = 0; l < p.n_layers; ++l) {
        Layer& L = e->layers[l];
        TRY(load_vec(cur, ar, d, 0, d, &L.in_norm, &wb));
        TRY(load_proj(cur, ar, Q, qd, d, Slice{pl.qh0 * hd, pl.qh1 * hd, 0, d}, &L.q, &wb));
        TRY(load_vec(cur, ar, qd, pl.qh0 * hd, pl.qh1 * hd, &L.bq, &wb));
        TRY(load_proj(cur, ar, Q, kd, d, Slice{pl.kvh0 * hd, pl.kvh1 * hd, 0, d}, &L.k, &wb));
        TRY(load_vec(cur, ar, kd, pl.kvh0 * hd, pl.kvh1 * hd, &L.bk, &wb));
        TRY(load_proj(cur, ar, Q, kd, d, Slice{pl.kvh0 * hd, pl.kvh1 * hd, 0, d}, &L.v, &wb));
        TRY(load_vec(cur, ar, kd, pl.kvh0 * hd, pl.kvh1 * hd, &L.bv, &wb));
        TRY(load_proj(cur, ar, Q, d, qd, Slice{0, d, pl.qh0 * hd, pl.qh1 * hd}, &L.o, &wb));
        TRY(load_vec(cur, ar, d, 0, d, &L.post_norm, &wb));
        TRY(load_proj(cur, ar, Q, I, d, Slice{(size_t)pl.i0, (size_t)pl.i1, 0, d}, &L.gate, &wb));
        TRY(load_proj(cur, ar, Q, I, d, Slice{(size_t)pl.i0, (size_t)pl.i1, 0, d}, &L.up, &wb));
        TRY(load_proj(cur, ar, Q, d, I, Slice{0, d, (size_t)pl.i0, (size_t)pl.i1}, &L.down, &wb));
    }
    TRY(load_vec(cur, ar, d, 0, d, &e->norm, &wb));
    if (lm_fmt == 1) {
        TRY(load_proj(cur, ar, 1, V, d, Slice{(size_t)pl.v0, (size_t)pl.v1, 0, d}, &e->lm, &wb));
        e->lm_quant = 1; e->lm_kind = 1;
    } else if (cur.size - cur.off >= V * d * 2) {      // untied fp16 head detected by remaining length (src/load_weights.cpp:148-156)
        TRY(load_proj(cur, ar, 0, V, d, Slice{(size_t)pl.v0, (size_t)pl.v1, 0, d}, &e->lm, &wb));
        e->lm_quant = 0; e->lm_kind = 0;
    } else {                                           // tied: alias the embedding rows (src/load_weights.cpp:157-160)
        e->lm.w = (uint8_t*)(e->embed + (size_t)pl.v0 * d); e->lm.s = nullptr; e->lm.rows = pl.v1 - pl.v0; e->lm.cols = (int)d;
        e->lm_quant = 0; e->lm_kind = 2;
        wb += (uint64_t)(pl.v1 - pl.v0) * d * 2;
    }
#undef TRY
    e->weight_bytes = wb + d * 2;    // + one embedding row
    return CUQWEN_OK;
}

extern "C" int cuqwen_load(cuqwen_engine* e, const char* path) {
    if (!e || !path) return fail(CUQWEN_ERR_ARG, "null argument");
    if (e->loaded) return fail(CUQWEN_ERR_STATE, "weights already loaded");
    CK(cudaSetDevice(e->p.device));
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(CUQWEN_ERR_IO, "cannot open binary file at: %s", path);
    struct stat st; fstat(fd, &st);
    const size_t size = (size_t)st.st_size;
    if (size < 11 * 4) { close(fd); return fail(CUQWEN_ERR_IO, "failed to read binary weight header"); }
    void* map = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return fail(CUQWEN_ERR_IO, "mmap failed for %s", path);
    struct Unmap { void* p; size_t n; ~Unmap() { munmap(p, n); } } unmap{map, size};
    int32_t h[11]; memcpy(h, map, sizeof h);
    const cuqwen_params& p = e->p;
    if (h[0] != 0x5157454E) return fail(CUQWEN_ERR_MAGIC, "magic number mismatch: expected 0x5157454e, found 0x%x", h[0]);
    if (h[1] != p.vocab_size || h[2] != p.dim || h[3] != p.intermediate_size || h[4] != p.n_layers || h[5] != p.n_heads || h[6] != p.n_kv_heads || h[7] != p.head_dim)
        return fail(CUQWEN_ERR_DIMS, "binary header dimensions do not match the engine configuration");
    if (h[9] != p.quant) return fail(CUQWEN_ERR_QUANT, "quantization mismatch: engine is %d, file is %d", p.quant, h[9]);
    if (size < 256) return fail(CUQWEN_ERR_IO, "unexpected end of file while reading tensor data");
    Cursor cur{(const uint8_t*)map, size, 256};
    Arena dry;
    int r = walk_file(e, cur, dry, h[10]);
    if (r) return fail(r, r == CUQWEN_ERR_IO ? "unexpected end of file while reading tensor data" : "load failed");
    e->warena_bytes = dry.used + 256;
    CK(cudaMalloc((void**)&e->warena, e->warena_bytes));
    Arena real; real.base = e->warena; real.dry = false;
    r = walk_file(e, cur, real, h[10]);
    if (r) { cudaFree(e->warena); e->warena = nullptr; return fail(r, "copying weights to the device failed: %s", cudaGetErrorString(cudaGetLastError())); }
    CK(cudaDeviceSynchronize());
    if (e->p.flags & CUQWEN_FLAG_STEP_TRACE) {      // eight timeline words per launch, zeroed by the reader between steps
        e->step_trace_bytes = (size_t)(1 + 8 * e->p.n_layers + 8) * kTraceWords * 8;
        CK(cudaMalloc((void**)&e->step_trace, e->step_trace_bytes));
        CK(cudaMemset(e->step_trace, 0, e->step_trace_bytes));
    }
    e->loaded = true;
    return CUQWEN_OK;
}

// ---------------------------------------------------------------------------
// one decode step as a sequence of launches (order: reference src/model.cu:76-181)
// ---------------------------------------------------------------------------
static GemvArgs gv(const __half* x, int K) { GemvArgs a; memset(&a, 0, sizeof a); a.x = x; a.K = K; a.err = t_err; return a; }

static int tp_allreduce(cuqwen_engine* e, float* buf, int n, cudaStream_t s) {
    NK(g_nccl.AllReduce(buf, buf, n, ncclFloat32, ncclSum, e->comm, s));
    return CUQWEN_OK;
}

// The matrix and attention work of one step, in order.  `reduce`: a row-parallel matrix whose fp32 partial must be
// summed over the tensor-parallel ranks and added to the residual stream afterwards.
enum PhaseKind : int { PH_GEMV = 0, PH_ATTN = 1 };
struct Phase { GemvArgs g; AttnArgs at; int kind, quant, epi; };
struct HostPhase {
    Phase ph; bool reduce;
    // peer exchange with many ranks: after this (pushing) matrix a small kernel sums the slots once into sum_dst
    bool sum_after; const __half* sum_src; __half* sum_dst; const void* sum_slots; int sum_seq;
};

static void describe_step(cuqwen_engine* e, std::vector<HostPhase>& out, int nsplit) {
    const cuqwen_params& p = e->p;
    const size_t kv_layer = (size_t)e->n_kv_l * p.max_seq_len * p.head_dim;
    const float eps = __half2float(__float2half(p.norm_eps));   // the reference narrows eps to fp16 (src/model.cu:96)
    auto gemv_phase = [&](int quant, int epi, const GemvArgs& a, bool reduce) {
        HostPhase h; memset(&h, 0, sizeof h);
        h.ph.kind = PH_GEMV; h.ph.quant = quant; h.ph.epi = epi; h.ph.g = a; h.reduce = reduce;
        out.push_back(h);
    };
    // Peer-exchange bookkeeping (tensor parallel): `cur` is the buffer that holds the residual stream, `pending` the
    // exchange whose partials still have to be added to it by the next kernel that reads it.
    const bool peer = e->tp > 1 && e->tp_peer;
    // SwiGLU output handed to the down projection in staged form: only when the gate/up launch will work on whole
    // 128-row groups, which the launcher decides from the row count
    const bool hand_over = p.quant != 0 && !(p.flags & CUQWEN_FLAG_NO_HANDOVER) && e->inter_l % 128 == 0 &&
                           gemv_block_rows(e->inter_l, p.dim, e->sms, EPI_SWIGLU) == 128;
    // attention output handed to o_proj in staged form: a head of 128 values is one scale group
    const bool att_hand_over = p.quant != 0 && p.head_dim == 128 && !(p.flags & CUQWEN_FLAG_NO_HANDOVER);
    __half* cur = e->x;
    int pending = -1, next_xi = 0;
    auto take_x = [&](GemvArgs& a) {                                        // a normed GEMV reads the residual stream
        a.x = cur;
        if (peer && pending >= 0 && !e->tp_sum_separate) {
            const int slot = pending & 1;
            __half* other = cur == e->x ? e->x2 : e->x;
            a.ngather = e->tp; a.gather = reinterpret_cast<const uint2*>(e->tp_rx) + (size_t)slot * e->tp * p.dim;
            a.x_next = other; a.step_no = &e->ctl->pad[1]; a.seq_index = pending;
            cur = other; pending = -1;
        }
    };
    auto push_to = [&](GemvArgs& a) {                                       // a row-parallel matrix hands its partial to every rank
        const int slot = next_xi & 1;
        a.npush = e->tp; a.step_no = &e->ctl->pad[1]; a.seq_index = next_xi;
        for (int d = 0; d < e->tp; ++d) a.push[d] = reinterpret_cast<uint2*>(e->peer_rx[d]) + ((size_t)slot * e->tp + e->rank) * p.dim;
        pending = next_xi++;
    };
    auto sum_after_push = [&]() {                                           // many ranks: one kernel sums the slots, the next GEMV reads x plainly
        if (!(peer && e->tp_sum_separate)) return;
        HostPhase& h = out.back();
        __half* other = cur == e->x ? e->x2 : e->x;
        h.sum_after = true; h.sum_src = cur; h.sum_dst = other; h.sum_seq = pending;
        h.sum_slots = reinterpret_cast<const uint2*>(e->tp_rx) + (size_t)(pending & 1) * e->tp * p.dim;
        cur = other; pending = -1;
    };
    for (int l = 0; l < p.n_layers; ++l) {
        const Layer& L = e->layers[l];
        {   // RMSNorm + QKV + bias + RoPE + KV store
            GemvArgs a = gv(e->x, p.dim);
            take_x(a);
            a.norm_w = L.in_norm; a.eps = eps;
            a.w[0] = L.q.w; a.w[1] = L.k.w; a.w[2] = L.v.w; a.s[0] = L.q.s; a.s[1] = L.k.s; a.s[2] = L.v.s;
            a.bias[0] = L.bq; a.bias[1] = L.bk; a.bias[2] = L.bv;
            a.q_out = e->q; a.k_out = e->k; a.v_out = e->v;
            if (!e->kv8) { a.kcache = e->kc + l * kv_layer; a.vcache = e->vc + l * kv_layer; }     // 8-bit cache: the attention kernel stores the row
            a.d_pos = &e->ctl->pos; a.n_heads = e->n_heads_l; a.n_kv = e->n_kv_l; a.hd = p.head_dim; a.max_seq = p.max_seq_len;
            a.theta = p.rope_theta; a.rope_fast = (p.flags & CUQWEN_FLAG_ACCURATE_ROPE) ? 0 : 1;
            gemv_phase(p.quant, EPI_QKV, a, false);
        }
        {   // split-KV attention + combine
            HostPhase h; memset(&h, 0, sizeof h);
            AttnArgs& a = h.ph.at;
            a.q = e->q; a.out = e->att; a.d_pos = &e->ctl->pos;
            if (e->kv8) {
                const size_t srow = (size_t)l * e->n_kv_l * p.max_seq_len;
                a.kc = reinterpret_cast<const __half*>(reinterpret_cast<const signed char*>(e->kc) + l * kv_layer);
                a.vc = reinterpret_cast<const __half*>(reinterpret_cast<const signed char*>(e->vc) + l * kv_layer);
                a.kscale = e->kscale + srow; a.vscale = e->vscale + srow; a.k_cur = e->k; a.v_cur = e->v;
            } else { a.kc = e->kc + l * kv_layer; a.vc = e->vc + l * kv_layer; }
            a.n_kv = e->n_kv_l; a.grp = e->plan.grp; a.max_seq = p.max_seq_len; a.nsplit = nsplit;
            a.scale_log2 = (1.0f / sqrtf((float)p.head_dim)) * 1.4426950408889634f;
            a.part_o = e->part_o; a.part_ml = e->part_ml; a.counters = e->counters; a.err = t_err;
            if (att_hand_over) { a.xd_out = e->att_xd; a.corr_out = e->att_corr; a.xscale_out = e->att_xscale; a.quant_out = p.quant; }
            h.ph.kind = PH_ATTN;
            out.push_back(h);
        }
        {   // o_proj + residual
            GemvArgs a = gv(e->att, e->q_dim_l);
            a.w[0] = L.o.w; a.s[0] = L.o.s; a.rows = p.dim;
            if (att_hand_over) { a.xd_in = e->att_xd; a.corr_in = e->att_corr; a.xscale_in = e->att_xscale; }
            if (e->tp == 1) { a.out_h = e->x; gemv_phase(p.quant, EPI_RESID, a, false); }
            else if (peer) { push_to(a); gemv_phase(p.quant, EPI_PUSH, a, false); sum_after_push(); }
            else { a.out_f = e->tp_partial; gemv_phase(p.quant, EPI_F32, a, true); }
        }
        {   // RMSNorm + gate/up + SwiGLU
            GemvArgs a = gv(e->x, p.dim);
            take_x(a);
            a.norm_w = L.post_norm; a.eps = eps;
            a.w[0] = L.gate.w; a.w[1] = L.up.w; a.s[0] = L.gate.s; a.s[1] = L.up.s; a.rows = e->inter_l; a.out_h = e->gate;
            if (hand_over) { a.xd_out = e->gate_xd; a.corr_out = e->gate_corr; a.xscale_out = e->gate_xscale; }
            gemv_phase(p.quant, EPI_SWIGLU, a, false);
        }
        {   // down + residual
            GemvArgs a = gv(e->gate, e->inter_l);
            a.w[0] = L.down.w; a.s[0] = L.down.s; a.rows = p.dim;
            if (hand_over) { a.xd_in = e->gate_xd; a.corr_in = e->gate_corr; a.xscale_in = e->gate_xscale; }
            if (e->tp == 1) { a.out_h = e->x; gemv_phase(p.quant, EPI_RESID, a, false); }
            else if (peer) { push_to(a); gemv_phase(p.quant, EPI_PUSH, a, false); sum_after_push(); }
            else { a.out_f = e->tp_partial; gemv_phase(p.quant, EPI_F32, a, true); }
        }
    }
    {   // final RMSNorm + lm_head
        GemvArgs a = gv(e->x, p.dim);
        take_x(a);
        a.norm_w = e->norm; a.eps = eps; a.w[0] = e->lm.w; a.s[0] = e->lm.s; a.rows = e->vocab_l; a.out_h = e->logits;
        gemv_phase(e->lm_quant, EPI_F16, a, false);
    }
    // Each GEMV warms L2 with the small tensors of the next GEMV that normalises its input: its RMSNorm weight and, for
    // the q/k/v kernel, the biases.
    for (size_t i = 0; i < out.size(); ++i) {
        if (out[i].ph.kind != PH_GEMV) continue;
        for (size_t j = i + 1; j < out.size(); ++j) {
            if (out[j].ph.kind != PH_GEMV) continue;
            const GemvArgs& nx = out[j].ph.g;
            GemvArgs& me = out[i].ph.g;
            if (nx.norm_w) { me.warm[0] = nx.norm_w; me.warm_bytes[0] = nx.K * 2; }
            if (out[j].ph.epi == EPI_QKV) {
                me.warm[1] = nx.bias[0]; me.warm_bytes[1] = nx.n_heads * nx.hd * 2;
                me.warm[2] = nx.bias[1]; me.warm_bytes[2] = nx.n_kv * nx.hd * 2;           // (the v bias, as small, is left to its first use)
            }
            break;
        }
    }
}

static int record_step(cuqwen_engine* e, cudaStream_t s, bool pdl) {
    const cuqwen_params& p = e->p;
    LaunchCfg cfg{s, e->sms, pdl};
    LaunchCfg cfg_plain{s, e->sms, false};
    t_err = reinterpret_cast<unsigned*>(&e->ctl->pad[0]);
    int n = 0;
    const float pen = __half2float(__float2half(p.repetition_penalty));
#define MARK() do { if (e->prof) { cudaEvent_t ev_; CK(cudaEventCreate(&ev_)); CK(cudaEventRecord(ev_, s)); e->prof->push_back(ev_); } } while (0)
#define LK(call) do { int r_ = (call); if (r_) return fail(CUQWEN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString((cudaError_t)r_)); ++n; MARK(); } while (0)
    MARK();
    LK(launch_embed_step(e->embed, e->ctl, e->x, p.dim, cfg_plain));
    {
        std::vector<HostPhase> hp;
        describe_step(e, hp, e->nsplit);
        for (HostPhase& h : hp) {
            unsigned long long* tr = e->step_trace && (size_t)(n + 2) * kTraceWords * 8 <= e->step_trace_bytes ? e->step_trace + (size_t)n * kTraceWords : nullptr;
            if (h.ph.kind == PH_ATTN) { h.ph.at.trace = tr; LK(launch_attn(p.head_dim, h.ph.at, cfg)); ++n; continue; }      // two launches: partials, fold
            h.ph.g.trace = tr;
            LK(launch_gemv(h.ph.quant, h.ph.epi, h.ph.g, cfg));
            if (h.sum_after) LK(launch_tp_sum(h.sum_src, h.sum_dst, h.sum_slots, e->tp, p.dim, &e->ctl->pad[1], h.sum_seq, t_err, 0, cfg));
            if (h.reduce) {
                if (int r = tp_allreduce(e, e->tp_partial, p.dim, s)) return r; ++n; MARK();
                LK(launch_resid_sum(e->x, e->tp_partial, 1, 0, p.dim, cfg_plain));
            }
        }
    }
    LK(launch_penalty(e->logits, e->d_hist, &e->ctl->hist_len, e->vocab_l, e->plan.v0, pen, e->bitmap, cfg));
    if (e->tp == 1) {
        LK(launch_argmax(e->logits, e->vocab_l, 0, e->ctl, e->out_ring, e->ring_cap, e->d_hist, e->bitmap, e->best, e->ticket, nullptr, nullptr, cfg));
    } else if (e->tp_peer) {
        // every rank stores its best (value, index) key straight into every rank's key slots; no collective call
        unsigned long long* slots[8];
        const size_t keys_off = (size_t)2 * e->tp * p.dim * 8;          // the key words follow the partial-sum slots in the receive block
        for (int d = 0; d < e->tp; ++d) slots[d] = reinterpret_cast<unsigned long long*>(e->peer_rx[d] + keys_off) + e->rank;
        LK(launch_argmax(e->logits, e->vocab_l, e->plan.v0, e->ctl, e->out_ring, e->ring_cap, e->d_hist, e->bitmap, e->best, e->ticket, nullptr, nullptr, cfg, slots, e->tp));
        LK(launch_merge_pushed_keys(reinterpret_cast<const unsigned long long*>(e->tp_rx + keys_off), e->tp, e->ctl, e->out_ring, e->ring_cap, t_err, 0, cfg));
    } else {
        LK(launch_argmax(e->logits, e->vocab_l, e->plan.v0, e->ctl, e->out_ring, e->ring_cap, e->d_hist, e->bitmap, e->best, e->ticket, e->tp_keys + e->tp, nullptr, cfg));
        NK(g_nccl.AllGather(e->tp_keys + e->tp, e->tp_keys, 1, ncclUint64, e->comm, s)); ++n; MARK();
        LK(launch_merge_keys(e->tp_keys, e->tp, e->ctl, e->out_ring, e->ring_cap, cfg_plain));
    }
#undef LK
#undef MARK
    e->launches = n;
    return CUQWEN_OK;
}

static int ensure_graph(cuqwen_engine* e) {
    if (e->graph_ready || (e->p.flags & CUQWEN_FLAG_NO_GRAPH)) return CUQWEN_OK;
    const bool pdl = !(e->p.flags & CUQWEN_FLAG_NO_PDL);
    CK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    int r = record_step(e, e->stream, pdl);
    cudaGraph_t g = nullptr;
    cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
    if (r) { if (g) cudaGraphDestroy(g); return r; }
    CK(ce);
    e->graph = g;
    CK(cudaGraphInstantiate(&e->gexec, e->graph, 0));
    e->graph_ready = true;
    return CUQWEN_OK;
}

static int run_step(cuqwen_engine* e) {
    if (e->p.flags & CUQWEN_FLAG_NO_GRAPH) return record_step(e, e->stream, !(e->p.flags & CUQWEN_FLAG_NO_PDL));
    CK(cudaGraphLaunch(e->gexec, e->stream));
    return CUQWEN_OK;
}

extern "C" int cuqwen_step(cuqwen_engine* e, int token, int pos, const int* history, int history_len, int* out_token) {
    if (!e) return fail(CUQWEN_ERR_ARG, "null engine");
    if (!e->loaded) return fail(CUQWEN_ERR_STATE, "cuqwen_step before cuqwen_load");
    if (e->tp > 1 && !e->comm) return fail(CUQWEN_ERR_STATE, "cuqwen_step before cuqwen_tp_init");
    if (token < 0 || token >= e->p.vocab_size || pos < 0 || pos >= e->p.max_seq_len || history_len < 0 || history_len > e->p.max_seq_len)
        return fail(CUQWEN_ERR_ARG, "token %d / pos %d / history_len %d out of range", token, pos, history_len);
    CK(cudaSetDevice(e->p.device));
    if (int r = ensure_graph(e)) return r;
    const int hist_len = (history && history_len > 0) ? history_len : 0;
    if (e->ctl_dirty) {         // after cuqwen_decode_n / a profile run / an error: the device block is put back into the host-fed state once
        StepCtl c{}; c.pad[1] = e->steps_done; c.io_seq = e->io_seq; c.hio = e->hio_dev;
        *e->h_ctl = c;
        CK(cudaMemcpyAsync(e->ctl, e->h_ctl, sizeof(StepCtl), cudaMemcpyHostToDevice, e->stream));
        e->ctl_dirty = false;
    }
    if (hist_len) CK(cudaMemcpyAsync(e->d_hist, history, (size_t)hist_len * 4, cudaMemcpyHostToDevice, e->stream));
    // token, position and history length travel through the mailbox: no copy call on the way in, none on the way out
    HostIo* h = e->hio;
    e->io_seq += 1;
    h->token = token; h->pos = pos; h->hist_len = hist_len;
    __atomic_thread_fence(__ATOMIC_RELEASE);
    *(volatile int*)&h->seq_in = e->io_seq;
    if (int r = run_step(e)) { e->ctl_dirty = true; return r; }
    e->steps_done += 1;
    bool got = false;
    for (long spins = 0; ; ++spins) {
        if (h->seq_out == e->io_seq) { got = true; break; }
        if ((spins & 0x3fff) == 0x3fff) {            // now and then ask the driver: an idle stream without a result, or a fault, ends the wait
            const cudaError_t q = cudaStreamQuery(e->stream);
            if (q == cudaSuccess) { got = h->seq_out == e->io_seq; break; }
            if (q != cudaErrorNotReady) { e->ctl_dirty = true; return fail(CUQWEN_ERR_CUDA, "cuqwen_step: %s", cudaGetErrorString(q)); }
        }
    }
    __atomic_thread_fence(__ATOMIC_ACQUIRE);
    int tok, err;
    if (got) { tok = h->sampled; err = h->err; }
    else {                      // the step finished without posting (cannot happen with the kernels of this library): read the block itself
        CK(cudaMemcpyAsync(e->h_out, &e->ctl->sampled, 8, cudaMemcpyDeviceToHost, e->stream));
        CK(cudaStreamSynchronize(e->stream));
        tok = e->h_out[0]; err = e->h_out[1];
    }
    if (err) { e->ctl_dirty = true; return fail(CUQWEN_ERR_TIMEOUT, "a bounded device-side wait expired (code %d)", err); }
    if (out_token) *out_token = tok;
    return CUQWEN_OK;
}

// ---------------------------------------------------------------------------
// batched prefill: the prompt's tokens go through every layer as tiles, the KV cache rows [pos0, pos0 + n) come out.
// The reference runs qwen_forward once per prompt token for the same effect (src/main.cu:86-92).
// ---------------------------------------------------------------------------
constexpr int kPrefillChunk = 2048;
#define PK(call) do { int r_ = (call); if (r_) return fail(r_ == (int)cudaErrorInvalidValue ? CUQWEN_ERR_ARG : CUQWEN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString((cudaError_t)r_)); } while (0)

static int prefill_gemm(cuqwen_engine* e, int mode, const __half* x, const Mat* const* mats, int nmat, void* out, int T, int ldo) {
    PfGemmArgs a; memset(&a, 0, sizeof a);
    const void* w[3] = {nullptr, nullptr, nullptr}; int rows[3] = {0, 0, 0};
    for (int m = 0; m < nmat; ++m) { w[m] = mats[m]->w; rows[m] = mats[m]->rows; a.s[m] = mats[m]->s; }
    a.out_h = (__half*)out; a.out_f = (float*)out; a.T = T; a.K = mats[0]->cols; a.ldo = ldo; a.mode = mode; a.err = t_err;
    PK(launch_prefill_gemm(e->p.quant, a, x, w, rows, nmat, e->stream));
    return CUQWEN_OK;
}

extern "C" int cuqwen_prefill(cuqwen_engine* e, const int* tokens, int n_tokens, int pos0) {
    if (!e || !tokens) return fail(CUQWEN_ERR_ARG, "null argument");
    if (!e->loaded) return fail(CUQWEN_ERR_STATE, "cuqwen_prefill before cuqwen_load");
    if (e->tp > 1) return fail(CUQWEN_ERR_ARG, "cuqwen_prefill runs on one GPU (tp_size 1); feed the prompt through cuqwen_step on tensor-parallel engines");
    if (e->kv8) return fail(CUQWEN_ERR_ARG, "cuqwen_prefill writes the fp16 KV cache; not available with CUQWEN_FLAG_KV_INT8");
    const cuqwen_params& p = e->p;
    if (n_tokens < 1 || pos0 < 0 || pos0 + n_tokens > p.max_seq_len) return fail(CUQWEN_ERR_ARG, "prefill range [%d, %d) outside the cache", pos0, pos0 + n_tokens);
    if (p.head_dim != 64 && p.head_dim != 128) return fail(CUQWEN_ERR_ARG, "cuqwen_prefill supports head_dim 64 and 128");
    for (int i = 0; i < n_tokens; ++i) if (tokens[i] < 0 || tokens[i] >= p.vocab_size) return fail(CUQWEN_ERR_ARG, "token %d out of range", tokens[i]);
    CK(cudaSetDevice(p.device));
    t_err = reinterpret_cast<unsigned*>(&e->ctl->pad[0]);
    const int qd = e->q_dim_l, kd = e->kv_dim_l, C = kPrefillChunk;
    if (!e->pf_x) {
        CK(cudaMalloc((void**)&e->pf_x, (size_t)C * p.dim * 2)); CK(cudaMalloc((void**)&e->pf_xn, (size_t)C * p.dim * 2));
        CK(cudaMalloc((void**)&e->pf_qkv, (size_t)C * (qd + 2 * kd) * 4)); CK(cudaMalloc((void**)&e->pf_q, (size_t)C * qd * 2));
        CK(cudaMalloc((void**)&e->pf_att, (size_t)C * qd * 2)); CK(cudaMalloc((void**)&e->pf_g, (size_t)C * e->inter_l * 2));
        CK(cudaMalloc((void**)&e->pf_tok, (size_t)C * 4));
    }
    const size_t kv_layer = (size_t)e->n_kv_l * p.max_seq_len * p.head_dim;
    const float eps = __half2float(__float2half(p.norm_eps));
    const int ldqkv = qd + 2 * kd;
    CK(cudaMemsetAsync(&e->ctl->pad[0], 0, 4, e->stream));
    CK(cudaEventRecord(e->ev0, e->stream));
    for (int c0 = 0; c0 < n_tokens; c0 += C) {
        const int T = n_tokens - c0 < C ? n_tokens - c0 : C, pos = pos0 + c0;
        CK(cudaMemcpyAsync(e->pf_tok, tokens + c0, (size_t)T * 4, cudaMemcpyHostToDevice, e->stream));
        PK(launch_pf_embed(e->embed, e->pf_tok, e->pf_x, T, p.dim, e->stream));
        for (int l = 0; l < p.n_layers; ++l) {
            const Layer& L = e->layers[l];
            PK(launch_pf_rmsnorm(e->pf_x, L.in_norm, e->pf_xn, T, p.dim, eps, e->stream));
            const Mat* qkv[3] = {&L.q, &L.k, &L.v}, *om[1] = {&L.o}, *gu[2] = {&L.gate, &L.up}, *dm[1] = {&L.down};
            if (int r = prefill_gemm(e, PF_OUT_F32, e->pf_xn, qkv, 3, e->pf_qkv, T, ldqkv)) return r;        // one launch: q, k, v side by side
            PfRopeArgs ra; memset(&ra, 0, sizeof ra);
            ra.qkv = e->pf_qkv; ra.bq = L.bq; ra.bk = L.bk; ra.bv = L.bv; ra.q_out = e->pf_q;
            ra.kcache = e->kc + l * kv_layer; ra.vcache = e->vc + l * kv_layer;
            ra.pos0 = pos; ra.n_heads = e->n_heads_l; ra.n_kv = e->n_kv_l; ra.hd = p.head_dim; ra.q_dim = qd; ra.kv_dim = kd; ra.max_seq = p.max_seq_len;
            ra.rope_fast = (p.flags & CUQWEN_FLAG_ACCURATE_ROPE) ? 0 : 1; ra.theta = p.rope_theta;
            PK(launch_pf_rope_kv(ra, T, e->stream));
            if (l == p.n_layers - 1) break;              // the last layer's keys and values are stored: nothing after them feeds the cache
            PfAttnArgs aa; memset(&aa, 0, sizeof aa);
            aa.q = e->pf_q; aa.kc = ra.kcache; aa.vc = ra.vcache; aa.out = e->pf_att; aa.T = T; aa.pos0 = pos; aa.n_heads = e->n_heads_l;
            aa.grp = e->plan.grp; aa.max_seq = p.max_seq_len; aa.ldq = qd; aa.scale_log2 = (1.0f / sqrtf((float)p.head_dim)) * 1.4426950408889634f;
            if (!(p.flags & CUQWEN_FLAG_PREFILL_ATTN_MMA)) PK(launch_prefill_attn_tc(p.head_dim, aa, e->n_kv_l, t_err, e->stream));
            else PK(launch_prefill_attn(p.head_dim, aa, e->stream));
            if (int r = prefill_gemm(e, PF_RESID, e->pf_att, om, 1, e->pf_x, T, p.dim)) return r;
            PK(launch_pf_rmsnorm(e->pf_x, L.post_norm, e->pf_xn, T, p.dim, eps, e->stream));
            if (int r = prefill_gemm(e, PF_SWIGLU, e->pf_xn, gu, 2, e->pf_g, T, e->inter_l)) return r;
            if (int r = prefill_gemm(e, PF_RESID, e->pf_g, dm, 1, e->pf_x, T, p.dim)) return r;
        }
    }
    CK(cudaEventRecord(e->ev1, e->stream));
    CK(cudaMemcpyAsync(e->h_out, &e->ctl->pad[0], 4, cudaMemcpyDeviceToHost, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    if (e->h_out[0]) return fail(CUQWEN_ERR_TIMEOUT, "a bounded device-side wait expired (code %d)", e->h_out[0]);
    CK(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
    return CUQWEN_OK;
}

// The host loop of the reference's chat program (src/main.cu:95-112) as one call: n times cuqwen_step, each token
// going out to the host and the next one coming back in from it.
extern "C" int cuqwen_step_loop(cuqwen_engine* e, int first_token, int start_pos, int n, int* out_tokens) {
    if (!e || !out_tokens) return fail(CUQWEN_ERR_ARG, "null argument");
    int tok = first_token;
    for (int i = 0; i < n; ++i) {
        if (int r = cuqwen_step(e, tok, start_pos + i, nullptr, 0, &tok)) return r;
        out_tokens[i] = tok;
    }
    return CUQWEN_OK;
}

extern "C" int cuqwen_decode_n(cuqwen_engine* e, int first_token, int start_pos, int n, int* out_tokens) {
    if (!e) return fail(CUQWEN_ERR_ARG, "null engine");
    if (!e->loaded) return fail(CUQWEN_ERR_STATE, "cuqwen_decode_n before cuqwen_load");
    if (e->tp > 1 && !e->comm) return fail(CUQWEN_ERR_STATE, "cuqwen_decode_n before cuqwen_tp_init");
    if (n < 1 || n > e->ring_cap || first_token < 0 || first_token >= e->p.vocab_size || start_pos < 0 || start_pos + n > e->p.max_seq_len)
        return fail(CUQWEN_ERR_ARG, "decode_n arguments out of range");
    CK(cudaSetDevice(e->p.device));
    if (int r = ensure_graph(e)) return r;
    StepCtl c{}; c.token = first_token; c.pos = start_pos; c.auto_advance = 1; c.pad[1] = e->steps_done; c.io_seq = e->io_seq; c.hio = e->hio_dev;
    e->ctl_dirty = true;
    *e->h_ctl = c;
    CK(cudaMemcpyAsync(e->ctl, e->h_ctl, sizeof(StepCtl), cudaMemcpyHostToDevice, e->stream));
    CK(cudaEventRecord(e->ev0, e->stream));
    for (int i = 0; i < n; ++i) if (int r = run_step(e)) return r;
    e->steps_done += n;
    CK(cudaEventRecord(e->ev1, e->stream));
    CK(cudaMemcpyAsync(e->h_out, e->out_ring, (size_t)n * 4, cudaMemcpyDeviceToHost, e->stream));
    CK(cudaMemcpyAsync(e->h_out + n, &e->ctl->pad[0], 4, cudaMemcpyDeviceToHost, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    if (e->h_out[n]) return fail(CUQWEN_ERR_TIMEOUT, "a bounded device-side wait expired (code %d)", e->h_out[n]);
    CK(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
    if (out_tokens) memcpy(out_tokens, e->h_out, (size_t)n * 4);
    return CUQWEN_OK;
}

extern "C" float cuqwen_last_decode_ms(const cuqwen_engine* e) { return e ? e->last_ms : 0.f; }

extern "C" int cuqwen_step_profile(cuqwen_engine* e, int token, int pos, float* us, int cap, int* n_out) {
    if (!e || !us || cap < 1) return fail(CUQWEN_ERR_ARG, "null argument");
    if (!e->loaded) return fail(CUQWEN_ERR_STATE, "cuqwen_step_profile before cuqwen_load");
    if (e->tp > 1 && !e->comm) return fail(CUQWEN_ERR_STATE, "cuqwen_step_profile before cuqwen_tp_init");
    if (token < 0 || token >= e->p.vocab_size || pos < 0 || pos >= e->p.max_seq_len) return fail(CUQWEN_ERR_ARG, "token / pos out of range");
    CK(cudaSetDevice(e->p.device));
    StepCtl c{}; c.token = token; c.pos = pos; c.pad[1] = e->steps_done; c.io_seq = e->io_seq; c.hio = e->hio_dev;
    e->ctl_dirty = true;
    *e->h_ctl = c;
    CK(cudaMemcpyAsync(e->ctl, e->h_ctl, sizeof(StepCtl), cudaMemcpyHostToDevice, e->stream));
    std::vector<cudaEvent_t> evs;
    e->prof = &evs;
    int r = record_step(e, e->stream, false);      // launch by launch, no graph, plain stream order
    e->prof = nullptr;
    e->steps_done += 1;
    cudaError_t ce = cudaStreamSynchronize(e->stream);
    int n = 0;
    if (!r && ce == cudaSuccess)
        for (size_t i = 1; i < evs.size() && n < cap; ++i, ++n) { float ms = 0.f; cudaEventElapsedTime(&ms, evs[i - 1], evs[i]); us[n] = ms * 1e3f; }
    for (cudaEvent_t ev : evs) cudaEventDestroy(ev);
    if (r) return r;
    CK(ce);
    if (n_out) *n_out = n;
    return CUQWEN_OK;
}

extern "C" int cuqwen_kv_fill_normal(cuqwen_engine* e, int ctx_len, uint64_t seed) {
    if (!e || ctx_len < 0 || ctx_len > e->p.max_seq_len) return fail(CUQWEN_ERR_ARG, "ctx_len out of range");
    CK(cudaSetDevice(e->p.device));
    const cuqwen_params& p = e->p;
    LaunchCfg cfg{e->stream, e->sms, false};
    const size_t head_stride = (size_t)p.max_seq_len * p.head_dim;
    for (int l = 0; l < p.n_layers; ++l)
        for (int h = 0; h < e->n_kv_l; ++h) {
            const size_t local = ((size_t)l * e->n_kv_l + h) * head_stride;
            const uint64_t global = ((uint64_t)l * p.n_kv_heads + (e->plan.kvh0 + h)) * head_stride;
            if (e->kv8) {      // the same values, quantised row by row
                const size_t srow = ((size_t)l * e->n_kv_l + h) * p.max_seq_len;
                CK(launch_fill_normal_q8(reinterpret_cast<signed char*>(e->kc) + local, e->kscale + srow, (size_t)ctx_len, p.head_dim, seed * 2 + 0, global, cfg));
                CK(launch_fill_normal_q8(reinterpret_cast<signed char*>(e->vc) + local, e->vscale + srow, (size_t)ctx_len, p.head_dim, seed * 2 + 1, global, cfg));
                continue;
            }
            CK(launch_fill_normal(e->kc + local, (size_t)ctx_len * p.head_dim, seed * 2 + 0, global, cfg));
            CK(launch_fill_normal(e->vc + local, (size_t)ctx_len * p.head_dim, seed * 2 + 1, global, cfg));
        }
    CK(cudaStreamSynchronize(e->stream));
    return CUQWEN_OK;
}

extern "C" int cuqwen_nccl_unique_id(void* out, size_t cap) {
    if (!out || cap < sizeof(ncclUniqueId)) return fail(CUQWEN_ERR_ARG, "buffer too small for an ncclUniqueId (%zu bytes)", sizeof(ncclUniqueId));
    if (int r = nccl_load()) return r;
    ncclUniqueId id; NK(g_nccl.GetUniqueId(&id));
    memcpy(out, &id, sizeof id);
    return CUQWEN_OK;
}

extern "C" int cuqwen_tp_init(cuqwen_engine* e, const void* id_bytes, size_t n) {
    if (!e || !id_bytes || n < sizeof(ncclUniqueId)) return fail(CUQWEN_ERR_ARG, "bad ncclUniqueId");
    if (e->tp <= 1) return CUQWEN_OK;
    if (int r = nccl_load()) return r;
    CK(cudaSetDevice(e->p.device));
    ncclUniqueId id; memcpy(&id, id_bytes, sizeof id);
    NK(g_nccl.CommInitRank(&e->comm, e->tp, id, e->rank));
    if (e->p.flags & CUQWEN_FLAG_TP_NCCL) return CUQWEN_OK;          // keep the collective-call path (baseline)
    // Receive block of this rank: [2 slots][tp][dim] words of {fp32 partial, sequence number}.  Every rank
    // maps every other rank's block (CUDA IPC; the 64-byte handles travel through one NCCL all-gather), so that the
    // row-parallel GEMVs can store their partial outputs straight into their consumers' memory.
    if (e->tp > 8) return CUQWEN_OK;
    const cuqwen_params& p = e->p;
    e->tp_rx_bytes = (size_t)2 * e->tp * p.dim * 8 + (size_t)2 * e->tp * 8;      // partial-sum slots [2][tp][dim], then the samplers' key words [2][tp]
    CK(cudaMalloc((void**)&e->tp_rx, e->tp_rx_bytes));
    CK(cudaMemset(e->tp_rx, 0, e->tp_rx_bytes));
    CK(cudaMalloc((void**)&e->x2, (size_t)p.dim * 2)); CK(cudaMemset(e->x2, 0, (size_t)p.dim * 2));
    cudaIpcMemHandle_t mine, all[8];
    CK(cudaIpcGetMemHandle(&mine, e->tp_rx));
    unsigned char* d_h = nullptr;
    CK(cudaMalloc((void**)&d_h, sizeof(all)));
    CK(cudaMemcpy(d_h + (size_t)e->rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice));
    ncclResult_t nr = g_nccl.AllGather(d_h + (size_t)e->rank * sizeof(mine), d_h, sizeof(mine), ncclChar, e->comm, e->stream);
    cudaError_t ce = cudaStreamSynchronize(e->stream);
    if (nr == ncclSuccess && ce == cudaSuccess) ce = cudaMemcpy(all, d_h, sizeof(mine) * e->tp, cudaMemcpyDeviceToHost);
    cudaFree(d_h);
    if (nr != ncclSuccess) return fail(CUQWEN_ERR_NCCL, "all-gather of IPC handles: %s", g_nccl.GetErrorString(nr));
    CK(ce);
    bool ok = true;
    for (int r = 0; r < e->tp && ok; ++r) {
        if (r == e->rank) { e->peer_rx[r] = e->tp_rx; continue; }
        void* ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); ok = false; break; }
        e->peer_rx[r] = (unsigned char*)ptr;
    }
    // all ranks must agree on the path: a rank that could not map a peer makes everybody fall back to the collective calls
    int* d_ok = nullptr;
    CK(cudaMalloc((void**)&d_ok, 8));
    const int mine_ok = ok ? 1 : 0;
    CK(cudaMemcpy(d_ok, &mine_ok, 4, cudaMemcpyHostToDevice));
    nr = g_nccl.AllReduce(d_ok, d_ok + 1, 1, ncclInt32, ncclMin, e->comm, e->stream);
    ce = cudaStreamSynchronize(e->stream);
    int all_ok = 0;
    if (nr == ncclSuccess && ce == cudaSuccess) ce = cudaMemcpy(&all_ok, d_ok + 1, 4, cudaMemcpyDeviceToHost);
    cudaFree(d_ok);
    if (nr != ncclSuccess) return fail(CUQWEN_ERR_NCCL, "all-reduce of the peer-mapping status: %s", g_nccl.GetErrorString(nr));
    CK(ce);
    e->tp_peer = all_ok == 1;
    // the slots are summed once by a small kernel; CUQWEN_FLAG_TP_SUM_IN_GEMV: every CTA of the next GEMV sums them while staging x (measured slower, kept for comparison)
    e->tp_sum_separate = !(e->p.flags & CUQWEN_FLAG_TP_SUM_IN_GEMV);
    return CUQWEN_OK;
}

extern "C" int cuqwen_tp_plan(int n_heads, int n_kv, int hd, int inter, int vocab, int rank, int size, int* out9) {
    if (!out9) return fail(CUQWEN_ERR_ARG, "null argument");
    TpPlan p;
    if (int r = tp_plan(n_heads, n_kv, hd, inter, vocab, rank, size, &p)) return fail(CUQWEN_ERR_ARG, "model cannot be split over tp_size %d (rule %d)", size, r);
    int v[9] = {p.qh0, p.qh1, p.kvh0, p.kvh1, p.grp, p.i0, p.i1, p.v0, p.v1};
    memcpy(out9, v, sizeof v);
    return CUQWEN_OK;
}

extern "C" int cuqwen_lm_head_kind(const cuqwen_engine* e) { return e ? e->lm_kind : -1; }
extern "C" int cuqwen_get_params(const cuqwen_engine* e, cuqwen_params* out) { if (!e || !out) return fail(CUQWEN_ERR_ARG, "null argument"); *out = e->p; out->attn_splits = e->nsplit; return CUQWEN_OK; }
extern "C" int cuqwen_step_launches(const cuqwen_engine* e) { return e ? e->launches : 0; }
extern "C" uint64_t cuqwen_step_bytes(const cuqwen_engine* e, int ctx) {
    if (!e) return 0;
    const uint64_t row = e->kv8 ? (uint64_t)e->p.head_dim + 4 : (uint64_t)e->p.head_dim * 2;       // one cached K or V row of one head (8-bit: + its scale)
    return e->weight_bytes + (uint64_t)2 * e->p.n_layers * e->n_kv_l * row * (uint64_t)ctx;
}

extern "C" int cuqwen_get_ptr(cuqwen_engine* e, int which, int layer, void** ptr, size_t* bytes) {
    if (!e || !ptr) return fail(CUQWEN_ERR_ARG, "null argument");
    const cuqwen_params& p = e->p;
    void* r = nullptr; size_t b = 0;
    auto matb = [&](const Mat& m, int quant) { return elem_bytes2(quant, m.rows, m.cols); };
    auto scb = [&](const Mat& m) { return (size_t)m.rows * (m.cols / kGroup) * 2; };
    if (which >= CUQWEN_PTR_IN_NORM) {
        if (!e->loaded || layer < 0 || layer >= p.n_layers) return fail(CUQWEN_ERR_ARG, "layer %d out of range or weights not loaded", layer);
        const Layer& L = e->layers[layer];
        switch (which) {
            case CUQWEN_PTR_IN_NORM: r = L.in_norm; b = p.dim * 2; break;
            case CUQWEN_PTR_WQ: r = L.q.w; b = matb(L.q, p.quant); break;
            case CUQWEN_PTR_SQ: r = L.q.s; b = scb(L.q); break;
            case CUQWEN_PTR_BQ: r = L.bq; b = e->q_dim_l * 2; break;
            case CUQWEN_PTR_WK: r = L.k.w; b = matb(L.k, p.quant); break;
            case CUQWEN_PTR_SK: r = L.k.s; b = scb(L.k); break;
            case CUQWEN_PTR_BK: r = L.bk; b = e->kv_dim_l * 2; break;
            case CUQWEN_PTR_WV: r = L.v.w; b = matb(L.v, p.quant); break;
            case CUQWEN_PTR_SV: r = L.v.s; b = scb(L.v); break;
            case CUQWEN_PTR_BV: r = L.bv; b = e->kv_dim_l * 2; break;
            case CUQWEN_PTR_WO: r = L.o.w; b = matb(L.o, p.quant); break;
            case CUQWEN_PTR_SO: r = L.o.s; b = scb(L.o); break;
            case CUQWEN_PTR_POST_NORM: r = L.post_norm; b = p.dim * 2; break;
            case CUQWEN_PTR_WGATE: r = L.gate.w; b = matb(L.gate, p.quant); break;
            case CUQWEN_PTR_SGATE: r = L.gate.s; b = scb(L.gate); break;
            case CUQWEN_PTR_WUP: r = L.up.w; b = matb(L.up, p.quant); break;
            case CUQWEN_PTR_SUP: r = L.up.s; b = scb(L.up); break;
            case CUQWEN_PTR_WDOWN: r = L.down.w; b = matb(L.down, p.quant); break;
            case CUQWEN_PTR_SDOWN: r = L.down.s; b = scb(L.down); break;
            default: return fail(CUQWEN_ERR_ARG, "unknown pointer id %d", which);
        }
    } else if (which >= CUQWEN_PTR_EMBED) {
        if (!e->loaded) return fail(CUQWEN_ERR_STATE, "weights not loaded");
        switch (which) {
            case CUQWEN_PTR_EMBED: r = e->embed; b = (size_t)p.vocab_size * p.dim * 2; break;
            case CUQWEN_PTR_NORM: r = e->norm; b = p.dim * 2; break;
            case CUQWEN_PTR_LM_HEAD: r = e->lm.w; b = matb(e->lm, e->lm_quant); break;
            case CUQWEN_PTR_LM_HEAD_SCALE: r = e->lm.s; b = e->lm.s ? scb(e->lm) : 0; break;
            default: return fail(CUQWEN_ERR_ARG, "unknown pointer id %d", which);
        }
    } else {
        const size_t kvb = (size_t)p.n_layers * e->n_kv_l * p.max_seq_len * p.head_dim * (e->kv8 ? 1 : 2);
        switch (which) {
            case CUQWEN_PTR_X: r = e->x; b = p.dim * 2; break;
            case CUQWEN_PTR_XN: r = e->xn; b = p.dim * 2; break;
            case CUQWEN_PTR_Q: r = e->q; b = e->q_dim_l * 2; break;
            case CUQWEN_PTR_K: r = e->k; b = e->kv_dim_l * 2; break;
            case CUQWEN_PTR_V: r = e->v; b = e->kv_dim_l * 2; break;
            case CUQWEN_PTR_ATT: r = e->att; b = e->q_dim_l * 2; break;
            case CUQWEN_PTR_GATE: r = e->gate; b = e->inter_l * 2; break;
            case CUQWEN_PTR_LOGITS: r = e->logits; b = e->vocab_l * 2; break;
            case CUQWEN_PTR_KEY_CACHE: r = e->kc; b = kvb; break;
            case CUQWEN_PTR_VALUE_CACHE: r = e->vc; b = kvb; break;
            case CUQWEN_PTR_HISTORY: r = e->d_hist; b = (size_t)p.max_seq_len * 4; break;
            case CUQWEN_PTR_STEP_TRACE: r = e->step_trace; b = e->step_trace_bytes; break;
            case CUQWEN_PTR_KEY_SCALE: r = e->kscale; b = e->kv8 ? (size_t)p.n_layers * e->n_kv_l * p.max_seq_len * 4 : 0; break;
            case CUQWEN_PTR_VALUE_SCALE: r = e->vscale; b = e->kv8 ? (size_t)p.n_layers * e->n_kv_l * p.max_seq_len * 4 : 0; break;
            case CUQWEN_PTR_TOKEN: r = &e->ctl->token; b = 4; break;
            case CUQWEN_PTR_POS: r = &e->ctl->pos; b = 4; break;
            case CUQWEN_PTR_HISTORY_LEN: r = &e->ctl->hist_len; b = 4; break;
            case CUQWEN_PTR_SAMPLED: r = &e->ctl->sampled; b = 4; break;
            case CUQWEN_PTR_PARTIAL_O: r = e->part_o; b = attn_scratch_floats_o(e->n_kv_l, e->nsplit, p.head_dim) * 4; break;
            case CUQWEN_PTR_PARTIAL_ML: r = e->part_ml; b = attn_scratch_floats_ml(e->n_kv_l, e->nsplit) * 4; break;
            case CUQWEN_PTR_UP: r = e->spare_up; b = (size_t)e->inter_l * 2; break;
            case CUQWEN_PTR_MLP_OUT: r = e->spare_out; b = (size_t)p.dim * 2; break;
            case CUQWEN_PTR_STREAM: r = (void*)e->stream; b = 0; break;
            default: return fail(CUQWEN_ERR_ARG, "unknown pointer id %d", which);
        }
    }
    *ptr = r; if (bytes) *bytes = b;
    return CUQWEN_OK;
}

// ---------------------------------------------------------------------------
// raw device helpers
// ---------------------------------------------------------------------------
extern "C" int cuqwen_dev_alloc(int device, size_t bytes, void** p) { DEV(device); (void)cfg; CK(cudaMalloc(p, bytes ? bytes : 1)); return CUQWEN_OK; }
extern "C" int cuqwen_dev_sm_count(int device, int* n) { DEV(device); (void)cfg; if (!n) return fail(CUQWEN_ERR_ARG, "null argument"); *n = dc->sms; return CUQWEN_OK; }
extern "C" int cuqwen_dev_free(int device, void* p) { DEV(device); (void)cfg; CK(cudaStreamSynchronize(dc->stream)); CK(cudaFree(p)); return CUQWEN_OK; }
extern "C" int cuqwen_dev_upload(int device, void* d, const void* h, size_t n) { DEV(device); (void)cfg; CK(cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, dc->stream)); CK(cudaStreamSynchronize(dc->stream)); return CUQWEN_OK; }
extern "C" int cuqwen_dev_download(int device, void* h, const void* d, size_t n) { DEV(device); (void)cfg; CK(cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, dc->stream)); CK(cudaStreamSynchronize(dc->stream)); return CUQWEN_OK; }
extern "C" int cuqwen_dev_memset(int device, void* p, int v, size_t n) { DEV(device); (void)cfg; CK(cudaMemsetAsync(p, v, n, dc->stream)); return CUQWEN_OK; }
extern "C" int cuqwen_dev_sync(int device) {
    DEV(device); (void)cfg;
    CK(cudaMemcpyAsync(dc->h_err, dc->err, 4, cudaMemcpyDeviceToHost, dc->stream));
    CK(cudaStreamSynchronize(dc->stream)); CK(cudaGetLastError());
    if (*dc->h_err) { unsigned c = *dc->h_err; CK(cudaMemset(dc->err, 0, 4)); return fail(CUQWEN_ERR_TIMEOUT, "a bounded device-side wait expired (code %u)", c); }
    return CUQWEN_OK;
}
// Orders the library's per-device stream against a caller's stream (0 = the legacy default stream):
// leave == 0: work queued from now on through cuqwen_k_* waits for what the caller's stream holds so far;
// leave != 0: what the caller queues on its stream from now on waits for the cuqwen_k_* work queued so far.
extern "C" int cuqwen_dev_join(int device, void* caller_stream, int leave) {
    DEV(device); (void)cfg;
    cudaStream_t from = leave ? dc->stream : (cudaStream_t)caller_stream;
    cudaStream_t to = leave ? (cudaStream_t)caller_stream : dc->stream;
    CK(cudaEventRecord(dc->ev_join, from));
    CK(cudaStreamWaitEvent(to, dc->ev_join, 0));
    return CUQWEN_OK;
}
// Timing without the caller in the measurement: between cuqwen_capture_begin and cuqwen_capture_replay every
// cuqwen_k_* call on this device is recorded into a CUDA graph instead of running (same launch attributes as in the
// engine's step graph); cuqwen_capture_replay instantiates it, replays it once untimed and then `replays` times
// between two events, and returns the milliseconds per replay.  Call every kernel once before capturing (the first
// launch of a kernel loads its module, which a capture does not allow).
extern "C" int cuqwen_capture_begin(int device) {
    DEV(device); (void)cfg;
    CK(cudaStreamBeginCapture(dc->stream, cudaStreamCaptureModeThreadLocal));
    return CUQWEN_OK;
}
extern "C" int cuqwen_capture_replay(int device, int replays, float* ms_per_replay) {
    DEV(device); (void)cfg;
    cudaGraph_t g = nullptr;
    CK(cudaStreamEndCapture(dc->stream, &g));
    if (!g) return fail(CUQWEN_ERR_STATE, "nothing was captured");
    if (replays < 1 || !ms_per_replay) { cudaGraphDestroy(g); return fail(CUQWEN_ERR_ARG, "replays must be positive"); }
    cudaGraphExec_t ge = nullptr;
    cudaError_t e_ = cudaGraphInstantiate(&ge, g, 0);
    if (e_ == cudaSuccess) e_ = cudaGraphLaunch(ge, dc->stream);
    if (e_ == cudaSuccess) e_ = cudaEventRecord(dc->ev0, dc->stream);
    for (int i = 0; i < replays && e_ == cudaSuccess; ++i) e_ = cudaGraphLaunch(ge, dc->stream);
    if (e_ == cudaSuccess) e_ = cudaEventRecord(dc->ev1, dc->stream);
    if (e_ == cudaSuccess) e_ = cudaEventSynchronize(dc->ev1);
    float ms = 0.f;
    if (e_ == cudaSuccess) e_ = cudaEventElapsedTime(&ms, dc->ev0, dc->ev1);
    if (ge) cudaGraphExecDestroy(ge);
    cudaGraphDestroy(g);
    if (e_ != cudaSuccess) return fail(CUQWEN_ERR_CUDA, "graph replay: %s", cudaGetErrorString(e_));
    *ms_per_replay = ms / (float)replays;
    return CUQWEN_OK;
}
extern "C" int cuqwen_bench_begin(int device) { DEV(device); (void)cfg; CK(cudaEventRecord(dc->ev0, dc->stream)); return CUQWEN_OK; }
extern "C" int cuqwen_bench_end(int device, float* ms) { DEV(device); (void)cfg; CK(cudaEventRecord(dc->ev1, dc->stream)); CK(cudaEventSynchronize(dc->ev1)); CK(cudaEventElapsedTime(ms, dc->ev0, dc->ev1)); return CUQWEN_OK; }

// ---------------------------------------------------------------------------
// per-kernel entry points
// ---------------------------------------------------------------------------
#define KK(call) do { int r_ = (call); if (r_) return fail(r_ == (int)cudaErrorInvalidValue ? CUQWEN_ERR_ARG : CUQWEN_ERR_CUDA, "%s: %s", #call, cudaGetErrorString((cudaError_t)r_)); } while (0)
static bool bad_q(int q) { return q < 0 || q > 2; }
// A null pointer handed to a kernel is a device fault, not an error code: every entry point checks the pointers it
// will dereference first.  Scales are required exactly when the weights are quantised.
#define NOT_NULL(...) do { const void* ps_[] = {__VA_ARGS__}; for (const void* p_ : ps_) if (!p_) return fail(CUQWEN_ERR_ARG, "%s: null pointer argument", __func__); } while (0)
#define SCALES_OK(quant, ...) do { if (quant) NOT_NULL(__VA_ARGS__); } while (0)

extern "C" int cuqwen_k_embedding(int device, const void* table, const int* d_token, void* out, int dim) {
    DEV(device); if (dim <= 0 || dim % 8) return fail(CUQWEN_ERR_ARG, "dim must be a positive multiple of 8");
    NOT_NULL(table, d_token, out);
    KK(launch_embed((const __half*)table, d_token, (__half*)out, dim, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_rmsnorm(int device, const void* x, const void* w, void* out, int dim, float eps) {
    DEV(device); if (dim <= 0) return fail(CUQWEN_ERR_ARG, "dim must be positive");
    NOT_NULL(x, w, out);
    KK(launch_rmsnorm((const __half*)x, (const __half*)w, (__half*)out, dim, eps, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_qkv(int device, int quant, const void* x, const void* norm_w, float eps, const void* wq, const void* wk, const void* wv,
                            const void* sq, const void* sk, const void* sv, const void* bq, const void* bk, const void* bv, void* q_out, void* k_out,
                            void* v_out, void* kcache, void* vcache, int dim, int n_heads, int n_kv, int hd, int max_seq, const int* d_pos, float theta, int fast) {
    DEV(device);
    if (bad_q(quant) || dim <= 0 || dim % kGroup || (hd != 64 && hd != 128) || n_heads < 1 || n_kv < 1) return fail(CUQWEN_ERR_ARG, "unsupported qkv shape");
    NOT_NULL(x, wq, wk, wv, bq, bk, bv, d_pos);          // the biases are required (every Qwen2.5 q/k/v projection has one); outputs may be null one by one
    SCALES_OK(quant, sq, sk, sv);
    if ((kcache || vcache) && max_seq < 1) return fail(CUQWEN_ERR_ARG, "max_seq_len must be positive when a cache is given");
    GemvArgs a = gv((const __half*)x, dim);
    a.norm_w = (const __half*)norm_w; a.eps = eps;
    a.w[0] = (const uint8_t*)wq; a.w[1] = (const uint8_t*)wk; a.w[2] = (const uint8_t*)wv;
    a.s[0] = (const __half*)sq; a.s[1] = (const __half*)sk; a.s[2] = (const __half*)sv;
    a.bias[0] = (const __half*)bq; a.bias[1] = (const __half*)bk; a.bias[2] = (const __half*)bv;
    a.q_out = (__half*)q_out; a.k_out = (__half*)k_out; a.v_out = (__half*)v_out; a.kcache = (__half*)kcache; a.vcache = (__half*)vcache;
    a.d_pos = d_pos; a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.max_seq = max_seq; a.theta = theta; a.rope_fast = fast;
    KK(launch_gemv(quant, EPI_QKV, a, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_rope(int device, void* q, void* k, int n_heads, int n_kv, int hd, const int* d_pos, float theta, int fast) {
    DEV(device); NOT_NULL(q, k, d_pos); KK(launch_rope((__half*)q, (__half*)k, n_heads, n_kv, hd, d_pos, theta, fast, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_kv_store(int device, const void* k, const void* v, void* kc, void* vc, const int* d_pos, int n_kv, int max_seq, int hd) {
    DEV(device); NOT_NULL(k, v, kc, vc, d_pos); KK(launch_kv_store((const __half*)k, (const __half*)v, (__half*)kc, (__half*)vc, d_pos, n_kv, max_seq, hd, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_attn_scratch_bytes(int n_kv, int hd, int nsplit, size_t* bo, size_t* bml, size_t* bc) {
    if (n_kv < 1 || nsplit < 1 || nsplit > kMaxSplit || (hd != 64 && hd != 128)) return fail(CUQWEN_ERR_ARG, "unsupported attention shape");
    if (bo) *bo = attn_scratch_floats_o(n_kv, nsplit, hd) * 4;
    if (bml) *bml = attn_scratch_floats_ml(n_kv, nsplit) * 4;
    if (bc) *bc = attn_scratch_counters(n_kv, nsplit) * 4;
    return CUQWEN_OK;
}
extern "C" int cuqwen_k_attention(int device, const void* q, const void* kc, const void* vc, void* out, const int* d_pos, int n_heads, int n_kv, int hd,
                                  int max_seq, int nsplit, void* so, void* sml, void* counters) {
    DEV(device);
    if (n_kv < 1 || n_heads % n_kv || n_heads / n_kv > kMaxGroup || (hd != 64 && hd != 128) || nsplit < 1 || nsplit > kMaxSplit)
        return fail(CUQWEN_ERR_ARG, "unsupported attention shape (heads %d/%d, head_dim %d, splits %d)", n_heads, n_kv, hd, nsplit);
    NOT_NULL(q, kc, vc, out, d_pos, so, sml);
    AttnArgs a{};
    a.q = (const __half*)q; a.kc = (const __half*)kc; a.vc = (const __half*)vc; a.out = (__half*)out; a.d_pos = d_pos;
    a.n_kv = n_kv; a.grp = n_heads / n_kv; a.max_seq = max_seq; a.nsplit = nsplit;
    a.scale_log2 = (1.0f / sqrtf((float)hd)) * 1.4426950408889634f;
    a.part_o = (float*)so; a.part_ml = (float*)sml; a.counters = (unsigned*)counters; a.err = t_err;
    KK(launch_attn(hd, a, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_attention_kv8(int device, const void* q, void* kc8, void* vc8, float* kscale, float* vscale, const void* k_cur, const void* v_cur,
                                      void* out, const int* d_pos, int n_heads, int n_kv, int hd, int max_seq, int nsplit, void* so, void* sml) {
    DEV(device);
    if (n_kv < 1 || n_heads % n_kv || n_heads / n_kv > kMaxGroup || (hd != 64 && hd != 128) || nsplit < 1 || nsplit > kMaxSplit || max_seq < 1 || max_seq % 4)
        return fail(CUQWEN_ERR_ARG, "unsupported attention shape (heads %d/%d, head_dim %d, splits %d, max_seq_len %d)", n_heads, n_kv, hd, nsplit, max_seq);
    NOT_NULL(q, kc8, vc8, kscale, vscale, k_cur, v_cur, out, d_pos, so, sml);
    AttnArgs a{};
    a.q = (const __half*)q; a.kc = (const __half*)kc8; a.vc = (const __half*)vc8; a.out = (__half*)out; a.d_pos = d_pos;
    a.n_kv = n_kv; a.grp = n_heads / n_kv; a.max_seq = max_seq; a.nsplit = nsplit;
    a.scale_log2 = (1.0f / sqrtf((float)hd)) * 1.4426950408889634f;
    a.part_o = (float*)so; a.part_ml = (float*)sml; a.err = t_err;
    a.kscale = kscale; a.vscale = vscale; a.k_cur = (const __half*)k_cur; a.v_cur = (const __half*)v_cur;
    KK(launch_attn(hd, a, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_prefill_gemm(int device, int quant, int mode, const void* x, const void* w0, const void* s0, const void* w1, const void* s1,
                                     const void* bias, void* out, int n_tokens, int rows, int cols, int out_stride) {
    DEV(device); (void)cfg;
    if (bad_q(quant)) return fail(CUQWEN_ERR_ARG, "quant out of range");
    if (mode < PF_OUT_F16 || mode > PF_SWIGLU) return fail(CUQWEN_ERR_ARG, "mode out of range");
    NOT_NULL(x, w0, out); SCALES_OK(quant, s0);
    if (mode == PF_SWIGLU) { NOT_NULL(w1); SCALES_OK(quant, s1); }
    else if (w1) return fail(CUQWEN_ERR_ARG, "a second matrix only in the SwiGLU mode");
    PfGemmArgs a; memset(&a, 0, sizeof a);
    a.s[0] = (const __half*)s0; a.s[1] = (const __half*)s1; a.bias = (const __half*)bias;
    a.out_h = (__half*)out; a.out_f = (float*)out; a.T = n_tokens; a.K = cols; a.ldo = out_stride; a.mode = mode; a.err = t_err;
    const void* w[2] = {w0, w1}; const int rws[2] = {rows, rows};
    KK(launch_prefill_gemm(quant, a, x, w, rws, mode == PF_SWIGLU ? 2 : 1, dc->stream)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_prefill_attention(int device, int impl, const void* q, const void* kcache, const void* vcache, void* out, int n_tokens, int pos0,
                                          int n_heads, int n_kv_heads, int head_dim, int max_seq_len, int q_stride) {
    DEV(device); (void)cfg;
    NOT_NULL(q, kcache, vcache, out);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return fail(CUQWEN_ERR_ARG, "n_heads must be a multiple of n_kv_heads");
    if ((head_dim != 64 && head_dim != 128) || impl < 0 || impl > 1) return fail(CUQWEN_ERR_ARG, "impl 0 / 1, head_dim 64 / 128");
    PfAttnArgs a; memset(&a, 0, sizeof a);
    a.q = (const __half*)q; a.kc = (const __half*)kcache; a.vc = (const __half*)vcache; a.out = (__half*)out; a.T = n_tokens; a.pos0 = pos0;
    a.n_heads = n_heads; a.grp = n_heads / n_kv_heads; a.max_seq = max_seq_len; a.ldq = q_stride;
    a.scale_log2 = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
    if (impl == 0) KK(launch_prefill_attn_tc(head_dim, a, n_kv_heads, t_err, dc->stream));
    else KK(launch_prefill_attn(head_dim, a, dc->stream));
    return CUQWEN_OK;
}
extern "C" int cuqwen_k_gemv_add(int device, int quant, const void* w, const void* s, const void* in, void* x, int rows, int cols) {
    DEV(device); if (bad_q(quant)) return fail(CUQWEN_ERR_ARG, "quant out of range");
    NOT_NULL(w, in, x); SCALES_OK(quant, s);
    GemvArgs a = gv((const __half*)in, cols); a.w[0] = (const uint8_t*)w; a.s[0] = (const __half*)s; a.rows = rows; a.out_h = (__half*)x;
    KK(launch_gemv(quant, EPI_RESID, a, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_gemv(int device, int quant, const void* w, const void* s, const void* x, const void* norm_w, float eps, void* y, int rows, int cols) {
    DEV(device); if (bad_q(quant)) return fail(CUQWEN_ERR_ARG, "quant out of range");
    NOT_NULL(w, x, y); SCALES_OK(quant, s);
    GemvArgs a = gv((const __half*)x, cols); a.norm_w = (const __half*)norm_w; a.eps = eps; a.w[0] = (const uint8_t*)w; a.s[0] = (const __half*)s; a.rows = rows; a.out_h = (__half*)y;
    KK(launch_gemv(quant, EPI_F16, a, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_gemv_f32(int device, int quant, const void* w, const void* s, const void* x, float* y, int rows, int cols) {
    DEV(device); if (bad_q(quant)) return fail(CUQWEN_ERR_ARG, "quant out of range");
    NOT_NULL(w, x, y); SCALES_OK(quant, s);
    GemvArgs a = gv((const __half*)x, cols); a.w[0] = (const uint8_t*)w; a.s[0] = (const __half*)s; a.rows = rows; a.out_f = y;
    KK(launch_gemv(quant, EPI_F32, a, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_mlp1(int device, int quant, const void* x, const void* norm_w, float eps, const void* wg, const void* wu, const void* sg,
                             const void* su, void* out, int dim, int inter) {
    DEV(device); if (bad_q(quant)) return fail(CUQWEN_ERR_ARG, "quant out of range");
    NOT_NULL(x, wg, wu, out); SCALES_OK(quant, sg, su);
    GemvArgs a = gv((const __half*)x, dim); a.norm_w = (const __half*)norm_w; a.eps = eps;
    a.w[0] = (const uint8_t*)wg; a.w[1] = (const uint8_t*)wu; a.s[0] = (const __half*)sg; a.s[1] = (const __half*)su; a.rows = inter; a.out_h = (__half*)out;
    KK(launch_gemv(quant, EPI_SWIGLU, a, cfg)); return CUQWEN_OK;
}
extern "C" int cuqwen_k_penalty(int device, void* logits, const int* hist, const int* d_len, int vocab, float pen, void* bitmap) {
    DEV(device);
    NOT_NULL(logits, hist, d_len, bitmap);
    KK(launch_penalty((__half*)logits, hist, d_len, vocab, 0, pen, (unsigned*)bitmap, cfg));
    KK(launch_clear_bitmap(hist, d_len, vocab, 0, (unsigned*)bitmap, cfg));
    return CUQWEN_OK;
}
extern "C" int cuqwen_k_argmax(int device, const void* logits, int* d_out, int vocab, void* scratch16) {
    DEV(device);
    NOT_NULL(logits, d_out, scratch16);
    unsigned long long* best = (unsigned long long*)scratch16;
    KK(launch_argmax((const __half*)logits, vocab, 0, nullptr, nullptr, 0, nullptr, nullptr, best, (unsigned*)(best + 1), nullptr, d_out, cfg));
    return CUQWEN_OK;
}
extern "C" int cuqwen_k_dequant(int device, int quant, const void* w, const void* s, void* out, long rows, long cols) {
    DEV(device); if (quant != 1 && quant != 2) return fail(CUQWEN_ERR_ARG, "dequant needs quant 1 or 2");
    NOT_NULL(w, s, out);
    KK(launch_dequant(quant, w, (const __half*)s, (__half*)out, rows, cols, cfg)); return CUQWEN_OK;
}

// Tensor-parallel helper, stand-alone: x_next = half(float(x) + sum over n_ranks receive slots [n_ranks][dim] of
// {fp32 partial, sequence} words), waiting (bounded) until every word carries step * 512 + seq_index + 1 with the step
// read from *d_step_no.  wait_cycles bounds the wait in SM cycles (0 = the default, two to four seconds); when it runs
// out the kernel returns, and the next cuqwen_dev_sync reports CUQWEN_ERR_TIMEOUT.
extern "C" int cuqwen_k_tp_sum(int device, const void* x, void* x_next, const void* slots, int n_ranks, int dim, const int* d_step_no, int seq_index,
                               long long wait_cycles) {
    DEV(device);
    if (n_ranks < 1 || n_ranks > 8 || dim <= 0 || dim % 8 || seq_index < 0 || seq_index >= (int)kSeqPerStep || wait_cycles < 0)
        return fail(CUQWEN_ERR_ARG, "unsupported tp_sum arguments");
    NOT_NULL(x, x_next, slots, d_step_no);
    KK(launch_tp_sum((const __half*)x, (__half*)x_next, slots, n_ranks, dim, d_step_no, seq_index, t_err, wait_cycles, cfg));
    return CUQWEN_OK;
}
