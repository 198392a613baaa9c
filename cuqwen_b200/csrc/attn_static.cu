// Split-KV decode attention whose scratch lives in a fixed device array instead of caller-supplied buffers.
//
// Who this is for: a host that has finished its start-up phase and from then on must not grow or shrink device
// memory — a serving loop with a fixed memory budget where cudaMalloc/cudaFree would stall every stream of the
// device while they run, a thread that holds a lock the allocator could contend on, or a region of code where the
// CUDA runtime refuses allocation calls outright.  cuqwen_k_attention needs three scratch buffers from its caller;
// such a host has nowhere to get them.  This entry needs none: the partial results, the (max, sum) pairs, the
// tickets and the status word all sit in `g_scratch` below, which the module loader places once.
//
// Limits: attn_slots(n_kv, n_splits) <= kStaticSlots (384) and attn_counters(n_kv, n_splits) <= kStaticCounters (256);
// e.g. 4 KV heads x 74 splits or 8 KV heads x 42 splits.  The array is 1,598,720 bytes per device.  Larger shapes are
// rejected with CUQWEN_ERR_ARG.
//
// Status: every wait inside the kernels is bounded; when one runs out the kernel finishes with meaningless numbers and
// leaves a non-zero code in a status word of the block.  That word is NOT part of what a call clears, so it survives
// until the host asks: cuqwen_k_attention_static_status copies it out (into the caller's own variable, no allocation),
// clears it, and answers CUQWEN_ERR_TIMEOUT when it was set.  Ask after the work has been queued and before trusting
// `out`; the query waits for `stream`.
//
// Set-up: the first call for a device (with that device current) looks the array's address up with
// cudaGetSymbolAddress and raises the kernel's dynamic shared-memory limit; make that first call before any stream
// capture begins.  Later calls only queue a 1 KB memset of the tickets and the kernel launch.
// Nothing here calls cudaMalloc, cudaFree or any routine that allocates.
//
// There is ONE scratch block per device: two calls that may overlap on the device (different streams, or different
// host threads without ordering between their streams) race on it.  Calls on one stream are ordered and safe.
//
// The kernels are the bodies of attn_split.cuh (partials, then the per-head fold) compiled under other names, so
// cuqwen_k_attention and the engine keep their own instantiations untouched and both entries compute the same bits.
#define attn_partial_kernel attn_partial_static_kernel
#define attn_fold_kernel attn_fold_static_kernel
#include "attn_split.cuh"
#undef attn_partial_kernel
#undef attn_fold_kernel

#include <mutex>

#include "../../include/cuqwen_b200.h"
#include "errors.h"

namespace {

using namespace cq;

constexpr int kStaticSlots = 384;
constexpr int kStaticCounters = 256;
constexpr int kStaticMaxHd = 128;

constexpr size_t kOffCounters = 0;                                   // u32 [kStaticCounters], zero between launches
constexpr size_t kClearBytes = kStaticCounters * 4;                  // what every call clears: the tickets, nothing else
constexpr size_t kOffErr = kClearBytes;                              // u32 status word (+ padding to 256 B); cleared only by the status query
constexpr size_t kOffMl = kOffErr + 256;                             // float [kStaticSlots][8][2]
constexpr size_t kOffO = kOffMl + (size_t)kStaticSlots * kMaxGroup * 2 * 4;   // float [kStaticSlots][8][hd]
constexpr size_t kScratchBytes = kOffO + (size_t)kStaticSlots * kMaxGroup * kStaticMaxHd * 4;

static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_base[kMaxDevices] = {};

// Address of g_scratch on `device`; the device must be current.  Done once per device.
int scratch_base(int device, unsigned char** out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_base[device]) {
        unsigned char* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_scratch);
        if (e != cudaSuccess || !p) return report_error(CUQWEN_ERR_CUDA, "cudaGetSymbolAddress(attention scratch): %s", cudaGetErrorString(e));
        e = cudaFuncSetAttribute(attn_partial_static_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_split_smem_bytes(128, kSplitStages));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_partial_static_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_split_smem_bytes(64, kSplitStages));
        if (e != cudaSuccess) return report_error(CUQWEN_ERR_CUDA, "cudaFuncSetAttribute(attention): %s", cudaGetErrorString(e));
        g_base[device] = p;
    }
    *out = g_base[device];
    return CUQWEN_OK;
}

template <int HD>
cudaError_t launch(const AttnArgs& a, cudaStream_t stream) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(a.n_kv, a.nsplit); lc.blockDim = dim3(kSplitThreads);
    lc.dynamicSmemBytes = attn_split_smem_bytes(HD, kSplitStages); lc.stream = stream;
    cudaError_t e = cudaLaunchKernelEx(&lc, attn_partial_static_kernel<HD>, a);
    if (e != cudaSuccess) return e;
    lc.gridDim = dim3(a.n_kv * a.grp); lc.blockDim = dim3(kFoldWarps * 32); lc.dynamicSmemBytes = 0;
    return cudaLaunchKernelEx(&lc, attn_fold_static_kernel<HD>, a);
}

}  // namespace

extern "C" int cuqwen_k_attention_static(int device, void* stream, const void* q, const void* kc, const void* vc, void* out, const int* d_pos,
                                         int n_heads, int n_kv, int hd, int max_seq, int nsplit) {
    if (device < 0 || device >= kMaxDevices) return report_error(CUQWEN_ERR_ARG, "device %d out of range", device);
    if (!q || !kc || !vc || !out || !d_pos) return report_error(CUQWEN_ERR_ARG, "null argument");
    if (n_kv < 1 || n_heads < n_kv || n_heads % n_kv || n_heads / n_kv > kMaxGroup || (hd != 64 && hd != 128) || nsplit < 1 || nsplit > kMaxSplit || max_seq < 1)
        return report_error(CUQWEN_ERR_ARG, "unsupported attention shape (heads %d/%d, head_dim %d, splits %d)", n_heads, n_kv, hd, nsplit);
    if (attn_slots(n_kv, nsplit) > (size_t)kStaticSlots || attn_counters(n_kv, nsplit) > (size_t)kStaticCounters)
        return report_error(CUQWEN_ERR_ARG, "shape needs %zu partial slots and %zu tickets; the fixed scratch holds %d and %d (use cuqwen_k_attention)",
                            attn_slots(n_kv, nsplit), attn_counters(n_kv, nsplit), kStaticSlots, kStaticCounters);
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return report_error(CUQWEN_ERR_CUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    unsigned char* base = nullptr;
    if (int r = scratch_base(device, &base)) return r;
    cudaStream_t st = (cudaStream_t)stream;
    e = cudaMemsetAsync(base + kOffCounters, 0, kClearBytes, st);
    if (e != cudaSuccess) return report_error(CUQWEN_ERR_CUDA, "cudaMemsetAsync(attention tickets): %s", cudaGetErrorString(e));
    AttnArgs a{};
    a.q = (const __half*)q; a.kc = (const __half*)kc; a.vc = (const __half*)vc; a.out = (__half*)out; a.d_pos = d_pos;
    a.n_kv = n_kv; a.grp = n_heads / n_kv; a.max_seq = max_seq; a.nsplit = nsplit;
    a.scale_log2 = (1.0f / sqrtf((float)hd)) * 1.4426950408889634f; a.stages = kSplitStages;
    a.part_o = reinterpret_cast<float*>(base + kOffO);
    a.part_ml = reinterpret_cast<float*>(base + kOffMl);
    a.counters = reinterpret_cast<unsigned*>(base + kOffCounters);
    a.err = reinterpret_cast<unsigned*>(base + kOffErr);
    e = hd == 128 ? launch<128>(a, st) : launch<64>(a, st);
    if (e != cudaSuccess) return report_error(CUQWEN_ERR_CUDA, "attention launch: %s", cudaGetErrorString(e));
    return CUQWEN_OK;
}

// Reads and clears the status word of the device's scratch block (see the file comment).  `code_out` receives the
// word (0 = no wait ran out since the last query).  Waits for `stream`; allocates nothing.
extern "C" int cuqwen_k_attention_static_status(int device, void* stream, unsigned* code_out) {
    if (device < 0 || device >= kMaxDevices) return report_error(CUQWEN_ERR_ARG, "device %d out of range", device);
    if (!code_out) return report_error(CUQWEN_ERR_ARG, "null argument");
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return report_error(CUQWEN_ERR_CUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    unsigned char* base = nullptr;
    if (int r = scratch_base(device, &base)) return r;
    cudaStream_t st = (cudaStream_t)stream;
    *code_out = 0u;
    e = cudaMemcpyAsync(code_out, base + kOffErr, 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return report_error(CUQWEN_ERR_CUDA, "reading the attention status word: %s", cudaGetErrorString(e));
    if (*code_out == 0u) return CUQWEN_OK;
    e = cudaMemsetAsync(base + kOffErr, 0, 4, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return report_error(CUQWEN_ERR_CUDA, "clearing the attention status word: %s", cudaGetErrorString(e));
    return report_error(CUQWEN_ERR_TIMEOUT, "a bounded device-side wait expired in cuqwen_k_attention_static (code %u)", *code_out);
}
