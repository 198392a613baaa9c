// Asynchronous-copy and mbarrier primitives (inline PTX) shared by the streaming kernels.
// No copy here uses cluster broadcast: every load lands in the issuing CTA's own shared memory.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace cq {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ long long sm_cycles() { long long t; asm volatile("mov.u64 %0, %clock64;" : "=l"(t)); return t; }
// Per-launch timeline (profiling aid, CUQWEN_FLAG_STEP_TRACE): a launch owns sixteen u64 words that its CTAs merge with
// atomic max - "earliest" stamps are stored complemented, so one memset to zero resets them all.  One thread per CTA calls.
//   0 first CTA started (~)   1 last CTA started   2 first consumer past the dependency wait (~)   3 last CTA had its
//   input vector staged   4 last CTA left its main loop   5 last CTA finished
//   6, 7 stamps inside the staging of the input vector   8 sum of the CTAs' start times (low 32 bits of each)   9 number of CTAs
constexpr int kTraceWords = 16;
__device__ __forceinline__ void trace_start(unsigned long long* t) { if (t) { atomicAdd(t + 8, global_ns() & 0xffffffffull); atomicAdd(t + 9, 1ull); } }
__device__ __forceinline__ void trace_first(unsigned long long* t, int i) { if (t) atomicMax(t + i, ~global_ns()); }
__device__ __forceinline__ void trace_last(unsigned long long* t, int i) { if (t) atomicMax(t + i, global_ns()); }
// Bounded wait: false when the phase did not complete within about 4e9 SM cycles (2 to 4 s at the clocks this part
// runs at).  The bound is kept on the SM's own cycle counter: a %globaltimer read is a long-latency operation, and
// one on every wait that does not succeed at once delays the moment the waiting warp sees the phase complete.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) if (mbar_try_wait(bar, parity)) return true;
        const long long now = sm_cycles();
        if (t0 == 0) t0 = now;
        else if (now - t0 > 4000000000ll) return false;
    }
}
// global -> shared bulk copy; completion is signalled on `bar` with the byte count.  dst, src and bytes are multiples of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 2-D tile copy: box of the tensor map at (x = innermost coordinate, y = row).  x times the element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// 3-D tile copy: box at (x, y, z); same alignment rule for x.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// Orders earlier generic-proxy accesses to shared memory before later async-proxy (TMA) writes to it.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_h(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}

}  // namespace cq
