// Shared device helpers for the sm_100a decode kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cq {

constexpr int kGroup = 128;  // weights per fp16 scale along the input dim (reference include/config.h:16)

enum Quant : int { Q_F16 = 0, Q_I8 = 1, Q_I4 = 2 };

// Tensor-parallel exchanges are numbered  step * kSeqPerStep + index + 1  (index < kSeqPerStep: two per layer and a few
// per token), so that a receive word left over from an earlier exchange can never carry the number a reader expects.
constexpr unsigned kSeqPerStep = 512u;
constexpr long long kWaitCyclesDefault = 4000000000ll;     // bound of every device-side wait, in SM cycles (two to four seconds)

// One exchange word = {fp32 value bits (low half), sequence number (high half)} moved as ONE 64-bit access, so that the
// pair is written and read indivisibly by the memory model (a vector access of two 32-bit elements would not be).
__device__ __forceinline__ void st_pair(void* p, unsigned value_bits, unsigned seq) {
    const unsigned long long w = ((unsigned long long)seq << 32) | value_bits;
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
// Two adjacent exchange words (16 bytes) as two 64-bit elements.
__device__ __forceinline__ void ld_pair2(const void* p, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned pair_seq(unsigned long long w) { return (unsigned)(w >> 32); }
__device__ __forceinline__ float pair_val(unsigned long long w) { return __uint_as_float((unsigned)(w & 0xffffffffull)); }

// Streaming 128-bit read of data that is touched once per step (weights, KV):
// read-only path, do not keep it in L1.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// 16-bit read into a full 32-bit register (zero-extended): the value can sit in flight without the
// compiler packing it next to a neighbour, which would put a dependent instruction right behind the load.
__device__ __forceinline__ uint32_t ldg_u16(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t u4c(const uint4& v, int j) { return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w; }
// (a & b) ^ c in one LOP3.
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col).  Lane = 4*g + t:
//   a0:(row g, k 2t..2t+1)  a1:(row g+8, same k)  a2:(row g, k 2t+8..)  a3:(row g+8, k 2t+8..)
//   b0:(k 2t..2t+1, col g)  b1:(k 2t+8.., col g)
//   c0,c1:(row g, col 2t,2t+1)  c2,c3:(row g+8, col 2t,2t+1)
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Programmatic dependent launch: a kernel may start while its predecessor in
// the stream drains; everything before pdl_wait() must not touch data the
// predecessor writes.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// sum of squares -> 1/rms, in the whole CTA.  `red` holds >= 33 floats.
__device__ __forceinline__ float block_inv_rms(const __half* __restrict__ x, int dim, float eps, float* red) {
    float ss = 0.f;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
        uint4 v = xv[i];
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 f = __half22float2(h[k]);
            ss += f.x * f.x + f.y * f.y;
        }
    }
    for (int i = (dim / 8) * 8 + threadIdx.x; i < dim; i += blockDim.x) {
        float f = __half2float(x[i]);
        ss += f * f;
    }
    ss = warp_sum(ss);
    __syncthreads();  // protects `red` against a previous use
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[32] = rsqrtf(v / (float)dim + eps);
    }
    __syncthreads();
    return red[32];
}

// RoPE angle terms.  fast = 1 reproduces the arithmetic the reference build
// gets from --use_fast_math (approximate pow/div/sin/cos), fast = 0 is the
// accurate form.  Reference: src/kernels.cu:385-388.
__device__ __forceinline__ void rope_cs(int i, int head_dim, int pos, float theta, int fast, float* c, float* s) {
    if (fast) {
        float e = __fdividef(2.0f * (float)i, (float)head_dim);
        float freq = __fdividef(1.0f, __powf(theta, e));
        float val = (float)pos * freq;
        *c = __cosf(val);
        *s = __sinf(val);
    } else {
        float freq = 1.0f / powf(theta, (2.0f * (float)i) / (float)head_dim);
        float val = (float)pos * freq;
        sincosf(val, s, c);
    }
}

}  // namespace cq
