// Counter-based normal generator used to fill KV caches with synthetic data.
// The value of element i depends only on (seed, i), so any shard of a tensor
// can be produced independently and two programs given the same (seed, i)
// produce the same fp16 bit pattern.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace cq {

__host__ __device__ inline uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ inline float normal_at(uint64_t seed, uint64_t i) {
    uint64_t h = splitmix64(seed * 0xD1342543DE82EF95ull + i);
    float u1 = ((float)((h >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f);   // (0,1]
    float u2 = (float)((h >> 16) & 0xFFFFFF) * (1.0f / 16777216.0f);            // [0,1)
    float r = sqrtf(-2.0f * __logf(u1));
    return r * __cosf(6.28318530718f * u2);
}

__global__ void fill_normal_kernel(__half* dst, size_t n, uint64_t seed, uint64_t base) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __float2half(normal_at(seed, base + i));
}

}  // namespace cq
