// Causal attention for a tile of prompt tokens over the head-major KV cache, and the row-wise kernels of the batched
// prefill (embedding rows, RMSNorm rows, bias + RoPE + cache store).  The reference prefills token by token through
// its decode kernels (src/main.cu:86-92); the arithmetic of every row here follows those kernels:
// RMSNorm src/kernels.cu:300-320, bias + rotate-half RoPE + cache store :370-398 / :326-347 / :468-472, attention
// softmax(q k / sqrt(d)) v :105-288.
//
// Attention: one CTA per (64 queries, query head); four warps of 16 query rows; 64-key tiles of K and V of the head's
// KV group double-buffered in shared memory (cp.async, 16-byte chunks XOR-swizzled by the row); Q K^T and P V on
// mma.sync.m16n8k16 with fp32 accumulation and an fp32 online softmax; query t (cache position pos0 + t) sees keys
// [0, pos0 + t].
#include "prefill.cuh"

namespace cq {

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
    const int n = pred ? 16 : 0;      // 0 source bytes: the 16 destination bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float pa_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }   // ex2(-inf) = 0

constexpr int kPaBM = 64, kPaBN = 64, kPaThreads = 128;

// rows [row0, row0 + 64) of a [.][HD] fp16 matrix with row pitch `pitch` elements -> swizzled tile; rows >= row_end zero
template <int HD>
__device__ __forceinline__ void load_tile(uint32_t dst, const __half* src, size_t pitch, int row0, int row_end) {
    constexpr int NCH = HD / 8;
#pragma unroll
    for (int j = 0; j < kPaBN * NCH / kPaThreads; ++j) {
        const int idx = threadIdx.x + j * kPaThreads;
        const int r = idx / NCH, c = idx % NCH;
        const bool ok = row0 + r < row_end;
        cp_async16(dst + r * (HD * 2) + ((c ^ (r & 7)) << 4), src + (size_t)(ok ? row0 + r : row0) * pitch + c * 8, ok);
    }
}

template <int HD>
__global__ void __launch_bounds__(kPaThreads) prefill_attn_kernel(const PfAttnArgs a) {
    constexpr int NCH = HD / 8, KS = HD / 16, TILE = kPaBN * HD * 2;
    extern __shared__ __align__(128) unsigned char pa_smem[];
    const uint32_t sq = smem_u32(pa_smem), sk = sq + TILE, sv = sk + 2 * TILE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int head = blockIdx.y, kvh = head / a.grp;
    const int q0 = (gridDim.x - 1 - blockIdx.x) * kPaBM;              // the longest tiles first
    const __half* kbase = a.kc + (size_t)kvh * a.max_seq * HD;
    const __half* vbase = a.vc + (size_t)kvh * a.max_seq * HD;
    const int q_hi = min(q0 + kPaBM, a.T);
    const int kmax = a.pos0 + q_hi;                                   // keys [0, kmax) matter to this tile
    const int n_tiles = (kmax + kPaBN - 1) / kPaBN;

    load_tile<HD>(sq, a.q + head * HD, (size_t)a.ldq, q0, a.T);
    load_tile<HD>(sk, kbase, HD, 0, kmax);
    load_tile<HD>(sv, vbase, HD, 0, kmax);
    cp_async_commit();

    uint32_t qf[KS][4];
    float o[NCH][4];
#pragma unroll
    for (int i = 0; i < NCH; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int p0 = a.pos0 + q0 + warp * 16 + g, p1 = p0 + 8;          // cache positions of this thread's two query rows

    for (int it = 0; it < n_tiles; ++it) {
        const int buf = it & 1;
        if (it + 1 < n_tiles) {
            load_tile<HD>(sk + (buf ^ 1) * TILE, kbase, HD, (it + 1) * kPaBN, kmax);
            load_tile<HD>(sv + (buf ^ 1) * TILE, vbase, HD, (it + 1) * kPaBN, kmax);
            cp_async_commit();
            cp_async_wait<1>();
        } else cp_async_wait<0>();
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int r = warp * 16 + (lane & 15), c = ks * 2 + (lane >> 4);
                ldsm_x4(sq + r * (HD * 2) + ((c ^ (r & 7)) << 4), qf[ks]);
            }
        }
        const uint32_t kt = sk + buf * TILE, vt = sv + buf * TILE;
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                const int r = np * 16 + (lane & 7) + (lane >> 4) * 8, c = ks * 2 + ((lane >> 3) & 1);
                ldsm_x4(kt + r * (HD * 2) + ((c ^ (r & 7)) << 4), b);
                mma_f16(s[2 * np], qf[ks], b[0], b[1]);
                mma_f16(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
        // scale, causal mask, online softmax (two rows per thread: g and g + 8)
        const int key0 = it * kPaBN + 2 * t;
        const bool need_mask = it * kPaBN + kPaBN - 1 > a.pos0 + q0 + warp * 16;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] *= a.scale_log2;
            if (need_mask) {
                const int k = key0 + i * 8;
                if (k > p0) s[i][0] = -INFINITY;
                if (k + 1 > p0) s[i][1] = -INFINITY;
                if (k > p1) s[i][2] = -INFINITY;
                if (k + 1 > p1) s[i][3] = -INFINITY;
            }
            mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
            mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);       // finite from the first tile on: key 0 is visible to every query
        const float al0 = pa_ex2(m0 - mn0), al1 = pa_ex2(m1 - mn1);
        m0 = mn0; m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t pf[4][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float e0 = pa_ex2(s[i][0] - mn0), e1 = pa_ex2(s[i][1] - mn0), e2 = pa_ex2(s[i][2] - mn1), e3 = pa_ex2(s[i][3] - mn1);
            rs0 += e0 + e1; rs1 += e2 + e3;
            pf[i >> 1][(i & 1) * 2] = pack_h2(e0, e1);
            pf[i >> 1][(i & 1) * 2 + 1] = pack_h2(e2, e3);
        }
        l0 = l0 * al0 + rs0; l1 = l1 * al1 + rs1;
#pragma unroll
        for (int i = 0; i < NCH; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int cp = 0; cp < NCH / 2; ++cp) {
                uint32_t b[4];
                const int r = j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = cp * 2 + (lane >> 4);
                ldsm_x4_t(vt + r * (HD * 2) + ((c ^ (r & 7)) << 4), b);
                mma_f16(o[2 * cp], pf[j], b[0], b[1]);
                mma_f16(o[2 * cp + 1], pf[j], b[2], b[3]);
            }
        }
        __syncthreads();            // everybody is done with this buffer before the copy after next overwrites it
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    const int t0 = q0 + warp * 16 + g, t1 = t0 + 8;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int col = head * HD + i * 8 + 2 * t;
        if (t0 < a.T) *reinterpret_cast<uint32_t*>(a.out + (size_t)t0 * a.ldq + col) = pack_h2(o[i][0] * i0, o[i][1] * i0);
        if (t1 < a.T) *reinterpret_cast<uint32_t*>(a.out + (size_t)t1 * a.ldq + col) = pack_h2(o[i][2] * i1, o[i][3] * i1);
    }
}

int launch_prefill_attn(int head_dim, const PfAttnArgs& a, cudaStream_t stream) {
    if (a.T <= 0 || a.pos0 < 0 || a.pos0 + a.T > a.max_seq || a.n_heads <= 0 || a.grp <= 0 || a.ldq % 8) return (int)cudaErrorInvalidValue;
    const dim3 grid((a.T + kPaBM - 1) / kPaBM, a.n_heads);
    const size_t smem = (size_t)5 * kPaBN * head_dim * 2;
    if (head_dim == 128) {
        static bool once = false;
        if (!once) { const cudaError_t e = cudaFuncSetAttribute(prefill_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return (int)e; once = true; }
        prefill_attn_kernel<128><<<grid, kPaThreads, smem, stream>>>(a);
    } else if (head_dim == 64) {
        static bool once = false;
        if (!once) { const cudaError_t e = cudaFuncSetAttribute(prefill_attn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return (int)e; once = true; }
        prefill_attn_kernel<64><<<grid, kPaThreads, smem, stream>>>(a);
    } else return (int)cudaErrorInvalidValue;
    return (int)cudaGetLastError();
}

// ---- row-wise kernels -----------------------------------------------------------------------------------------------
__global__ void pf_embed_kernel(const __half* __restrict__ table, const int* __restrict__ tokens, __half* __restrict__ x, int dim) {
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)tokens[blockIdx.x] * dim);
    uint4* dst = reinterpret_cast<uint4*>(x + (size_t)blockIdx.x * dim);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = src[i];
}

// out[t] = half(x[t] * rsqrt(mean(x[t]^2) + eps) * w), one CTA per token
__global__ void __launch_bounds__(256) pf_rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ w, __half* __restrict__ out, int dim, float eps) {
    __shared__ float red[33];
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)blockIdx.x * dim);
    uint4* orow = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * dim);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    const float inv = block_inv_rms(x + (size_t)blockIdx.x * dim, dim, eps, red);
    for (int i = threadIdx.x; i < dim / 8; i += 256) {
        uint4 v = xr[i];
        const uint4 wv = wr[i];
        __half2* xh = reinterpret_cast<__half2*>(&v);
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 xf = __half22float2(xh[k]), wf = __half22float2(wh[k]);
            xh[k] = __floats2half2_rn(xf.x * inv * wf.x, xf.y * inv * wf.y);
        }
        orow[i] = v;
    }
}

// qkv: fp32 [T][q_dim + 2 kv_dim] straight from the GEMMs.  Bias in fp32, one rounding to fp16, rotate-half RoPE on q
// and k from the rounded values, k and v into cache row pos0 + t - the arithmetic of the decode kernel's epilogue.
__global__ void pf_rope_kv_kernel(const PfRopeArgs a) {
    const int tkn = blockIdx.x, half_hd = a.hd / 2;
    const int nq = a.n_heads * half_hd, nk = a.n_kv * half_hd;
    const float* row = a.qkv + (size_t)tkn * (a.q_dim + 2 * a.kv_dim);
    const int pos = a.pos0 + tkn;
    for (int i = threadIdx.x; i < nq + 2 * nk; i += blockDim.x) {
        const int mat = i < nq ? 0 : i < nq + nk ? 1 : 2;
        const int j = mat == 0 ? i : mat == 1 ? i - nq : i - nq - nk;
        const int head = j / half_hd, d = j % half_hd;
        const int ra = head * a.hd + d, rb = ra + half_hd;
        const int off = mat == 0 ? 0 : mat == 1 ? a.q_dim : a.q_dim + a.kv_dim;
        const __half* bias = mat == 0 ? a.bq : mat == 1 ? a.bk : a.bv;
        const float b0 = bias ? __half2float(bias[ra]) : 0.f, b1 = bias ? __half2float(bias[rb]) : 0.f;
        const float f0 = __half2float(__float2half(row[off + ra] + b0)), f1 = __half2float(__float2half(row[off + rb] + b1));
        __half o0, o1;
        if (mat < 2) {
            float c, s;
            rope_cs(d, a.hd, pos, a.theta, a.rope_fast, &c, &s);
            o0 = __float2half(f0 * c - f1 * s); o1 = __float2half(f1 * c + f0 * s);
        } else { o0 = __float2half(f0); o1 = __float2half(f1); }
        if (mat == 0) { a.q_out[(size_t)tkn * a.q_dim + ra] = o0; a.q_out[(size_t)tkn * a.q_dim + rb] = o1; }
        else {
            __half* cache = mat == 1 ? a.kcache : a.vcache;
            const size_t base = ((size_t)head * a.max_seq + pos) * a.hd;
            cache[base + d] = o0; cache[base + d + half_hd] = o1;
        }
    }
}

int launch_pf_embed(const __half* table, const int* d_tokens, __half* x, int T, int dim, cudaStream_t s) {
    pf_embed_kernel<<<T, 128, 0, s>>>(table, d_tokens, x, dim);
    return (int)cudaGetLastError();
}
int launch_pf_rmsnorm(const __half* x, const __half* w, __half* out, int T, int dim, float eps, cudaStream_t s) {
    pf_rmsnorm_kernel<<<T, 256, 0, s>>>(x, w, out, dim, eps);
    return (int)cudaGetLastError();
}
int launch_pf_rope_kv(const PfRopeArgs& a, int T, cudaStream_t s) {
    pf_rope_kv_kernel<<<T, 256, 0, s>>>(a);
    return (int)cudaGetLastError();
}

}  // namespace cq
