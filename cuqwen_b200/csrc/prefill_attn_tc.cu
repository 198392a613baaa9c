// Causal attention for a tile of prompt tokens on the tcgen05 tensor cores (head_dim 64 or 128): the batched counterpart of
// the reference's decode attention (src/kernels.cu:105-288), which the reference applies once per prompt token
// (src/main.cu:86-92).  prefill_attn.cu holds the mma.sync kernel this one replaces (kept as the comparison variant).
//
// One CTA = 128 queries of one head, two CTAs to an SM.  Per tile of 64 keys:
//   warp 0      TMA: K and V tiles of the head's KV group (two 64-column boxes each, hardware-swizzled), two slots
//   warp 1      one lane issues S = Q K^T (eight MMAs 128 x 64 x 16, both operands K-major) into one of two TMEM
//               buffers, and - once the softmax warps have written P - O += P V (four MMAs 128 x 128 x 16, V as the MN-major B
//               operand straight from its cache layout) into a third
//   warps 2-9   two threads per query row (TMEM lane = row), 32 of the tile's keys each: read S, scale, mask, write
//               P = 2^(s - m) as fp16 into the swizzled A tile, row sums in fp32; when a row's maximum outgrows m by
//               2^8, m moves and O is rescaled in TMEM by 2^(m_old - m_new) (rare after the first tiles)
// S of the next tile is issued before the current tile's P is waited for, so Q K^T overlaps the softmax.
// Every mbarrier wait is bounded; a wait that runs out sets *err and the CTA drains.
#include "prefill.cuh"
#include "tcgen05.cuh"

namespace cq {

constexpr int kTaBM = 128, kTaBN = 64;
constexpr int kTaThreads = 320;                   // warp 0 TMA, warp 1 MMA, warps 2-9 softmax
constexpr int kTaPTile = kTaBM * kTaBN * 2;       // 16 KB: [128 rows][64 keys]
// Per head_dim HD (128 or 64): Q tile = HD / 64 blocks of [128 rows][128 bytes], K and V tiles = HD / 64 blocks of
// [64 keys][128 bytes].  Q, K x 2, V x 2, P, barriers (the dynamic shared memory is declared 1024-byte aligned):
// 113 KB for HD 128 and at most 102 registers, so two CTAs share an SM and one's softmax runs under the other's MMAs.
// Twice 115,456 B and the 1 KB the system keeps per CTA fit an SM's 228 KB.
__host__ __device__ constexpr int ta_q_tile(int hd) { return kTaBM * hd * 2; }
__host__ __device__ constexpr int ta_k_tile(int hd) { return kTaBN * hd * 2; }
__host__ __device__ constexpr int ta_smem(int hd) { return ta_q_tile(hd) + 4 * ta_k_tile(hd) + kTaPTile + 256 + 512; }   // + barriers, + the softmax warps' exchange words
constexpr uint32_t kTaCols = 256;                 // TMEM columns: S x 2 (64 each), O (HD)

struct PfAttnTcArgs {
    CUtensorMap tq;          // q as [T][ldq] fp16, box 64 x 128, swizzled
    CUtensorMap tk, tv;      // caches as [n_kv][max_seq][hd] fp16, box 64 x 64 x 1, swizzled
    __half* out;
    int T, pos0, n_heads, grp, ldq;
    float scale_log2;
    unsigned* err;
};

__device__ __forceinline__ float ta_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void ta_sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(kTaThreads, 2) prefill_attn_tc_kernel(const __grid_constant__ PfAttnTcArgs a) {
    constexpr int kTaHD = HD, kTaQTile = ta_q_tile(HD), kTaQHalf = kTaBM * 128, kTaKTile = ta_k_tile(HD), kTaKHalf = kTaBN * 128, NBLK = HD / 64;
    extern __shared__ __align__(1024) unsigned char ta_smem[];
    const uint32_t base = smem_u32(ta_smem);
    const uint32_t sQ = base, sK = base + kTaQTile, sV = sK + 2 * kTaKTile, sP = sV + 2 * kTaKTile;
    const uint32_t bars = sP + kTaPTile;
    const uint32_t b_q = bars, b_kvfull = bars + 8, b_kvfree = bars + 24, b_sfull = bars + 40, b_p = bars + 56, b_pv = bars + 64, tmem_slot = bars + 72;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y, kvh = head / a.grp;
    const int q0 = (gridDim.x - 1 - blockIdx.x) * kTaBM;                  // the longest tiles first
    const int kmax = a.pos0 + min(q0 + kTaBM, a.T);                      // keys [0, kmax) matter to this tile
    const int nj = (kmax + kTaBN - 1) / kTaBN;
    bool failed = false;

    if (threadIdx.x == 0) {
        mbar_init(b_q, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(b_kvfull + 8 * s, 1); mbar_init(b_kvfree + 8 * s, 1); mbar_init(b_sfull + 8 * s, 1); }
        mbar_init(b_p, 8); mbar_init(b_pv, 1);
        mbar_fence_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, kTaCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = lds32(tmem_slot);
    const uint32_t tS = tmem, tO = tmem + 2u * kTaBN;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(b_q, (uint32_t)kTaQTile);
            for (int b = 0; b < NBLK; ++b) tma_load_2d(sQ + b * kTaQHalf, &a.tq, head * kTaHD + 64 * b, q0, b_q);
            for (int j = 0; j < nj; ++j) {
                const int s = j & 1;
                if (!mbar_wait(b_kvfree + 8 * s, (((uint32_t)j >> 1) & 1u) ^ 1u)) { failed = true; break; }
                mbar_expect_tx(b_kvfull + 8 * s, 2u * kTaKTile);
                for (int b = 0; b < NBLK; ++b) {
                    tma_load_3d(sK + s * kTaKTile + b * kTaKHalf, &a.tk, 64 * b, j * kTaBN, kvh, b_kvfull + 8 * s);
                    tma_load_3d(sV + s * kTaKTile + b * kTaKHalf, &a.tv, 64 * b, j * kTaBN, kvh, b_kvfull + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idS = umma_idesc_f16(kTaBM, kTaBN, 0), idPV = umma_idesc_f16(kTaBM, kTaHD, 1);
            auto issue_s = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait(b_kvfull + 8 * s, ((uint32_t)j >> 1) & 1u)) return false;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kTaHD / 16; ++ks) {
                    umma_f16(tS + (uint32_t)(s * kTaBN), umma_desc_sw128(sQ + (uint32_t)((ks >> 2) * kTaQHalf + (ks & 3) * 32), 16, 1024),
                             umma_desc_sw128(sK + s * kTaKTile + (uint32_t)((ks >> 2) * kTaKHalf + (ks & 3) * 32), 16, 1024), idS, (uint32_t)(ks != 0));
                }
                umma_commit(b_sfull + 8 * s);
                return true;
            };
            if (!mbar_wait(b_q, 0u)) failed = true;
            if (!failed && !issue_s(0)) failed = true;
            for (int j = 0; j < nj && !failed; ++j) {
                const int s = j & 1;
                if (j + 1 < nj && !issue_s(j + 1)) { failed = true; break; }
                if (!mbar_wait(b_p, (uint32_t)j & 1u)) { failed = true; break; }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kTaBN / 16; ++ks)       // sixteen keys a step: V rows 16 ks .., P columns 16 ks ..
                    umma_f16(tO, umma_desc_sw128(sP + (uint32_t)(ks * 32), 16, 1024),
                             umma_desc_sw128(sV + s * kTaKTile + ks * 2048, kTaKHalf, 1024), idPV, (uint32_t)((j | ks) != 0));
                umma_commit(b_pv);
                umma_commit(b_kvfree + 8 * s);
            }
        }
    } else {
        // Eight softmax warps: two per TMEM lane quarter (a warp reaches the 32 lanes its number mod 4 names), each with
        // 32 of a tile's 64 keys and half of the output columns of the same 32 query rows.  The two threads of a row
        // agree on the row's scaling exponent through 512 bytes of shared memory and two named barriers per tile - so
        // nothing below leaves the tile loop early: after a wait has run out the warp keeps going without waiting.
        const int q = warp & 3, hsel = (warp - 2) >> 2;
        const int r = q * 32 + lane;                                      // query row of the tile = TMEM lane
        const int qpos = a.pos0 + q0 + r;
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        __half* mxbuf = reinterpret_cast<__half*>(ta_smem + (bars - base) + 256);      // [2 halves][128 rows]
        constexpr int OC = HD / 2;                                        // output columns of this thread
        // m is the exponent the row's probabilities are scaled by, not always its running maximum: it moves only when
        // a tile's maximum exceeds it by more than 2^8 (probabilities then stay below 256, well inside fp16, and the
        // row sum is fp32), so that most tiles need no rescale of O in TMEM.
        float m = -INFINITY, l = 0.f;
        for (int j = 0; j < nj; ++j) {
            const int s = j & 1;
            if (!failed && !mbar_wait(b_sfull + 8 * s, ((uint32_t)j >> 1) & 1u)) failed = true;
            tc_fence_after();
            const bool diag = j * kTaBN + kTaBN - 1 > a.pos0 + q0;        // some key of this tile may lie past some query (uniform over the CTA)
            float x[32];
            tmem_ld32(tS + (uint32_t)(s * kTaBN + hsel * 32) + lane_off, x);
            float mxl = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                x[i] *= a.scale_log2;
                if (diag && j * kTaBN + hsel * 32 + i > qpos) x[i] = -INFINITY;
                mxl = fmaxf(mxl, x[i]);
            }
            const __half hmx = __float2half_ru(mxl);                      // rounded up: both threads of the row then hold the same two numbers
            mxbuf[hsel * 128 + r] = hmx;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float mx = fmaxf(__half2float(hmx), __half2float(mxbuf[(hsel ^ 1) * 128 + r]));
            asm volatile("bar.sync 1, 256;" ::: "memory");                // everybody has read before the next tile's maxima are written
            float alpha = 1.f;
            const bool mine = mx > m + 8.0f;                              // also true on the first tile (m = -inf; key 0 is visible to every query)
            const bool moved = __any_sync(0xffffffffu, mine);             // warp-uniform (the TMEM accesses below are warp-wide); the row's other warp decides alike
            if (mine) { alpha = m == -INFINITY ? 0.f : ta_ex2(m - mx); m = mx; }
            float rs = 0.f;
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float e0 = ta_ex2(x[i] - m), e1 = ta_ex2(x[i + 1] - m);
                rs += e0 + e1;
                pk[i >> 1] = pack_h2(e0, e1);
            }
            if (j > 0) {
                if (!failed && !mbar_wait(b_pv, (uint32_t)(j - 1) & 1u)) failed = true;   // P V of the previous tile is complete: O and the P tile are ours
                tc_fence_after();
                if (moved) {
#pragma unroll 1
                    for (int c = 0; c < OC / 32; ++c) {
                        float v[32];
                        tmem_ld32(tO + lane_off + (uint32_t)(hsel * OC + c * 32), v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] *= alpha;
                        tmem_st32(tO + lane_off + (uint32_t)(hsel * OC + c * 32), v);
                    }
                    tmem_wait_st();
                }
            }
            const uint32_t prow = sP + (uint32_t)(r * 128);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                ta_sts128(prow + ((uint32_t)((hsel * 4 + i) ^ (r & 7)) << 4), make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]));
            l = l * alpha + rs;
            fence_async_smem();                                           // the tensor core reads P through the async proxy
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_p);
        }
        // the row's sum: the second half hands its part to the first, which hands back the total
        float* lbuf = reinterpret_cast<float*>(mxbuf);                    // 128 floats
        if (hsel == 1) lbuf[r] = l;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (hsel == 0) { l += lbuf[r]; lbuf[r] = l; }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (hsel == 1) l = lbuf[r];
        if (!failed && !mbar_wait(b_pv, (uint32_t)(nj - 1) & 1u)) failed = true;
        tc_fence_after();
        {
            const float inv = 1.0f / l;
            const int t = q0 + r;
#pragma unroll 1
            for (int c = 0; c < OC / 32; ++c) {
                float v[32];
                tmem_ld32(tO + lane_off + (uint32_t)(hsel * OC + c * 32), v);
                if (t < a.T && !failed) {
                    __half* dst = a.out + (size_t)t * a.ldq + head * kTaHD + hsel * OC + c * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        *reinterpret_cast<uint4*>(dst + i) = make_uint4(pack_h2(v[i] * inv, v[i + 1] * inv), pack_h2(v[i + 2] * inv, v[i + 3] * inv),
                                                                        pack_h2(v[i + 4] * inv, v[i + 5] * inv), pack_h2(v[i + 6] * inv, v[i + 7] * inv));
                }
                __syncwarp();
            }
        }
    }
    if (failed && a.err) atomicExch(a.err, 12u);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTaCols);
}

typedef CUresult (*TaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TaEncodeFn ta_encode() {
    static TaEncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return (TaEncodeFn)p;
    }();
    return fn;
}

template <int HD>
static int ta_go(const PfAttnTcArgs& k, dim3 grid, cudaStream_t stream) {
    static bool once = false;
    if (!once) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_attn_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, ta_smem(HD));
        if (e != cudaSuccess) return (int)e;
        once = true;
    }
    prefill_attn_tc_kernel<HD><<<grid, kTaThreads, ta_smem(HD), stream>>>(k);
    return (int)cudaGetLastError();
}

int launch_prefill_attn_tc(int head_dim, const PfAttnArgs& a, int n_kv, unsigned* err, cudaStream_t stream) {
    const int kTaHD = head_dim;
    if (head_dim != 64 && head_dim != 128) return (int)cudaErrorInvalidValue;
    if (a.T <= 0 || a.pos0 < 0 || a.pos0 + a.T > a.max_seq || a.n_heads <= 0 || a.grp <= 0 || a.ldq % 8 || n_kv <= 0) return (int)cudaErrorInvalidValue;
    TaEncodeFn fn = ta_encode();
    if (!fn) return (int)cudaErrorNotSupported;
    PfAttnTcArgs k; memset(&k, 0, sizeof k);
    const cuuint32_t estr[3] = {1, 1, 1};
    {
        const cuuint64_t dims[2] = {(cuuint64_t)a.ldq, (cuuint64_t)a.T}, strides[1] = {(cuuint64_t)a.ldq * 2};
        const cuuint32_t box[2] = {64, kTaBM};
        if (fn(&k.tq, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(a.q), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    const __half* caches[2] = {a.kc, a.vc};
    CUtensorMap* maps[2] = {&k.tk, &k.tv};
    for (int i = 0; i < 2; ++i) {
        const cuuint64_t dims[3] = {(cuuint64_t)kTaHD, (cuuint64_t)a.max_seq, (cuuint64_t)n_kv};
        const cuuint64_t strides[2] = {(cuuint64_t)kTaHD * 2, (cuuint64_t)a.max_seq * kTaHD * 2};
        const cuuint32_t box[3] = {64, kTaBN, 1};
        if (fn(maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(caches[i]), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    }
    k.out = a.out; k.T = a.T; k.pos0 = a.pos0; k.n_heads = a.n_heads; k.grp = a.grp; k.ldq = a.ldq; k.scale_log2 = a.scale_log2; k.err = err;
    const dim3 grid((a.T + kTaBM - 1) / kTaBM, a.n_heads);
    return head_dim == 128 ? ta_go<128>(k, grid, stream) : ta_go<64>(k, grid, stream);
}

}  // namespace cq
