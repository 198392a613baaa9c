// One 16-key tile of decode attention for all query heads of a KV head, on mma.sync.m16n8k16:
// Q.K^T with the query heads on the M side, online softmax in fp32 (log2 units), P.V with the head dimension on the M
// side and the heads on the N side, so that the C fragment of the first product is the B fragment of the second.
// Reference arithmetic being replaced: src/kernels.cu:105-219 (there: fp16 scores and probabilities, WMMA).
#pragma once
#include "attn_combine.cuh"
#include "tma.cuh"

namespace cq {

template <int HD>
struct AttnState {
    float o[HD / 16][4];   // un-normalised output: m-tile = 16 d values, columns = heads 2t, 2t+1
    float m_run, l_run;    // running maximum (log2 units) and sum of head g (lanes of one g hold partial sums of l)
    __device__ __forceinline__ void reset() {
#pragma unroll
        for (int m = 0; m < HD / 16; ++m) o[m][0] = o[m][1] = o[m][2] = o[m][3] = 0.f;
        m_run = -INFINITY; l_run = 0.f;
    }
};

// A operand of Q.K^T: q of head g of the KV head's group (zero rows for g >= grp), read through L2.
template <int HD>
__device__ __forceinline__ void attn_load_q(uint32_t (&qa)[HD / 32][4], const __half* q_group, int grp, int g, int t) {
    const __half* qrow = q_group + (size_t)g * HD;
#pragma unroll
    for (int i = 0; i < HD / 32; ++i) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < grp) v = __ldcg(reinterpret_cast<const uint4*>(qrow + (i * 4 + t) * 8));
        qa[i][0] = v.x; qa[i][1] = v.y; qa[i][2] = v.z; qa[i][3] = v.w;
    }
}

template <bool FROM_GLOBAL>
__device__ __forceinline__ uint4 attn_ld16(const unsigned char* p) {
    if (FROM_GLOBAL) return __ldcg(reinterpret_cast<const uint4*>(p));
    return lds128(smem_u32(p));        // explicit shared-window load: stays ld.shared even where the pointer's origin is not visible
}

// sK / sV: rows [key][HD] fp16 of the tile's 16 keys; nvalid >= 1 of them exist (the rest are never read).
// FROM_GLOBAL: the rows are in global memory and were written during this step (read through L2).
template <int HD, bool FROM_GLOBAL>
__device__ __forceinline__ void attn_tile(AttnState<HD>& st, const uint32_t (&qa)[HD / 32][4], const unsigned char* sK, const unsigned char* sV,
                                          int nvalid, float scale_log2, int g, int t) {
    constexpr int NCH = HD / 32;   // 16-byte chunks of a K row per lane (4 lanes cover 64 B)
    constexpr int NC = HD / 64;    // 16-byte chunks of a V row per lane (8 lanes cover 128 B)
    constexpr int NMT = HD / 16;
    constexpr int ROWB = HD * 2;
    uint4 kA[NCH], kB[NCH], vv[4][NC];
    const bool vA = g < nvalid, vB = 8 + g < nvalid;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        kA[i] = vA ? attn_ld16<FROM_GLOBAL>(sK + g * ROWB + (i * 4 + t) * 16) : make_uint4(0, 0, 0, 0);
        kB[i] = vB ? attn_ld16<FROM_GLOBAL>(sK + (g + 8) * ROWB + (i * 4 + t) * 16) : make_uint4(0, 0, 0, 0);
    }
    float sA[4] = {0.f, 0.f, 0.f, 0.f}, sB[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        mma16816(sA, qa[i][0], 0u, qa[i][1], 0u, kA[i].x, kA[i].y);
        mma16816(sA, qa[i][2], 0u, qa[i][3], 0u, kA[i].z, kA[i].w);
        mma16816(sB, qa[i][0], 0u, qa[i][1], 0u, kB[i].x, kB[i].y);
        mma16816(sB, qa[i][2], 0u, qa[i][3], 0u, kB[i].z, kB[i].w);
    }
    // lane holds head g, keys 2t, 2t+1 (sA) and 8+2t, 9+2t (sB)
    const float s0 = 2 * t < nvalid ? sA[0] * scale_log2 : -INFINITY;
    const float s1 = 2 * t + 1 < nvalid ? sA[1] * scale_log2 : -INFINITY;
    const float s2 = 8 + 2 * t < nvalid ? sB[0] * scale_log2 : -INFINITY;
    const float s3 = 9 + 2 * t < nvalid ? sB[1] * scale_log2 : -INFINITY;
    float mx = fmaxf(fmaxf(s0, s1), fmaxf(s2, s3));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m_run, mx);       // finite: key 0 of the tile is always valid
    const float alpha = ex2(st.m_run - m_new);
    const float p0 = ex2(s0 - m_new), p1 = ex2(s1 - m_new), p2 = ex2(s2 - m_new), p3 = ex2(s3 - m_new);
    st.l_run = st.l_run * alpha + ((p0 + p1) + (p2 + p3));
    st.m_run = m_new;
    const uint32_t pb0 = pack_h2(p0, p1), pb1 = pack_h2(p2, p3);
    // V fragments only now: the K fragments are dead by here, which keeps the register peak of the tile low
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int kr = 2 * t + (r & 1) + (r >> 1) * 8;
#pragma unroll
        for (int c = 0; c < NC; ++c)
            vv[r][c] = kr < nvalid ? attn_ld16<FROM_GLOBAL>(sV + kr * ROWB + (c * 8 + g) * 16) : make_uint4(0, 0, 0, 0);
    }
    // O columns of this lane are heads 2t and 2t+1
    const float al = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4), ah = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
    if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int m = 0; m < NMT; ++m) { st.o[m][0] *= al; st.o[m][1] *= ah; st.o[m][2] *= al; st.o[m][3] *= ah; }
    }
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int ep = 0; ep < 4; ++ep) {
            const uint32_t wA = u4c(vv[0][c], ep), wB = u4c(vv[1][c], ep), wC = u4c(vv[2][c], ep), wD = u4c(vv[3][c], ep);
            mma16816(st.o[c * 4 + ep], prmt(wA, wB, 0x5410), prmt(wA, wB, 0x7632), prmt(wC, wD, 0x5410), prmt(wC, wD, 0x7632), pb0, pb1);
        }
}

// Eight signed bytes (two 32-bit words) -> eight fp16 values in four half2 registers, exactly: the byte with its sign
// bit flipped becomes the mantissa of 1024 + (v + 128) (prmt with 0x64 as the high byte), from which 1152 is taken.
__device__ __forceinline__ uint4 s8x8_to_h8(uint2 w) {
    const uint32_t x0 = w.x ^ 0x80808080u, x1 = w.y ^ 0x80808080u;
    const __half2 off = __halves2half2(__ushort_as_half((unsigned short)0x6480), __ushort_as_half((unsigned short)0x6480));   // 1152
    uint32_t r[4] = {prmt(x0, 0x64646464u, 0x5140), prmt(x0, 0x64646464u, 0x7362), prmt(x1, 0x64646464u, 0x5140), prmt(x1, 0x64646464u, 0x7362)};
#pragma unroll
    for (int i = 0; i < 4; ++i) { __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r[i]), off); r[i] = *reinterpret_cast<uint32_t*>(&h); }
    return make_uint4(r[0], r[1], r[2], r[3]);
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
// Eight consecutive head-dimension values of one cached row as fp16 fragments: from an fp16 row (16 bytes) or, KV8,
// from an int8 row (8 bytes; the row's scale is applied by the caller, to the score or to the probability).
template <bool KV8>
__device__ __forceinline__ uint4 attn_row8(const unsigned char* row, int chunk8) {
    if (KV8) return s8x8_to_h8(lds64(smem_u32(row + chunk8 * 8)));
    return lds128(smem_u32(row + chunk8 * 16));
}

// Two adjacent 16-key tiles (32 keys) in one step.  Same arithmetic per key as attn_tile, but the four 8-key score
// blocks form four independent MMA chains, the softmax state is updated once for all 32 keys (one maximum, one
// rescale of O) and every output tile takes two chained MMAs - more independent work per warp between the points
// where everything waits on a shuffle or an ex2.  nvalid in [1, 32].
// KV8: the rows are int8 (HD bytes each) and sKs / sVs hold the 32 keys' fp32 scales: a key's K scale multiplies its
// score, its V scale its probability on the way into P.V (the softmax sum keeps the unscaled probability).
template <int HD, bool KV8 = false>
__device__ __forceinline__ void attn_tile32(AttnState<HD>& st, const uint32_t (&qa)[HD / 32][4], const unsigned char* sK, const unsigned char* sV,
                                            int nvalid, float scale_log2, int g, int t, const float* sKs = nullptr, const float* sVs = nullptr) {
    constexpr int NCH = HD / 32, NC = HD / 64, NMT = HD / 16, ROWB = KV8 ? HD : HD * 2;
    float sc[4][4];                          // block b = keys 8b .. 8b+7: lane holds head g, keys 8b+2t, 8b+2t+1 in [0], [1]
#pragma unroll
    for (int b = 0; b < 4; ++b) sc[b][0] = sc[b][1] = sc[b][2] = sc[b][3] = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        uint4 kf[4];
#pragma unroll
        for (int b = 0; b < 4; ++b)
            kf[b] = 8 * b + g < nvalid ? attn_row8<KV8>(sK + (8 * b + g) * ROWB, i * 4 + t) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            mma16816(sc[b], qa[i][0], 0u, qa[i][1], 0u, kf[b].x, kf[b].y);
            mma16816(sc[b], qa[i][2], 0u, qa[i][3], 0u, kf[b].z, kf[b].w);
        }
    }
    float s[4][2];
    float mx = -INFINITY;
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[b][j] = 8 * b + 2 * t + j < nvalid ? sc[b][j] * (KV8 ? scale_log2 * sKs[8 * b + 2 * t + j] : scale_log2) : -INFINITY;
            mx = fmaxf(mx, s[b][j]);
        }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m_run, mx);       // finite: key 0 is always valid
    const float alpha = ex2(st.m_run - m_new);
    float psum = 0.f;
    uint32_t pb[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float p0 = ex2(s[b][0] - m_new), p1 = ex2(s[b][1] - m_new);
        psum += p0 + p1;
        if (KV8) pb[b] = pack_h2(8 * b + 2 * t < nvalid ? p0 * sVs[8 * b + 2 * t] : 0.f, 8 * b + 2 * t + 1 < nvalid ? p1 * sVs[8 * b + 2 * t + 1] : 0.f);
        else pb[b] = pack_h2(p0, p1);
    }
    st.l_run = st.l_run * alpha + psum;
    st.m_run = m_new;
    const float al = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4), ah = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
    if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int m = 0; m < NMT; ++m) { st.o[m][0] *= al; st.o[m][1] *= ah; st.o[m][2] *= al; st.o[m][3] *= ah; }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {            // keys 16h .. 16h+15: one k-step of P.V
        uint4 vv[4][NC];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int kr = 16 * h + 2 * t + (r & 1) + (r >> 1) * 8;
#pragma unroll
            for (int c = 0; c < NC; ++c)
                vv[r][c] = kr < nvalid ? attn_row8<KV8>(sV + kr * ROWB, c * 8 + g) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int ep = 0; ep < 4; ++ep) {
                const uint32_t wA = u4c(vv[0][c], ep), wB = u4c(vv[1][c], ep), wC = u4c(vv[2][c], ep), wD = u4c(vv[3][c], ep);
                mma16816(st.o[c * 4 + ep], prmt(wA, wB, 0x5410), prmt(wA, wB, 0x7632), prmt(wC, wD, 0x5410), prmt(wC, wD, 0x7632), pb[2 * h], pb[2 * h + 1]);
            }
    }
}

// attn_tile32 over an 8-bit cache.  Same arithmetic per key as attn_tile, but the four 8-key score
// blocks form four independent MMA chains, the softmax state is updated once for all 32 keys (one maximum, one
// rescale of O) and every output tile takes two chained MMAs - more independent work per warp between the points
// where everything waits on a shuffle or an ex2.  nvalid in [1, 32].
// KV8: the rows are int8 (HD bytes each) and sKs / sVs hold the 32 keys' fp32 scales: a key's K scale multiplies its
// score, its V scale its probability on the way into P.V (the softmax sum keeps the unscaled probability).
template <int HD, bool KV8 = true>
__device__ __forceinline__ void attn_tile32_q8(AttnState<HD>& st, const uint32_t (&qa)[HD / 32][4], const unsigned char* sK, const unsigned char* sV,
                                            int nvalid, float scale_log2, int g, int t, const float* sKs = nullptr, const float* sVs = nullptr) {
    constexpr int NCH = HD / 32, NC = HD / 64, NMT = HD / 16, ROWB = KV8 ? HD : HD * 2;
    float sc[4][4];                          // block b = keys 8b .. 8b+7: lane holds head g, keys 8b+2t, 8b+2t+1 in [0], [1]
#pragma unroll
    for (int b = 0; b < 4; ++b) sc[b][0] = sc[b][1] = sc[b][2] = sc[b][3] = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        uint4 kf[4];
#pragma unroll
        for (int b = 0; b < 4; ++b)
            kf[b] = 8 * b + g < nvalid ? attn_row8<KV8>(sK + (8 * b + g) * ROWB, i * 4 + t) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            mma16816(sc[b], qa[i][0], 0u, qa[i][1], 0u, kf[b].x, kf[b].y);
            mma16816(sc[b], qa[i][2], 0u, qa[i][3], 0u, kf[b].z, kf[b].w);
        }
    }
    float s[4][2];
    float mx = -INFINITY;
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[b][j] = 8 * b + 2 * t + j < nvalid ? sc[b][j] * (KV8 ? scale_log2 * sKs[8 * b + 2 * t + j] : scale_log2) : -INFINITY;
            mx = fmaxf(mx, s[b][j]);
        }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m_run, mx);       // finite: key 0 is always valid
    const float alpha = ex2(st.m_run - m_new);
    float psum = 0.f;
    uint32_t pb[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float p0 = ex2(s[b][0] - m_new), p1 = ex2(s[b][1] - m_new);
        psum += p0 + p1;
        if (KV8) pb[b] = pack_h2(8 * b + 2 * t < nvalid ? p0 * sVs[8 * b + 2 * t] : 0.f, 8 * b + 2 * t + 1 < nvalid ? p1 * sVs[8 * b + 2 * t + 1] : 0.f);
        else pb[b] = pack_h2(p0, p1);
    }
    st.l_run = st.l_run * alpha + psum;
    st.m_run = m_new;
    const float al = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4), ah = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
    if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int m = 0; m < NMT; ++m) { st.o[m][0] *= al; st.o[m][1] *= ah; st.o[m][2] *= al; st.o[m][3] *= ah; }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {            // keys 16h .. 16h+15: one k-step of P.V
        uint4 vv[4][NC];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int kr = 16 * h + 2 * t + (r & 1) + (r >> 1) * 8;
#pragma unroll
            for (int c = 0; c < NC; ++c)
                vv[r][c] = kr < nvalid ? attn_row8<KV8>(sV + kr * ROWB, c * 8 + g) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int ep = 0; ep < 4; ++ep) {
                const uint32_t wA = u4c(vv[0][c], ep), wB = u4c(vv[1][c], ep), wC = u4c(vv[2][c], ep), wD = u4c(vv[3][c], ep);
                mma16816(st.o[c * 4 + ep], prmt(wA, wB, 0x5410), prmt(wA, wB, 0x7632), prmt(wC, wD, 0x5410), prmt(wC, wD, 0x7632), pb[2 * h], pb[2 * h + 1]);
            }
    }
}

// Spill a warp's state to shared memory for the merge of the CTA's warps: o_w [kMaxGroup][HD], ml_w [kMaxGroup][2].
template <int HD>
__device__ __forceinline__ void attn_state_to_smem(AttnState<HD>& st, float* o_w, float* ml_w, int g, int t) {
    constexpr int NC = HD / 64;
    st.l_run += __shfl_xor_sync(0xffffffffu, st.l_run, 1);
    st.l_run += __shfl_xor_sync(0xffffffffu, st.l_run, 2);
    if (t == 0) { ml_w[g * 2] = st.m_run; ml_w[g * 2 + 1] = st.l_run; }
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int ep = 0; ep < 4; ++ep) {
            const int d = (c * 8 + g) * 8 + 2 * ep, m = c * 4 + ep;
            o_w[(2 * t) * HD + d] = st.o[m][0]; o_w[(2 * t + 1) * HD + d] = st.o[m][1];
            o_w[(2 * t) * HD + d + 1] = st.o[m][2]; o_w[(2 * t + 1) * HD + d + 1] = st.o[m][3];
        }
}

// Merge nw warp states (o_all [nw][kMaxGroup][HD], ml_all [nw][kMaxGroup][2]; a warp that saw no key has m = -inf,
// l = 0) into one partial slot.  Called by `nthreads` threads, `tid` in [0, nthreads).
template <int HD>
__device__ __forceinline__ void attn_merge_warps(const float* o_all, const float* ml_all, int nw, int grp, float* po, float* pml, int tid, int nthreads) {
    for (int idx = tid; idx < grp * HD; idx += nthreads) {
        const int h = idx / HD, d = idx % HD;
        float M = -INFINITY;
        for (int w = 0; w < nw; ++w) M = fmaxf(M, ml_all[(w * kMaxGroup + h) * 2]);
        float acc = 0.f, L = 0.f;
        for (int w = 0; w < nw; ++w) {
            const float mw = ml_all[(w * kMaxGroup + h) * 2];
            const float f = mw == -INFINITY ? 0.f : ex2(mw - M);
            acc += o_all[((size_t)w * kMaxGroup + h) * HD + d] * f;
            L += ml_all[(w * kMaxGroup + h) * 2 + 1] * f;
        }
        po[h * HD + d] = acc;
        if (d == 0) { pml[h * 2] = M; pml[h * 2 + 1] = L; }
    }
}

}  // namespace cq
