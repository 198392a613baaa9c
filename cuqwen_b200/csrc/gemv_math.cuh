// Inner arithmetic of the GEMV family: how one 128-column group of a 16-row tile is multiplied with the activation
// vector, and how the activation vector is prepared in shared memory for it.
//
// Quantised weights (int4 / int8) run on the integer tensor-core path, exactly:
//   * per 128-column group the fp16 activations are rewritten as integers X_k = rint(x_k * 2^e) with e chosen from the
//     group's largest magnitude so that |X_k| < 2^14, and split into two signed byte digits X = d0 + 256*d1;
//   * mma.sync.m16n8k32 (u8 x s8 for int4 stored as q+8, s8 x s8 for int8) forms sum q*d0 and sum q*d1 in int32 in
//     columns 0 and 1 of the accumulator - the other six columns of the B operand are zero;
//   * sum q*X = C0 + 256*C1 - 8*sum(X) (the last term only for int4) is exact integer arithmetic; it is converted to
//     fp32 once per group and scaled by scale_group * 2^-e, then accumulated in fp32 across groups.
// The only departure from "fp32 sum of float(q)*float(x)" (reference src/kernels.cu:27-41) is the rounding of x to the
// group's 15-bit integer grid: an absolute error below 2^-15 of the group's largest |x| per element, i.e. 16 times
// finer than the fp16 spacing of that largest element.
// fp16 weights use mma.sync.m16n8k16 with fp32 accumulation; x stays fp16 in shared memory.
#pragma once
#include "tma.cuh"

namespace cq {

constexpr int kChunkBytes = 64;   // a staged box is chunk-major: [64-byte chunk][row][64 bytes] (see make_weight_map)

template <int Q> struct QT;
template <> struct QT<Q_I4> { static constexpr int NI = 1, GB = 64; };    // 16-byte loads per row-group per lane, bytes per row-group
template <> struct QT<Q_I8> { static constexpr int NI = 2, GB = 128; };
template <> struct QT<Q_F16> { static constexpr int NI = 4, GB = 256; };

// D(16x8,s32) += A(16x32, 8-bit, row) * B(32x8, s8, col).  Lane = 4g+t:
//   a0:(row g, k 4t..4t+3) a1:(row g+8, same k) a2:(row g, k 16+4t..) a3:(row g+8, k 16+4t..)
//   b0:(k 4t..4t+3, col g) b1:(k 16+4t.., col g)     c0,c1:(row g, col 2t,2t+1) c2,c3:(row g+8, ...)
__device__ __forceinline__ void imma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same with a zero accumulator on input (the first MMA of a chain): no registers need clearing beforehand.
__device__ __forceinline__ void imma_u8s8_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_s8s8_z(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// four packed nibbles -> four bytes holding q+8: (v & 0x0f0f0f0f) ^ 0x08080808 in one LOP3
__device__ __forceinline__ uint32_t nib4(uint32_t v) { return and_xor(v, 0x0f0f0f0fu, 0x08080808u); }

// Integer path, one 128-column group for the MT tiles of a warp, in two halves so that a caller can put the loads of
// a group in flight before the first MMA.  wbase: shared address of this lane's 16 bytes (column t) of row g of tile 0
// in the group's first chunk; the group's next chunk is cstride bytes further, tile m mstride bytes.  The B operand is
// the group's digit block, laid out [half (2)][t (4)][digit plane (2)][16 bytes]; lanes with g >= 2 feed zero columns.
// Two accumulator sets per tile alternate to shorten the dependent chain.
// load_group_w fetches the fragments, mma_group_int consumes them (c need not be cleared: it is overwritten).
template <int Q, int MT>
__device__ __forceinline__ void load_group_w(uint32_t wbase, int cstride, int mstride, uint4 (&w)[MT][2][QT<Q>::NI]) {
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < QT<Q>::NI; ++i) w[m][h][i] = lds128(wbase + m * mstride + h * 8 * kChunkBytes + i * cstride);
}
template <int Q, int MT>
__device__ __forceinline__ void mma_group_int(const uint4 (&w)[MT][2][QT<Q>::NI], const uint4 (&xv)[2], int (&c)[MT][2][4]) {
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (Q == Q_I4) {
                const uint32_t a0 = u4c(w[m][0][0], 2 * jj), b0 = u4c(w[m][1][0], 2 * jj);
                const uint32_t a1 = u4c(w[m][0][0], 2 * jj + 1), b1 = u4c(w[m][1][0], 2 * jj + 1);
                if (jj == 0) {      // first MMA of each accumulator chain: c comes in undefined and leaves initialised
                    imma_u8s8_z(c[m][0], nib4(a0), nib4(b0), nib4(a0 >> 4), nib4(b0 >> 4), xv[jj].x, xv[jj].y);
                    imma_u8s8_z(c[m][1], nib4(a1), nib4(b1), nib4(a1 >> 4), nib4(b1 >> 4), xv[jj].z, xv[jj].w);
                } else {
                    imma_u8s8(c[m][0], nib4(a0), nib4(b0), nib4(a0 >> 4), nib4(b0 >> 4), xv[jj].x, xv[jj].y);
                    imma_u8s8(c[m][1], nib4(a1), nib4(b1), nib4(a1 >> 4), nib4(b1 >> 4), xv[jj].z, xv[jj].w);
                }
            } else {
                const uint4& a = w[m][0][jj < QT<Q>::NI ? jj : 0];
                const uint4& b = w[m][1][jj < QT<Q>::NI ? jj : 0];
                if (jj == 0) {
                    imma_s8s8_z(c[m][0], a.x, b.x, a.y, b.y, xv[jj].x, xv[jj].y);
                    imma_s8s8_z(c[m][1], a.z, b.z, a.w, b.w, xv[jj].z, xv[jj].w);
                } else {
                    imma_s8s8(c[m][0], a.x, b.x, a.y, b.y, xv[jj].x, xv[jj].y);
                    imma_s8s8(c[m][1], a.z, b.z, a.w, b.w, xv[jj].z, xv[jj].w);
                }
            }
        }
    }
}
// The B operand of a group: the two halves of its digit block (lanes with g >= 2 feed zero columns).
__device__ __forceinline__ void load_group_x(uint32_t xd, int g, int t, uint4 (&xv)[2]) {
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
        xv[jj] = make_uint4(0u, 0u, 0u, 0u);
        if (g < 2) xv[jj] = lds128(xd + jj * 128 + t * 32 + g * 16);
    }
}

// fp16-weight path: x fp16 in natural order (xg = the group's 16 uint4), fp32 accumulators.
template <int MT>
__device__ __forceinline__ void compute_group_f16(uint32_t wbase, int cstride, int mstride, int t, const uint4* __restrict__ xg, float (&c)[MT][2][4]) {
    uint4 w[MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) w[m][h][i] = lds128(wbase + m * mstride + h * 8 * kChunkBytes + i * cstride);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 xv = xg[i * 4 + t];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint4& a = w[m][0][i];
            const uint4& b = w[m][1][i];
            mma16816(c[m][0], a.x, b.x, a.y, b.y, xv.x, xv.y);
            mma16816(c[m][1], a.z, b.z, a.w, b.w, xv.z, xv.w);
        }
    }
}

}  // namespace cq
