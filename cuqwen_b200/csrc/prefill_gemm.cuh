// Batched-token ("prefill") GEMM on the fifth-generation tensor cores:  Y[T][R] = X[T][K] * W[R][K]^T  for a tile of
// prompt tokens at once, W in the model file's own format (int4 / int8 with one fp16 scale per row and 128 columns,
// or fp16).  The reference has no such path: it prefills one token at a time through the decode kernels
// (src/main.cu:86-92; its roadmap names the batched form, README.md:145).
//
// One CTA computes a 256-token x NT-row tile as two 128-token halves (one half when the launch has at most 128
// tokens); NT = 256 weight rows, or 128 / 64 where 256-row tiles would leave most SMs without a CTA.  UMMA shape
// M = 128 (tokens) x N = NT x K = 16, fp16 operands from shared memory in the K-major 128-byte-swizzled canonical
// layout, one fp32 accumulator of NT tensor-memory columns per half: the widened weight tile, which costs the CUDA
// cores more than one half's MMAs cost the tensor core, is used twice.  Per 64-column K block:
//   warp 0     one lane issues the TMA copies into a ring of three or four slots: the X tiles (128 x 64 fp16,
//              hardware-swizzled) and the raw weight rows
//   warps 2-9  quantised weights: a row (or a half / quarter of one) per thread, fp16(q) * scale into the swizzled B
//              tile, a ring of two slots (fp16 weights arrive swizzled by TMA and skip this)
//   warp 1     one lane issues four tcgen05.mma (K = 16 each) per half and commits the slots back to their fillers
// After the last K block warps 2-9 read the accumulators (tcgen05.ld, warp w owns TMEM lanes 32 * (w % 4) ..) and
// apply the epilogue.  Every mbarrier wait is bounded (tma.cuh); a wait that runs out sets *err and the CTA drains.
#pragma once
#include "tma.cuh"

namespace cq {

constexpr int kPfM = 128;            // tokens per tile
constexpr int kPfN = 256;            // weight rows per tile at the most (two matrices of half as many rows each in the SwiGLU mode)
constexpr int kPfKB = 64;            // K per pipeline stage: 128 bytes of fp16, one swizzle row
constexpr int kPfMH = 2;             // token tiles per CTA: two accumulators share every widened weight tile
constexpr int kPfConvWarps = 8;      // 8: a weight row of a K block per thread; 16: half a row (measured: no faster, the kernel is bound elsewhere)
constexpr int kPfThreads = (2 + kPfConvWarps) * 32;
constexpr int kPfABytes = kPfM * 128;          // one X tile of a stage
// Shared memory: a ring of NA slots that TMA fills (kPfMH X tiles + the raw weight rows of a K block: int4 32, int8 64
// bytes a row) and a ring of NB slots for the fp16 B tile.  The raw data and the X tiles have a TMA round trip to
// cover, so their ring is the deep one; a widened B tile is consumed by the very next MMAs, two slots suffice.
// fp16 weights have no raw form: their B tile arrives by TMA, NB = NA.
__host__ __device__ constexpr int pf_raw_bytes(int quant, int nt) { return quant == 2 ? nt * 32 : quant == 1 ? nt * 64 : 0; }
__host__ __device__ constexpr int pf_na(int quant) { return quant == 2 ? 4 : 3; }
__host__ __device__ constexpr int pf_nb(int quant) { return quant == 0 ? 3 : 2; }
__host__ __device__ constexpr int pf_smem_bytes(int quant, int nt) {
    return pf_na(quant) * (kPfMH * kPfABytes + pf_raw_bytes(quant, nt)) + pf_nb(quant) * nt * 128 + 1024 /* alignment slack */ + 256 /* barriers, TMEM address */;
}

enum PfMode : int {
    PF_OUT_F16 = 0,     // out_h[t][r] = half(acc + bias[r])
    PF_OUT_F32 = 1,     // out_f[t][r] = acc
    PF_RESID = 2,       // out_h[t][r] = half(float(out_h[t][r]) + acc)          (reference src/kernels.cu:670-671)
    PF_SWIGLU = 3       // out_h[t][r] = half(silu(acc_gate) * acc_up), fast-math exp / divide (src/kernels.cu:565-567)
};

struct PfGemmArgs {
    CUtensorMap tx;            // X as [T][K] fp16, box 64 x 128, 128-byte swizzle
    CUtensorMap tw[3];         // weights: bytes [rows][row bytes], box (raw bytes of a K block) x rows; fp16: box 64 x rows, swizzled
    const __half* s[3];        // scales [rows][K / 128] (quantised formats)
    // Plain modes: up to three matrices over the same X side by side in one launch (q, k and v: 16-CTA launches of
    // their own would leave most of the GPU idle); matrix i owns ceil(seg_rows[i] / NT) row tiles and the output
    // columns after those of the matrices before it.  PF_SWIGLU: tw[0] / tw[1] are gate and up, nseg = 1.
    int seg_rows[3];
    int nseg;
    const __half* bias;        // PF_OUT_F16, may be null
    __half* out_h;
    float* out_f;
    int T, R, K, ldo;          // R: rows of all matrices together; ldo: elements between consecutive tokens of the output
    int mode;
    int mh;                    // token halves per CTA (1 or 2), set by the launcher
    unsigned* err;
};

// Fills the tensor maps and launches.  PF_SWIGLU: w = {gate, up}, nmat = 2, rows[0] = rows of each.  Other modes: nmat
// matrices of rows[i] rows each, outputs side by side; a.s[i] hold their scales.
int launch_prefill_gemm(int quant, PfGemmArgs& a, const void* x, const void* const* w, const int* rows, int nmat, cudaStream_t stream);

}  // namespace cq
