// Batched-token ("prefill") GEMM on the fifth-generation tensor cores:  Y[T][R] = X[T][K] * W[R][K]^T  for a tile of
// prompt tokens at once, W in the model file's own format (int4 / int8 with one fp16 scale per row and 128 columns,
// or fp16).  The reference has no such path: it prefills one token at a time through the decode kernels
// (src/main.cu:86-92; its roadmap names the batched form, README.md:145).
//
// One CTA computes a 128-token x 256-row tile.  UMMA shape M = 128 (tokens) x N = 256 (weight rows) x K = 16, fp16
// operands from shared memory in the K-major 128-byte-swizzled canonical layout, fp32 accumulator in tensor memory
// (256 columns).  Per 64-column K block:
//   warp 0     one lane issues the TMA copies: the X tile (128 x 64 fp16, hardware-swizzled) and the raw weight rows
//   warps 2-9  quantised weights: one row per thread, 64 weights -> fp16 * scale -> the swizzled B tile
//              (fp16 weights arrive swizzled by TMA and skip this)
//   warp 1     one lane issues four tcgen05.mma (K = 16 each) and commits the stage back to the producer
// After the last K block warps 2-9 read the accumulator (tcgen05.ld, warp w owns TMEM lanes 32 * (w % 4) ..) and apply
// the epilogue.  Every mbarrier wait is bounded (tma.cuh); a wait that runs out sets *err and the CTA drains.
#pragma once
#include "tma.cuh"

namespace cq {

constexpr int kPfM = 128;            // tokens per tile
constexpr int kPfN = 256;            // weight rows per tile (two matrices of 128 rows each in the SwiGLU mode)
constexpr int kPfKB = 64;            // K per pipeline stage: 128 bytes of fp16, one swizzle row
constexpr int kPfStages = 3;
constexpr int kPfConvWarps = 8;
constexpr int kPfThreads = (2 + kPfConvWarps) * 32;
constexpr int kPfABytes = kPfM * 128;          // X tile of a stage
constexpr int kPfBBytes = kPfN * 128;          // B tile of a stage
constexpr int kPfRawBytes = kPfN * 64;         // raw weight rows of a stage (int8: 64 bytes a row; int4 uses half)
constexpr int kPfStageBytes = kPfABytes + kPfBBytes + kPfRawBytes;
constexpr int kPfSmemBytes = kPfStages * kPfStageBytes + 1024 /* alignment slack */ + 256 /* barriers, TMEM address */;

enum PfMode : int {
    PF_OUT_F16 = 0,     // out_h[t][r] = half(acc + bias[r])
    PF_OUT_F32 = 1,     // out_f[t][r] = acc
    PF_RESID = 2,       // out_h[t][r] = half(float(out_h[t][r]) + acc)          (reference src/kernels.cu:670-671)
    PF_SWIGLU = 3       // out_h[t][r] = half(silu(acc_gate) * acc_up), fast-math exp / divide (src/kernels.cu:565-567)
};

struct PfGemmArgs {
    CUtensorMap tx;            // X as [T][K] fp16, box 64 x 128, 128-byte swizzle
    CUtensorMap tw[2];         // weights: bytes [R][row bytes], box (raw bytes of a K block) x rows; fp16: box 64 x rows, swizzled
    const __half* s[2];        // scales [R][K / 128] (quantised formats)
    const __half* bias;        // PF_OUT_F16, may be null
    __half* out_h;
    float* out_f;
    int T, R, K, ldo;          // ldo: elements between consecutive tokens of the output
    int mode;
    unsigned* err;
};

int launch_prefill_gemm(int quant, PfGemmArgs& a, const void* x, const void* w0, const void* w1, cudaStream_t stream);

}  // namespace cq
