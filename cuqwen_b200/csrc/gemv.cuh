// Weight-streaming GEMV family for batch-1 decode on sm_100a: argument block, shared-memory layout, tile addressing
// and epilogues.  The kernel itself is in gemv_kernel.cuh, its arithmetic in gemv_math.cuh / gemv_stage.cuh.
//
// y[r] = sum_k W[r,k] * x[k], W row-major fp16 / int8 / packed int4 with one fp16 scale per 128 input columns (the
// on-disk layout of the reference, export_weights.py:123-205).  The reference computes, per 8-wide chunk,
// "p = sum float(q)*float(x); acc += p*scale" (src/kernels.cu:11-57).
//
// Data path.  A producer warp issues TMA tile copies (cp.async.bulk.tensor.3d: boxes of 16*rw rows x up to 256 bytes
// of the row-major weight matrix, delivered chunk-major) into a CTA-wide ring of shared-memory stages; each box signals
// an mbarrier, so the HBM stream is decoupled from the register file and the scoreboards.  Rows past the end of the
// matrix are zero-filled by the TMA unit.  Eight consumer warps, each owning 16 output rows (x MT matrices) of a block
// and a share of K, read their fragments from the stages and run the tensor-core inner product of gemv_math.cuh.
//
// Every wait on an mbarrier is bounded (4e9 SM cycles, two to four seconds); when it expires the kernel records a code
// in *err, stops waiting and finishes with meaningless numbers rather than hanging.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace cq {

enum Epi : int { EPI_F16 = 0, EPI_F32 = 1, EPI_RESID = 2, EPI_SWIGLU = 3, EPI_QKV = 4, EPI_PUSH = 5 };

struct alignas(64) GemvArgs {
    CUtensorMap tmap[3];      // one 3-D byte map per weight matrix: dims {64, rows, row bytes / 64}, box {64, 16*rw, piece bytes / 64}
    const uint8_t* w[3];      // matrices: [0] generic / gate / q, [1] up / k, [2] v
    const __half* s[3];       // their group scales (null for fp16 weights)
    const __half* x;          // input vector [K]
    const __half* norm_w;     // non-null: x is RMS-normalised with this weight in the prologue
    float eps;
    int K;                    // input columns, multiple of 128
    int rows;                 // output rows of one matrix (QKV: unused)
    int nsets;                // EPI_QKV: number of 16-row tile sets (one per block)
    int brows, nblk;          // rows of a CTA block (at most 16 * rw; the last block may be shorter) and number of blocks
    int rw, kw;               // the consumer warps form rw row-warps x kw K-parts x gw group-parts: a CTA block is up to rw 16-row tiles, each split kw ways along K
    int gw;                   // warps that share one (row-warp, K-part) cell: they take the 128-column groups of a staged piece in turn
    int pg;                   // 128-column groups per staged row piece
    int nst;                  // stages in the CTA's ring
    int nsb;                  // scale blocks in shared memory: 2 (the next block's scales arrive while this one computes) or 1 when no CTA has a second block
    unsigned* err;            // device word that receives a non-zero code when a bounded wait expires (may be null)
    __half* out_h;            // EPI_F16 / EPI_RESID (in-out) / EPI_SWIGLU
    float* out_f;             // EPI_F32
    // EPI_QKV
    const __half* bias[3];
    __half *q_out, *k_out, *v_out;
    __half *kcache, *vcache;  // this layer's [n_kv][max_seq][hd] caches, may be null
    const int* d_pos;
    int n_heads, n_kv, hd, max_seq;
    float theta;
    int rope_fast;
    // Tensor-parallel exchange of a row-parallel matrix (o_proj, down): no collective call, no fence, no flag word.
    // EPI_PUSH stores each fp32 partial output, paired with the exchange's sequence number in one 8-byte word, straight
    // into every rank's receive slot over NVLink peer stores.  The kernel that consumes the vector next (always a GEMV
    // with fused RMSNorm) reads the words until every one carries the expected sequence number and forms
    // x_next = half(float(x) + sum_r partial_r) while it stages x ("gather").  A word travels as one 64-bit scalar
    // store and is read as one 64-bit element, so it is either old (wrong number) or complete.  Reference: single-GPU only; the sum replaces
    // src/kernels.cu:670-671 / :620-621 across ranks.
    uint2* push[8];                // EPI_PUSH: start of this rank's slot inside rank d's receive buffer, {value bits, sequence}
    int npush;
    int ngather;                   // consumer: number of slots to add to x (0 = plain x)
    const uint2* gather;           // this rank's receive slots, [ngather][K] words
    __half* x_next;                // where CTA 0 stores the summed vector (never the buffer x points at)
    const int* step_no;            // sequence number of an exchange = *step_no * kSeqPerStep + seq_index + 1
    int seq_index;
    long long wait_cycles;         // bound of the gather's re-read loop in SM cycles (0 = kWaitCyclesDefault)
    // Hand-over of an activation vector in staged form.  A SwiGLU kernel whose blocks are whole 128-row groups (rw = 8,
    // no K split) also writes its outputs as the digit blocks, corrections and scales that a quantised GEMV's inner loop
    // reads (gemv_stage.cuh), once; the GEMV that consumes the vector then fetches them with three bulk copies
    // instead of converting the whole vector again in every one of its CTAs.
    unsigned char* xd_out; int* corr_out; float* xscale_out;                 // producer side (EPI_SWIGLU), may be null
    const unsigned char* xd_in; const int* corr_in; const float* xscale_in;  // consumer side, may be null
    // Small read-only tensors that the NEXT kernels of the step will want at once (RMSNorm weight, biases): the producer
    // warp asks L2 for them while this kernel streams, so that their first use is an L2 hit instead of an HBM miss.
    const void* warm[3];
    int warm_bytes[3];
    unsigned long long* trace;     // optional: this launch's eight timeline words (tma.cuh), else null
};

template <int EPI> struct EpiMT { static constexpr int MT = (EPI == EPI_SWIGLU || EPI == EPI_QKV) ? 2 : 1; };

// Shared-memory carve-up, computed the same way by the host (for the launch size) and the kernel.
//   [x: K*2 bytes (fp16 vector, or the two digit planes)] [per-group corr (int) and xscale (float)] [reduction buffer]
//   [1 or 2 scale blocks] [ring of stages] [mbarriers]
// A stage holds, for each K-part kp and tile m, one TMA box of (16*rw rows) x piece_bytes, chunk-major:
// [kp][m][64-byte chunk][row][64 bytes].
constexpr int kConsumerWarps = 8;
struct GemvLayout {
    int piece_bytes, box_rows, box_bytes, box_stride, stage_bytes, scale_block_bytes;
    int off_corr, off_xscale, off_red, off_scales, off_stages, off_bars, total;
};
__host__ __device__ inline GemvLayout gemv_layout(int K, int group_bytes, int MT, int box_rows, int kw, int pg, int nst, bool quantised, int nsb) {
    GemvLayout L;
    const int ng = K / kGroup;
    L.piece_bytes = pg * group_bytes;
    L.box_rows = box_rows;
    L.box_bytes = L.box_rows * L.piece_bytes;
    L.box_stride = (L.box_bytes + 127) / 128 * 128;     // a TMA destination is 128-byte aligned; an odd row count times an odd chunk count is not
    L.stage_bytes = kw * MT * L.box_stride;
    L.scale_block_bytes = quantised ? MT * L.box_rows * ng * 2 : 0;
    // x (fp16 or digits).  Vectors of up to 6144 values are staged from registers (stage_x_regs); longer ones up to
    // 8192 get room for the RMSNorm weight beside them while x is staged.
    int o = K <= 6144 ? K * 2 : K <= 8192 ? K * 4 : K * 2;
    L.off_corr = o; o += (ng * 4 + 15) / 16 * 16;
    L.off_xscale = o; o += (ng * 4 + 15) / 16 * 16;
    L.off_red = o; o += kConsumerWarps * 32 * 4 + 16;
    o = (o + 127) / 128 * 128;
    L.off_scales = o; o += nsb * L.scale_block_bytes;
    o = (o + 127) / 128 * 128;               // TMA destinations are 128-byte aligned
    L.off_stages = o; o += nst * L.stage_bytes;
    L.off_bars = o; o += (2 * nst + 5) * 8;  // full[nst], empty[nst], scale full[2], scale empty[2], x staged[1]
    o += 1024;                               // a block whose row count is not a multiple of 16 lets the last tile's fragment loads run
                                             // up to 15 rows (960 bytes) past the last box of the last stage: they must stay inside the allocation
    L.total = o;
    return L;
}
inline size_t gemv_smem_bytes(int K, int quant, int MT, int box_rows, int kw, int pg, int nst, int nsb) {
    const int gb = quant == Q_I4 ? 64 : quant == Q_I8 ? 128 : 256;
    return (size_t)gemv_layout(K, gb, MT, box_rows, kw, pg, nst, quant != Q_F16, nsb).total;
}

// Where the 16 x MT rows of tile `rwi` of block `blk` live.  mrow[m] / mmat[m]: first row of tile m inside matrix
// mmat[m]; row0: first output row (generic) or the row inside its q / k / v matrix (QKV); row_end: one past the last
// row this tile may write (the block's and the matrix's end; row0 >= row_end = nothing to do).
// Generic: block blk covers rows [blk * brows, blk * brows + brows), tile rwi the sixteen rows from row0 on.
template <int EPI>
struct TileMap {
    int mrow[EpiMT<EPI>::MT];
    int mmat[EpiMT<EPI>::MT];
    const __half* sbase[EpiMT<EPI>::MT];
    int row0, mat, row_end;
};
template <int EPI>
__device__ __forceinline__ TileMap<EPI> map_tile(const GemvArgs& a, int blk, int rwi) {
    constexpr int MT = EpiMT<EPI>::MT;
    const int ng = a.K / kGroup;
    TileMap<EPI> m;
    if (EPI == EPI_QKV) {
        const int ts = blk;                     // one tile set per block
        const int spt = a.hd / 32;              // tile sets per head: rows i and i + hd/2 of a head travel together (RoPE pairs)
        const int hh = ts / spt, sub = ts % spt;
        const int mat = hh < a.n_heads ? 0 : hh < a.n_heads + a.n_kv ? 1 : 2;
        const int lh = mat == 0 ? hh : mat == 1 ? hh - a.n_heads : hh - a.n_heads - a.n_kv;
        m.row0 = lh * a.hd + sub * 16; m.mat = mat; m.row_end = m.row0 + 16;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int row = m.row0 + mt * (a.hd / 2);
            m.mrow[mt] = row; m.mmat[mt] = mat;
            m.sbase[mt] = a.s[mat] ? a.s[mat] + (size_t)row * ng : nullptr;
        }
    } else {
        const int b0 = blk * a.brows;
        m.row0 = b0 + rwi * 16; m.mat = 0;
        m.row_end = b0 + a.brows < a.rows ? b0 + a.brows : a.rows;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            m.mrow[mt] = b0; m.mmat[mt] = mt;                   // the TMA box and the scale block start at the block's first row
            m.sbase[mt] = a.s[mt] ? a.s[mt] + (size_t)b0 * ng : nullptr;
        }
    }
    return m;
}

// Operands of the epilogue that come from global memory (the residual value, the biases).  Fetched at the start of a
// block so that their latency hides behind the block's arithmetic.  The residual is read through L2: inside a
// multi-matrix kernel another SM wrote it and L1 may hold an older copy.
template <int EPI>
__device__ __forceinline__ void epilogue_fetch(const GemvArgs& a, int row0, int row_end, int mat, int r, float (&pre)[2]) {
    pre[0] = pre[1] = 0.f;
    if (EPI == EPI_RESID) {
        const int row = row0 + r;
        if (row < row_end) pre[0] = __half2float(__ldcg(a.out_h + row));
    } else if (EPI == EPI_QKV) {
        const int ra = row0 + r;
        pre[0] = __half2float(a.bias[mat][ra]);
        pre[1] = __half2float(a.bias[mat][ra + a.hd / 2]);
    } else if (EPI == EPI_PUSH) {
        pre[1] = __uint_as_float((unsigned)(*a.step_no) * kSeqPerStep + (unsigned)a.seq_index + 1u);     // the exchange's sequence number, as bits
    }
}

// Finish one output row (pair).  r = row slot 0..15 inside the tile set; pre = what epilogue_fetch returned for it.
template <int EPI>
__device__ __forceinline__ void epilogue(const GemvArgs& a, int row0, int row_end, int mat, int r, float v0, float v1, const float (&pre)[2], __half* hbuf = nullptr) {
    if (EPI == EPI_F16) {
        const int row = row0 + r;
        if (row < row_end) a.out_h[row] = __float2half(v0);
    } else if (EPI == EPI_F32) {
        const int row = row0 + r;
        if (row < row_end) a.out_f[row] = v0;
    } else if (EPI == EPI_PUSH) {
        const int row = row0 + r;
        if (row < row_end) {
            const unsigned vb = __float_as_uint(v0), seq = __float_as_uint(pre[1]);
            for (int d = 0; d < a.npush; ++d) st_pair(a.push[d] + row, vb, seq);      // peer stores (one of them local), value and number in one 64-bit word
        }
    } else if (EPI == EPI_RESID) {
        // reference src/kernels.cu:670-671 and :620-621
        const int row = row0 + r;
        if (row < row_end) a.out_h[row] = __float2half(pre[0] + v0);
    } else if (EPI == EPI_SWIGLU) {
        // reference src/kernels.cu:565-567 (fast-math exp and divide, as that build uses)
        const int row = row0 + r;
        if (row < row_end) {
            const float sig = __fdividef(1.0f, 1.0f + __expf(-v0));
            const __half h = __float2half(v0 * sig * v1);
            a.out_h[row] = h;
            if (hbuf) hbuf[r] = h;              // the block's 128 outputs meet in shared memory for the digit hand-over
        }
    } else {
        // bias in fp32, one rounding to fp16 (src/kernels.cu:468-472); rotate-half RoPE on q and k from the rounded
        // values (src/kernels.cu:370-398); k and v also go to the cache row `pos` (src/kernels.cu:326-347).
        const int half_hd = a.hd / 2;
        const int ra = row0 + r, rb2 = ra + half_hd;
        const float f0 = __half2float(__float2half(v0 + pre[0]));
        const float f1 = __half2float(__float2half(v1 + pre[1]));
        __half o0, o1;
        const int pos = *a.d_pos;
        if (mat < 2) {
            float c, s;
            rope_cs(ra % a.hd, a.hd, pos, a.theta, a.rope_fast, &c, &s);
            o0 = __float2half(f0 * c - f1 * s);
            o1 = __float2half(f1 * c + f0 * s);
        } else {
            o0 = __float2half(f0); o1 = __float2half(f1);
        }
        __half* dst = mat == 0 ? a.q_out : mat == 1 ? a.k_out : a.v_out;
        if (dst) { dst[ra] = o0; dst[rb2] = o1; }
        __half* cache = mat == 1 ? a.kcache : mat == 2 ? a.vcache : nullptr;
        if (cache) {
            const int head = ra / a.hd, d = ra % a.hd;
            const size_t base = ((size_t)head * a.max_seq + pos) * a.hd;
            cache[base + d] = o0; cache[base + d + half_hd] = o1;
        }
    }
}

}  // namespace cq
