/*
 * CPU oracle for the CuQwen batch-1 decode step.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain scalar C, the arithmetic of the reference
 * engine's decode hot path (CuQwen: src/kernels.cu, src/model.cu,
 * src/load_weights.cpp, export_weights.py).  It is the checker for the CUDA
 * kernels of this repository and the timed "port" CPU baseline.  It is never
 * part of the product path: only tests, the smoke check and the benchmark's
 * cpu-baseline leg may load it.
 *
 * Parity pinning: the reference ships no tests, golden vectors or CPU path.
 * The oracle is pinned two ways: (1) the weight-format / quantisation half is
 * checked against fixtures produced by importing the reference's own
 * export_weights.py; (2) the arithmetic half is checked against outputs of the
 * reference's CUDA kernels (launch_*) captured on a B200 and committed as
 * fixtures under tests/golden/.  Where (2) is absent for an op the op is
 * "parity unpinned".
 *
 * Conventions: fp16 values travel as uint16_t bit patterns; every rounding to
 * fp16 happens exactly where the reference rounds (cited per function).
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_GROUP 128          /* include/config.h:16 QUANT_GROUP_SIZE */
#define ORC_MAGIC 0x5157454E   /* include/config.h:53 */
#define ORC_REF_PARTS 64       /* include/config.h:146 ATTN_PARTITIONS */

typedef uint16_t h16;

static inline float h2f(h16 h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline h16 f2h(float f) { _Float16 v = (_Float16)f; h16 h; memcpy(&h, &v, 2); return h; }

float orc_h2f(h16 h) { return h2f(h); }
h16 orc_f2h(float f) { return f2h(f); }
int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------- */
/* Weight decode (src/kernels.cu:27-42 INT4, :12-25 INT8)                     */
/* ------------------------------------------------------------------------- */

/* INT4: byte k of a row holds element 2k in the low nibble and 2k+1 in the
 * high nibble, 4-bit two's complement: ((n ^ 8) - 8).  kernels.cu:35-37,
 * export_weights.py:198-199. */
static inline int nib_lo(uint8_t b) { return ((b & 0xF) ^ 0x8) - 0x8; }
static inline int nib_hi(uint8_t b) { return (((b >> 4) & 0xF) ^ 0x8) - 0x8; }

void orc_unpack_int4(const uint8_t* packed, long rows, long cols, int8_t* out) {
    for (long r = 0; r < rows; ++r)
        for (long p = 0; p < cols / 2; ++p) {
            uint8_t b = packed[r * (cols / 2) + p];
            out[r * cols + 2 * p] = (int8_t)nib_lo(b);
            out[r * cols + 2 * p + 1] = (int8_t)nib_hi(b);
        }
}

/* Dequantised fp16 value of one weight: half(float(q) * float(scale)); one
 * scale per 128 input columns (kernels.cu:31 "c >> 4" on 8-wide chunks). */
void orc_dequant(int quant, const void* w, const h16* scales, long rows, long cols, h16* out) {
    long ng = cols / ORC_GROUP;
    for (long r = 0; r < rows; ++r)
        for (long c = 0; c < cols; ++c) {
            int q;
            if (quant == 2) {
                uint8_t b = ((const uint8_t*)w)[r * (cols / 2) + c / 2];
                q = (c & 1) ? nib_hi(b) : nib_lo(b);
            } else {
                q = ((const int8_t*)w)[r * cols + c];
            }
            out[r * cols + c] = f2h((float)q * h2f(scales[r * ng + c / ORC_GROUP]));
        }
}

/* ------------------------------------------------------------------------- */
/* GEMV in the reference's accumulation order.                                */
/* One warp per row; lane L takes the 8-wide chunks c = L, L+32, ...          */
/* (kernels.cu:459-462); inside a chunk the fma chain runs hi-then-lo per     */
/* byte pair starting from p = 0 (kernels.cu:33-40); the chunk contributes    */
/* p * scale; the 32 lane sums are folded by the shfl_down tree               */
/* (kernels.cu:464-466).  `contract` = 1 models nvcc's default fused          */
/* multiply-add of "acc += p * s".                                            */
/* ------------------------------------------------------------------------- */
static float row_dot(int quant, const void* wrow, const h16* srow, const float* xf, long cols, int contract) {
    float lane[32];
    for (int i = 0; i < 32; ++i) lane[i] = 0.0f;
    long nchunk = cols / 8;
    for (long c = 0; c < nchunk; ++c) {
        const float* x = xf + 8 * c;
        float p = 0.0f;
        float* acc = &lane[c & 31];
        if (quant == 2) {
            const uint8_t* b = (const uint8_t*)wrow + 4 * c;
            for (int k = 0; k < 4; ++k)
                p = fmaf((float)nib_lo(b[k]), x[2 * k], fmaf((float)nib_hi(b[k]), x[2 * k + 1], p));
        } else if (quant == 1) {
            const int8_t* b = (const int8_t*)wrow + 8 * c;
            for (int k = 0; k < 4; ++k)
                p = fmaf((float)b[2 * k], x[2 * k], fmaf((float)b[2 * k + 1], x[2 * k + 1], p));
        } else {
            const h16* b = (const h16*)wrow + 8 * c;
            for (int k = 0; k < 4; ++k)
                p = fmaf(h2f(b[2 * k]), x[2 * k], fmaf(h2f(b[2 * k + 1]), x[2 * k + 1], p));
        }
        if (quant) {
            float s = h2f(srow[c >> 4]);
            if (contract) *acc = fmaf(p, s, *acc);
            else *acc = *acc + p * s;
        } else {
            *acc = *acc + p;
        }
    }
    for (int off = 16; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) lane[i] += lane[i + off];
    return lane[0];
}

static int g_contract = 1;
void orc_set_contract(int on) { g_contract = on; }

/* out_f32[r] = W[r,:] . x   (no rounding of the result) */
void orc_gemv_f32(int quant, const void* W, const h16* scales, const h16* x, long rows, long cols, float* out) {
    float* xf = (float*)malloc(sizeof(float) * cols);
    for (long i = 0; i < cols; ++i) xf[i] = h2f(x[i]);
    long rb = quant == 2 ? cols / 2 : quant == 1 ? cols : cols * 2;
    long ng = cols / ORC_GROUP;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        out[r] = row_dot(quant, (const uint8_t*)W + r * rb, scales ? scales + r * ng : NULL, xf, cols, g_contract);
    free(xf);
}

/* ------------------------------------------------------------------------- */
/* Element-wise ops                                                           */
/* ------------------------------------------------------------------------- */

/* kernels.cu:689-751.  eps arrives as fp16 (model.cu:96, kernels.cuh:137). */
void orc_rmsnorm(const h16* x, const h16* w, h16* out, long dim, h16 eps_h) {
    /* 256 threads, thread t sums the 8-wide vectors t, t+256, ...; then the
     * warp tree and the 8-warp tree of block_reduce_sum (kernels.cu:67-83). */
    float th[256];
    for (int t = 0; t < 256; ++t) th[t] = 0.0f;
    long nv = dim / 8;
    for (long i = 0; i < nv; ++i) {
        float* s = &th[i & 255];
        for (int k = 0; k < 4; ++k) {
            float f1 = h2f(x[8 * i + 2 * k]), f2 = h2f(x[8 * i + 2 * k + 1]);
            *s += fmaf(f1, f1, f2 * f2);
        }
    }
    for (long i = nv * 8; i < dim; ++i) { float v = h2f(x[i]); th[(i - nv * 8) & 255] += v * v; }
    float wsum[32];
    for (int wdx = 0; wdx < 32; ++wdx) wsum[wdx] = 0.0f;
    for (int wdx = 0; wdx < 8; ++wdx) {
        float* l = &th[32 * wdx];
        for (int off = 16; off > 0; off >>= 1)
            for (int i = 0; i < off; ++i) l[i] += l[i + off];
        wsum[wdx] = l[0];
    }
    for (int off = 16; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) wsum[i] += wsum[i + off];
    float inv = 1.0f / sqrtf(wsum[0] / (float)dim + h2f(eps_h));
    for (long i = 0; i < dim; ++i) out[i] = f2h(h2f(x[i]) * inv * h2f(w[i]));
}

/* kernels.cu:370-398.  Accurate libm transcendentals (the reference build uses
 * the GPU's fast-math approximations of the same formulas). */
void orc_rope(h16* q, h16* k, int n_heads, int n_kv, int hd, int pos, float theta) {
    int half_hd = hd / 2;
    for (int t = 0; t < (n_heads + n_kv) * half_hd; ++t) {
        int is_q = t < n_heads * half_hd;
        int lt = is_q ? t : t - n_heads * half_hd;
        int head = lt / half_hd, i = lt % half_hd;
        float freq = 1.0f / powf(theta, (2.0f * i) / (float)hd);
        float val = (float)pos * freq;
        float c = cosf(val), s = sinf(val);
        h16* buf = is_q ? q : k;
        int b = head * hd + i;
        float v0 = h2f(buf[b]), v1 = h2f(buf[b + half_hd]);
        buf[b] = f2h(v0 * c - v1 * s);
        buf[b + half_hd] = f2h(v1 * c + v0 * s);
    }
}

/* kernels.cu:402-474: q/k/v = half(W.xn + bias), bias added in fp32. */
void orc_qkv(int quant, const h16* xn, const void* Wq, const void* Wk, const void* Wv,
             const h16* Sq, const h16* Sk, const h16* Sv, const h16* bq, const h16* bk, const h16* bv,
             h16* q, h16* k, h16* v, long dim, long q_dim, long kv_dim) {
    float* t = (float*)malloc(sizeof(float) * (q_dim > kv_dim ? q_dim : kv_dim));
    orc_gemv_f32(quant, Wq, Sq, xn, q_dim, dim, t);
    for (long i = 0; i < q_dim; ++i) q[i] = f2h(t[i] + h2f(bq[i]));
    orc_gemv_f32(quant, Wk, Sk, xn, kv_dim, dim, t);
    for (long i = 0; i < kv_dim; ++i) k[i] = f2h(t[i] + h2f(bk[i]));
    orc_gemv_f32(quant, Wv, Sv, xn, kv_dim, dim, t);
    for (long i = 0; i < kv_dim; ++i) v[i] = f2h(t[i] + h2f(bv[i]));
    free(t);
}

/* kernels.cu:640-672 / :590-622: x[r] = half(float(x[r]) + W[r,:].in) */
void orc_gemv_add(int quant, const void* W, const h16* S, const h16* in, h16* x, long rows, long cols) {
    float* t = (float*)malloc(sizeof(float) * rows);
    orc_gemv_f32(quant, W, S, in, rows, cols, t);
    for (long i = 0; i < rows; ++i) x[i] = f2h(h2f(x[i]) + t[i]);
    free(t);
}

/* kernels.cu:523-569: h = half(g * sigmoid(g) * u), g and u kept in fp32. */
void orc_mlp1(int quant, const h16* xn, const void* Wg, const void* Wu, const h16* Sg, const h16* Su,
              h16* out, long dim, long inter) {
    float* g = (float*)malloc(sizeof(float) * inter * 2);
    float* u = g + inter;
    orc_gemv_f32(quant, Wg, Sg, xn, inter, dim, g);
    orc_gemv_f32(quant, Wu, Su, xn, inter, dim, u);
    for (long i = 0; i < inter; ++i) {
        float sig = 1.0f / (1.0f + expf(-g[i]));
        out[i] = f2h(g[i] * sig * u[i]);
    }
    free(g);
}

/* kernels.cu:772-806 (fp16) / :820-859 (int8): logits = half(W.xn) */
void orc_logits(int quant, const void* W, const h16* S, const h16* xn, h16* logits, long vocab, long dim) {
    float* t = (float*)malloc(sizeof(float) * vocab);
    orc_gemv_f32(quant, W, S, xn, vocab, dim, t);
    for (long i = 0; i < vocab; ++i) logits[i] = f2h(t[i]);
    free(t);
}

/* kernels.cu:873-891.  Only the first 4096 history entries are visited
 * (fixed 16x256 launch, kernels.cu:901-903).  The reference applies the
 * penalty once per occurrence with a data race on duplicates; this oracle
 * (and the CUDA path) apply it once per distinct id, which equals the
 * reference whenever the ids are distinct. */
void orc_penalty(h16* logits, const int* hist, int hist_len, int vocab, h16 pen_h) {
    int n = hist_len < 4096 ? hist_len : 4096;
    float pen = h2f(pen_h);
    for (int i = 0; i < n; ++i) {
        int id = hist[i];
        if (id < 0 || id >= vocab) continue;
        int seen = 0;
        for (int j = 0; j < i; ++j) if (hist[j] == id) { seen = 1; break; }
        if (seen) continue;
        float l = h2f(logits[id]);
        logits[id] = f2h(l < 0.0f ? l * pen : l / pen);
    }
}

/* kernels.cu:907-950: max of (orderkey(float(l)) << 32 | ~idx): ties go to the
 * lowest index; a NaN with sign bit 0 sorts above +inf. */
int orc_argmax(const h16* logits, int vocab) {
    uint64_t best = 0;
    for (int i = 0; i < vocab; ++i) {
        float v = h2f(logits[i]);
        uint32_t fu; memcpy(&fu, &v, 4);
        uint32_t key = (fu & 0x80000000u) ? ~fu : (fu | 0x80000000u);
        uint64_t p = ((uint64_t)key << 32) | (uint32_t)(~i);
        if (p > best) best = p;
    }
    return (int)(~((uint32_t)(best & 0xffffffffu)));
}

/* ------------------------------------------------------------------------- */
/* Attention.  K/V cache is head-major [n_kv][max_seq][hd] (model.cuh:25).    */
/* ------------------------------------------------------------------------- */

/* Exact form: softmax(q.K^T / sqrt(hd)) V with fp32 scores and double sums;
 * only the output is rounded to fp16.  (The un-fused statement of the same
 * math is cuda_optimizations/v1_cublas/src/kernels.cu:147-236.) */
void orc_attention_exact(const h16* q, const h16* K, const h16* V, h16* out,
                         int n_heads, int n_kv, int hd, long max_seq, int len) {
    int grp = n_heads / n_kv;
    float scale = 1.0f / sqrtf((float)hd);
#pragma omp parallel for schedule(static)
    for (int h = 0; h < n_heads; ++h) {
        const h16* Kh = K + (size_t)(h / grp) * max_seq * hd;
        const h16* Vh = V + (size_t)(h / grp) * max_seq * hd;
        float* s = (float*)malloc(sizeof(float) * len);
        double* o = (double*)calloc(hd, sizeof(double));
        float m = -INFINITY;
        for (int t = 0; t < len; ++t) {
            float a = 0.0f;
            for (int d = 0; d < hd; ++d) a = fmaf(h2f(q[h * hd + d]), h2f(Kh[(size_t)t * hd + d]), a);
            s[t] = a * scale;
            if (s[t] > m) m = s[t];
        }
        double l = 0.0;
        for (int t = 0; t < len; ++t) {
            double e = exp((double)s[t] - (double)m);
            l += e;
            for (int d = 0; d < hd; ++d) o[d] += e * (double)h2f(Vh[(size_t)t * hd + d]);
        }
        for (int d = 0; d < hd; ++d) out[h * hd + d] = f2h((float)(o[d] / l));
        free(s); free(o);
    }
}

/* Reference-faithful form: 64 fixed partitions (kernels.cu:143-147); score
 * rounded to fp16 (:171); e = exp(float(s) - m) summed in fp32 while P is
 * stored as half(e) (:184-186); O = sum P.V in fp32, un-normalised; stage 2
 * (:222-288) rescales by exp(m_s - M) and divides by (sum + 1e-9). */
void orc_attention_ref(const h16* q, const h16* K, const h16* V, h16* out,
                       int n_heads, int n_kv, int hd, long max_seq, int len) {
    int grp = n_heads / n_kv;
    float scale = 1.0f / sqrtf((float)hd);
    int chunk = (len + ORC_REF_PARTS - 1) / ORC_REF_PARTS;
    int nonempty = (len + chunk - 1) / chunk;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < n_heads; ++h) {
        const h16* Kh = K + (size_t)(h / grp) * max_seq * hd;
        const h16* Vh = V + (size_t)(h / grp) * max_seq * hd;
        float pm[ORC_REF_PARTS], ps[ORC_REF_PARTS];
        float* po = (float*)calloc((size_t)ORC_REF_PARTS * hd, sizeof(float));
        for (int p = 0; p < nonempty; ++p) {
            int t0 = p * chunk, t1 = t0 + chunk < len ? t0 + chunk : len;
            int nk = t1 - t0;
            h16* sc = (h16*)malloc(sizeof(h16) * nk);
            float mx = -1e30f;
            for (int t = 0; t < nk; ++t) {
                float a = 0.0f;
                for (int d = 0; d < hd; ++d) a = fmaf(h2f(Kh[(size_t)(t0 + t) * hd + d]), h2f(q[h * hd + d]), a);
                sc[t] = f2h(a * scale);
                mx = fmaxf(mx, h2f(sc[t]));
            }
            float sum = 0.0f;
            for (int t = 0; t < nk; ++t) {
                float e = expf(h2f(sc[t]) - mx);
                sum += e;
                float pe = h2f(f2h(e));
                for (int d = 0; d < hd; ++d) po[(size_t)p * hd + d] = fmaf(pe, h2f(Vh[(size_t)(t0 + t) * hd + d]), po[(size_t)p * hd + d]);
            }
            pm[p] = mx; ps[p] = sum;
            free(sc);
        }
        float M = -1e30f;
        for (int p = 0; p < nonempty; ++p) M = fmaxf(M, pm[p]);
        float tot = 0.0f;
        for (int p = 0; p < nonempty; ++p) tot += ps[p] * expf(pm[p] - M);
        float invs = 1.0f / (tot + 1e-9f);
        for (int d = 0; d < hd; ++d) {
            float a = 0.0f;
            for (int p = 0; p < nonempty; ++p) a += po[(size_t)p * hd + d] * expf(pm[p] - M);
            out[h * hd + d] = f2h(a * invs);
        }
        free(po);
    }
}

/* ------------------------------------------------------------------------- */
/* Whole model: loader (load_weights.cpp:36-165) + step (model.cu:76-181)     */
/* ------------------------------------------------------------------------- */
typedef struct {
    h16* in_norm; void* wq; h16* sq; h16* bq; void* wk; h16* sk; h16* bk; void* wv; h16* sv; h16* bv;
    void* wo; h16* so; h16* post_norm; void* wg; h16* sg; void* wu; h16* su; void* wd; h16* sd;
} orc_layer;

typedef struct orc_model {
    int vocab, dim, inter, n_layers, n_heads, n_kv, hd, max_seq, quant, lm_fmt;
    long ctx_cap;             /* KV rows allocated per head */
    uint8_t* blob; size_t blob_size;
    h16* embed; orc_layer* layers; h16* norm; void* lm_w; h16* lm_s; int lm_quant;
    h16 *K, *V;               /* [L][n_kv][ctx_cap][hd] */
    h16 *x, *xn, *q, *k, *v, *att, *h, *logits;
} orc_model;

static size_t proj_bytes(int quant, size_t rows, size_t cols) {
    return quant == 2 ? rows * cols / 2 : quant == 1 ? rows * cols : rows * cols * 2;
}

/* Returns NULL and writes a message on failure.  Error cases mirror the
 * reference loader: unreadable file, short header, bad magic, quant id out of
 * range, truncated tensor data. */
orc_model* orc_load(const char* path, long ctx_cap, char* err, int errlen) {
    FILE* f = fopen(path, "rb");
    if (!f) { snprintf(err, errlen, "cannot open %s", path); return NULL; }
    fseek(f, 0, SEEK_END); size_t sz = (size_t)ftell(f); fseek(f, 0, SEEK_SET);
    if (sz < 256) { snprintf(err, errlen, "short header"); fclose(f); return NULL; }
    orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
    m->blob = (uint8_t*)malloc(sz); m->blob_size = sz;
    if (fread(m->blob, 1, sz, f) != sz) { snprintf(err, errlen, "short read"); fclose(f); free(m->blob); free(m); return NULL; }
    fclose(f);
    int32_t hdr[11]; memcpy(hdr, m->blob, sizeof hdr);
    if (hdr[0] != ORC_MAGIC) { snprintf(err, errlen, "bad magic 0x%x", hdr[0]); free(m->blob); free(m); return NULL; }
    m->vocab = hdr[1]; m->dim = hdr[2]; m->inter = hdr[3]; m->n_layers = hdr[4]; m->n_heads = hdr[5];
    m->n_kv = hdr[6]; m->hd = hdr[7]; m->max_seq = hdr[8]; m->quant = hdr[9]; m->lm_fmt = hdr[10];
    if (m->quant < 0 || m->quant > 2) { snprintf(err, errlen, "bad quant id %d", m->quant); free(m->blob); free(m); return NULL; }
    size_t d = m->dim, qd = (size_t)m->n_heads * m->hd, kd = (size_t)m->n_kv * m->hd, I = m->inter, V = m->vocab;
    int Q = m->quant;
    size_t off = 256;
#define TAKE(ptr, type, nbytes) do { if (off + (nbytes) > sz) goto trunc; ptr = (type)(m->blob + off); off += (nbytes); } while (0)
#define TAKEP(w, s, rows, cols) do { TAKE(w, void*, proj_bytes(Q, rows, cols)); if (Q) TAKE(s, h16*, (rows) * ((cols) / ORC_GROUP) * 2); else s = NULL; } while (0)
    TAKE(m->embed, h16*, V * d * 2);
    m->layers = (orc_layer*)calloc(m->n_layers, sizeof(orc_layer));
    for (int l = 0; l < m->n_layers; ++l) {
        orc_layer* L = &m->layers[l];
        TAKE(L->in_norm, h16*, d * 2);
        TAKEP(L->wq, L->sq, qd, d); TAKE(L->bq, h16*, qd * 2);
        TAKEP(L->wk, L->sk, kd, d); TAKE(L->bk, h16*, kd * 2);
        TAKEP(L->wv, L->sv, kd, d); TAKE(L->bv, h16*, kd * 2);
        TAKEP(L->wo, L->so, d, qd);
        TAKE(L->post_norm, h16*, d * 2);
        TAKEP(L->wg, L->sg, I, d); TAKEP(L->wu, L->su, I, d); TAKEP(L->wd, L->sd, d, I);
    }
    TAKE(m->norm, h16*, d * 2);
    if (m->lm_fmt == 1) {
        TAKE(m->lm_w, void*, V * d); TAKE(m->lm_s, h16*, V * (d / ORC_GROUP) * 2); m->lm_quant = 1;
    } else if (sz - off >= V * d * 2) {
        TAKE(m->lm_w, void*, V * d * 2); m->lm_quant = 0;
    } else { m->lm_w = m->embed; m->lm_quant = 0; }
#undef TAKE
#undef TAKEP
    m->ctx_cap = ctx_cap;
    size_t kvn = (size_t)m->n_layers * m->n_kv * ctx_cap * m->hd;
    m->K = (h16*)calloc(kvn, 2); m->V = (h16*)calloc(kvn, 2);
    m->x = (h16*)calloc(d, 2); m->xn = (h16*)calloc(d, 2); m->q = (h16*)calloc(qd, 2); m->k = (h16*)calloc(kd, 2);
    m->v = (h16*)calloc(kd, 2); m->att = (h16*)calloc(qd, 2); m->h = (h16*)calloc(I, 2); m->logits = (h16*)calloc(V, 2);
    return m;
trunc:
    snprintf(err, errlen, "unexpected end of file in tensor data");
    free(m->layers); free(m->blob); free(m); return NULL;
}

void orc_free(orc_model* m) {
    if (!m) return;
    free(m->K); free(m->V); free(m->x); free(m->xn); free(m->q); free(m->k); free(m->v); free(m->att); free(m->h); free(m->logits);
    free(m->layers); free(m->blob); free(m);
}

void orc_dims(const orc_model* m, int* out10) {
    int v[10] = { m->vocab, m->dim, m->inter, m->n_layers, m->n_heads, m->n_kv, m->hd, m->max_seq, m->quant, m->lm_fmt };
    memcpy(out10, v, sizeof v);
}
h16* orc_kcache(orc_model* m) { return m->K; }
h16* orc_vcache(orc_model* m) { return m->V; }
h16* orc_logits_ptr(orc_model* m) { return m->logits; }
h16* orc_x_ptr(orc_model* m) { return m->x; }

/* One decode step (model.cu:76-181).  attn_mode 0 = exact attention,
 * 1 = reference-faithful rounding.  Returns the greedy token. */
int orc_step(orc_model* m, int token, int pos, const int* hist, int hist_len, int attn_mode) {
    long d = m->dim, qd = (long)m->n_heads * m->hd, kd = (long)m->n_kv * m->hd;
    int Q = m->quant;
    h16 eps = f2h(1e-6f), pen = f2h(1.1f);
    memcpy(m->x, m->embed + (size_t)token * d, d * 2);                       /* model.cu:89 */
    for (int l = 0; l < m->n_layers; ++l) {
        orc_layer* L = &m->layers[l];
        orc_rmsnorm(m->x, L->in_norm, m->xn, d, eps);                        /* :94 */
        orc_qkv(Q, m->xn, L->wq, L->wk, L->wv, L->sq, L->sk, L->sv, L->bq, L->bk, L->bv, m->q, m->k, m->v, d, qd, kd);
        orc_rope(m->q, m->k, m->n_heads, m->n_kv, m->hd, pos, 1000000.0f);   /* :99 */
        h16* Kl = m->K + (size_t)l * m->n_kv * m->ctx_cap * m->hd;
        h16* Vl = m->V + (size_t)l * m->n_kv * m->ctx_cap * m->hd;
        for (int h = 0; h < m->n_kv; ++h) {                                  /* :117 */
            memcpy(Kl + ((size_t)h * m->ctx_cap + pos) * m->hd, m->k + h * m->hd, m->hd * 2);
            memcpy(Vl + ((size_t)h * m->ctx_cap + pos) * m->hd, m->v + h * m->hd, m->hd * 2);
        }
        if (attn_mode) orc_attention_ref(m->q, Kl, Vl, m->att, m->n_heads, m->n_kv, m->hd, m->ctx_cap, pos + 1);
        else orc_attention_exact(m->q, Kl, Vl, m->att, m->n_heads, m->n_kv, m->hd, m->ctx_cap, pos + 1);   /* :122 */
        orc_gemv_add(Q, L->wo, L->so, m->att, m->x, d, qd);                  /* :129 */
        orc_rmsnorm(m->x, L->post_norm, m->xn, d, eps);                      /* :131 */
        orc_mlp1(Q, m->xn, L->wg, L->wu, L->sg, L->su, m->h, d, m->inter);   /* :136 */
        orc_gemv_add(Q, L->wd, L->sd, m->h, m->x, d, m->inter);              /* :148 */
    }
    orc_rmsnorm(m->x, m->norm, m->xn, d, eps);                               /* :158 */
    orc_logits(m->lm_quant, m->lm_w, m->lm_s, m->xn, m->logits, m->vocab, d); /* :163-173 */
    orc_penalty(m->logits, hist, hist_len, m->vocab, pen);                   /* :175 */
    return orc_argmax(m->logits, m->vocab);                                  /* :180 */
}
