// Writes a random-initialised Qwen2.5 weight file in CuQwen's binary format
// (layout: export_weights.py:267-323 of that project; quantisation rule:
// export_weights.py:123-205): 256-byte header of int32 fields, fp16 embedding,
// per-layer tensors in the reference's fixed order, final norm, optional
// lm_head.  Projection weights ~ N(0, 0.02) before quantisation, biases and
// embeddings ~ N(0, 0.02), RMSNorm weights ~ 1 + N(0, 0.02).  Every value is a
// pure function of (seed, tensor id, element index), so the file does not
// depend on the number of threads.
//
// Usage:
//   gen_random_bin --out FILE --model 0.5b|1.5b|3b|7b|14b --quant fp16|int8|int4 [--seed N] [--threads N]
//   gen_random_bin --out FILE --dims VOCAB DIM INTER LAYERS HEADS KV HD --quant ... [--untied]
//   gen_random_bin --quantize IN.f32 ROWS COLS int8|int4 OUT.bin     (quantise one fp32 matrix; used by tests)
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

static const int kGroup = 128;

static inline uint64_t mix(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// Two N(0,1) values for pair index j of tensor t.
static inline void normal2(uint64_t seed, uint64_t tensor, uint64_t j, float* a, float* b) {
    uint64_t h = mix(mix(seed * 0x2545F4914F6CDD1Dull + tensor) + j);
    float u1 = ((float)((h >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f);
    float u2 = (float)((h >> 16) & 0xFFFFFF) * (1.0f / 16777216.0f);
    float r = std::sqrt(-2.0f * std::log(u1)), th = 6.28318530718f * u2;
    *a = r * std::cos(th); *b = r * std::sin(th);
}

// fp32 -> fp16 bits, round to nearest even (matches numpy astype(float16)).
static inline uint16_t f2h(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u; x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);                  // rounds to inf
    if (x < 0x33000001u) return (uint16_t)sign;                               // rounds to zero
    int e = (int)(x >> 23) - 127;
    uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    int shift = e < -14 ? (13 + (-14 - e)) : 13;
    uint32_t hm = m >> shift, rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (hm & 1))) ++hm;
    uint32_t he = e < -14 ? 0 : (uint32_t)(e + 15);
    return (uint16_t)(sign | ((he << 10) + (e < -14 ? hm : (hm - 0x400u))));
}
static inline float h2f(uint16_t h) {
    uint32_t s = (h & 0x8000u) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF, x;
    if (e == 0) { if (!m) x = s; else { int k = 0; while (!(m & 0x400)) { m <<= 1; ++k; } x = s | ((uint32_t)(113 - k) << 23) | ((m & 0x3FF) << 13); } }
    else if (e == 31) x = s | 0x7F800000u | (m << 13);
    else x = s | ((e + 112) << 23) | (m << 13);
    float f; memcpy(&f, &x, 4); return f;
}

// Symmetric group quantisation of one row (export_weights.py:123-183): scale = max|w| / qmax in fp32, q =
// clip(rint(w / scale_fp32)), the stored scale is the fp16 rounding of scale_fp32; an all-zero group gets scale 0.
static void quant_row(const float* w, int cols, int qmax, int8_t* q, uint16_t* scales) {
    for (int g = 0; g < cols / kGroup; ++g) {
        float mx = 0.f;
        for (int i = 0; i < kGroup; ++i) { float a = std::fabs(w[g * kGroup + i]); if (a > mx) mx = a; }
        float scale = mx / (float)qmax, safe = scale > 0.f ? scale : 1.0f;
        for (int i = 0; i < kGroup; ++i) {
            float v = std::nearbyintf(w[g * kGroup + i] / safe);
            if (v > qmax) v = (float)qmax; if (v < -qmax) v = (float)-qmax;
            q[g * kGroup + i] = (int8_t)v;
        }
        scales[g] = f2h(scale);
    }
}
static void pack_row(int quant, const float* w, int cols, uint8_t* wout, uint16_t* sout, int8_t* tmp) {
    if (quant == 0) { uint16_t* o = (uint16_t*)wout; for (int i = 0; i < cols; ++i) o[i] = f2h(w[i]); return; }
    if (quant == 1) { quant_row(w, cols, 127, (int8_t*)wout, sout); return; }
    quant_row(w, cols, 7, tmp, sout);
    for (int p = 0; p < cols / 2; ++p) wout[p] = (uint8_t)((tmp[2 * p] & 0xF) | ((tmp[2 * p + 1] & 0xF) << 4));
}
static size_t row_bytes(int quant, size_t cols) { return quant == 2 ? cols / 2 : quant == 1 ? cols : cols * 2; }

struct Writer {
    FILE* f; uint64_t seed; int threads; uint64_t tensor = 0;
    // mode 0: N(0, sigma); mode 1: 1 + N(0, sigma)
    void matrix(int quant, size_t rows, size_t cols, float sigma, int mode = 0) {
        const uint64_t tid = tensor++;
        const size_t rb = row_bytes(quant, cols), ng = cols / kGroup;
        std::vector<uint16_t> scales(quant ? rows * ng : 0);
        const size_t chunk = 2048;
        std::vector<uint8_t> buf(chunk * rb);
        for (size_t r0 = 0; r0 < rows; r0 += chunk) {
            const size_t nr = rows - r0 < chunk ? rows - r0 : chunk;
            std::vector<std::thread> th;
            for (int t = 0; t < threads; ++t)
                th.emplace_back([&, t]() {
                    std::vector<float> row(cols + 1); std::vector<int8_t> tmp(cols);
                    for (size_t r = r0 + t; r < r0 + nr; r += threads) {
                        const uint64_t base = (uint64_t)r * cols;
                        for (size_t c = 0; c < cols; c += 2) {
                            float a, b; normal2(seed, tid, (base + c) >> 1, &a, &b);
                            row[c] = (mode ? 1.0f : 0.0f) + sigma * a;
                            row[c + 1] = (mode ? 1.0f : 0.0f) + sigma * b;
                        }
                        pack_row(quant, row.data(), (int)cols, buf.data() + (r - r0) * rb, quant ? scales.data() + r * ng : nullptr, tmp.data());
                    }
                });
            for (auto& x : th) x.join();
            if (fwrite(buf.data(), 1, nr * rb, f) != nr * rb) { perror("fwrite"); exit(1); }
        }
        if (quant && fwrite(scales.data(), 2, scales.size(), f) != scales.size()) { perror("fwrite"); exit(1); }
    }
};

struct Dims { int vocab, dim, inter, layers, heads, kv, hd; bool tied; };
static bool lookup(const std::string& m, Dims* d) {
    if (m == "0.5b") *d = {151936, 896, 4864, 24, 14, 2, 64, true};
    else if (m == "1.5b") *d = {151936, 1536, 8960, 28, 12, 2, 128, true};
    else if (m == "3b") *d = {151936, 2048, 11008, 36, 16, 2, 128, true};
    else if (m == "7b") *d = {152064, 3584, 18944, 28, 28, 4, 128, false};
    else if (m == "14b") *d = {152064, 5120, 13824, 48, 40, 8, 128, false};
    else return false;
    return true;
}
static int quant_id(const std::string& q) { return q == "fp16" ? 0 : q == "int8" ? 1 : q == "int4" ? 2 : -1; }

int main(int argc, char** argv) {
    std::string out, model, quant = "fp16";
    Dims d{}; bool have_dims = false, untied = false; uint64_t seed = 1234; int threads = (int)std::thread::hardware_concurrency();
    if (threads < 1) threads = 1;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        if (a == "--quantize" && i + 5 < argc) {
            const char* in = argv[i + 1]; size_t rows = atol(argv[i + 2]), cols = atol(argv[i + 3]); int q = quant_id(argv[i + 4]); const char* o = argv[i + 5];
            if (q < 1 || cols % kGroup) { fprintf(stderr, "bad --quantize arguments\n"); return 2; }
            std::vector<float> w(rows * cols);
            FILE* fi = fopen(in, "rb"); if (!fi || fread(w.data(), 4, w.size(), fi) != w.size()) { fprintf(stderr, "cannot read %s\n", in); return 2; } fclose(fi);
            std::vector<uint8_t> wb(rows * row_bytes(q, cols)); std::vector<uint16_t> sb(rows * (cols / kGroup)); std::vector<int8_t> tmp(cols);
            for (size_t r = 0; r < rows; ++r) pack_row(q, w.data() + r * cols, (int)cols, wb.data() + r * row_bytes(q, cols), sb.data() + r * (cols / kGroup), tmp.data());
            FILE* fo = fopen(o, "wb"); fwrite(wb.data(), 1, wb.size(), fo); fwrite(sb.data(), 2, sb.size(), fo); fclose(fo);
            return 0;
        }
        else if (a == "--out" && i + 1 < argc) out = argv[++i];
        else if (a == "--model" && i + 1 < argc) model = argv[++i];
        else if (a == "--quant" && i + 1 < argc) quant = argv[++i];
        else if (a == "--seed" && i + 1 < argc) seed = strtoull(argv[++i], nullptr, 10);
        else if (a == "--threads" && i + 1 < argc) threads = atoi(argv[++i]);
        else if (a == "--untied") untied = true;
        else if (a == "--dims" && i + 7 < argc) {
            d.vocab = atoi(argv[i + 1]); d.dim = atoi(argv[i + 2]); d.inter = atoi(argv[i + 3]); d.layers = atoi(argv[i + 4]);
            d.heads = atoi(argv[i + 5]); d.kv = atoi(argv[i + 6]); d.hd = atoi(argv[i + 7]); d.tied = true; have_dims = true; i += 7;
        } else { fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
    }
    if (!have_dims) { Dims t; if (!lookup(model, &t)) { fprintf(stderr, "need --model or --dims\n"); return 2; } d = t; }
    if (untied) d.tied = false;
    const int Q = quant_id(quant);
    if (Q < 0 || out.empty()) { fprintf(stderr, "need --out and a valid --quant\n"); return 2; }
    if (d.dim % kGroup || d.inter % kGroup || (d.heads * d.hd) % kGroup) { fprintf(stderr, "dims must be multiples of 128\n"); return 2; }
    FILE* f = fopen(out.c_str(), "wb");
    if (!f) { perror("fopen"); return 1; }
    // INT8 lm_head iff quantised and untied (export_weights.py:261)
    const int lm_fmt = (Q != 0 && !d.tied) ? 1 : 0;
    int32_t hdr[64] = {0};
    hdr[0] = 0x5157454E; hdr[1] = d.vocab; hdr[2] = d.dim; hdr[3] = d.inter; hdr[4] = d.layers; hdr[5] = d.heads; hdr[6] = d.kv; hdr[7] = d.hd;
    hdr[8] = 32768; hdr[9] = Q; hdr[10] = lm_fmt;
    fwrite(hdr, 4, 64, f);
    Writer w{f, seed, threads};
    const size_t qd = (size_t)d.heads * d.hd, kd = (size_t)d.kv * d.hd;
    const float S = 0.02f;
    w.matrix(0, d.vocab, d.dim, S);
    for (int l = 0; l < d.layers; ++l) {
        w.matrix(0, 1, d.dim, S, 1);
        w.matrix(Q, qd, d.dim, S); w.matrix(0, 1, qd, S);
        w.matrix(Q, kd, d.dim, S); w.matrix(0, 1, kd, S);
        w.matrix(Q, kd, d.dim, S); w.matrix(0, 1, kd, S);
        w.matrix(Q, d.dim, qd, S);
        w.matrix(0, 1, d.dim, S, 1);
        w.matrix(Q, d.inter, d.dim, S); w.matrix(Q, d.inter, d.dim, S); w.matrix(Q, d.dim, d.inter, S);
    }
    w.matrix(0, 1, d.dim, S, 1);
    if (!d.tied) w.matrix(lm_fmt ? 1 : 0, d.vocab, d.dim, S);
    fclose(f);
    return 0;
}
