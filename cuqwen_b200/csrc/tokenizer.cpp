// Qwen2.5 byte-level BPE tokenizer behind the C ABI of include/cuqwen_tokenizer.h.  Host code only.
//
// Behaviour follows the reference's QwenTokenizer (src/tokenizer.cpp): GPT-2 byte alphabet (:10-38), ranks file
// (:41-62), special tokens longest first (:64-67, :169-201), the Qwen2.5 pre-tokenising pattern (:72) applied
// left to right (:146-167), merges by lowest token id (:101-144), byte decoding (:211-240), ChatML (:90-99).
// The reference leans on PCRE2 and nlohmann::json; here the pattern is a hand-written scanner over the category
// tables of unicode_tables.h and the ranks file is read by the small JSON reader below.
#include "../../include/cuqwen_tokenizer.h"

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

#include "unicode_tables.h"

namespace {

thread_local std::string g_error;

int fail(int code, const std::string& msg) {
    g_error = msg;
    return code;
}

// ---------------------------------------------------------------------------------------------------------------
// Code point classes.  With PCRE2_UCP, \p{L} and \p{N} are the general categories and \s is "\p{Z} or \h or \v".
// ---------------------------------------------------------------------------------------------------------------
bool in_ranges(const uint32_t (*r)[2], int n, uint32_t cp) {
    int lo = 0, hi = n - 1;
    while (lo <= hi) {
        const int mid = (lo + hi) / 2;
        if (cp < r[mid][0]) hi = mid - 1;
        else if (cp > r[mid][1]) lo = mid + 1;
        else return true;
    }
    return false;
}

enum : uint8_t { C_OTHER = 0, C_LETTER = 1, C_NUMBER = 2, C_SPACE = 3 };

uint8_t classify_slow(uint32_t cp) {
    if (in_ranges(kUniLetter, kUniLetter_count, cp)) return C_LETTER;
    if (in_ranges(kUniNumber, kUniNumber_count, cp)) return C_NUMBER;
    if (in_ranges(kUniSeparator, kUniSeparator_count, cp)) return C_SPACE;
    // \h beyond category Z (tab; U+180E left category Zs in Unicode 6.3 but PCRE2 keeps it in \h), and \v
    if (cp == 0x09 || cp == 0x180E || (cp >= 0x0A && cp <= 0x0D) || cp == 0x85) return C_SPACE;
    return C_OTHER;
}

struct ClassTable {
    uint8_t low[0x3000];
    ClassTable() {
        for (uint32_t c = 0; c < 0x3000; ++c) low[c] = classify_slow(c);
    }
};
const ClassTable g_classes;

inline uint8_t classify(uint32_t cp) { return cp < 0x3000 ? g_classes.low[cp] : classify_slow(cp); }

// ---------------------------------------------------------------------------------------------------------------
// UTF-8: validation with the rules PCRE2 applies to a subject (no overlong forms, no surrogates, nothing above
// U+10FFFF, no 5/6-byte forms), and decoding into code points with their byte offsets.
// ---------------------------------------------------------------------------------------------------------------
struct CodePoints {
    std::vector<uint32_t> cp;
    std::vector<uint32_t> off;   // off[i] = byte offset of cp[i]; off[n] = text length
};

bool decode_utf8(const char* s, size_t n, CodePoints& out) {
    out.cp.clear();
    out.off.clear();
    out.cp.reserve(n);
    out.off.reserve(n + 1);
    const unsigned char* p = (const unsigned char*)s;
    size_t i = 0;
    while (i < n) {
        const uint32_t b0 = p[i];
        uint32_t cp;
        int len;
        if (b0 < 0x80) { cp = b0; len = 1; }
        else if (b0 >= 0xC2 && b0 <= 0xDF) { cp = b0 & 0x1F; len = 2; }
        else if (b0 >= 0xE0 && b0 <= 0xEF) { cp = b0 & 0x0F; len = 3; }
        else if (b0 >= 0xF0 && b0 <= 0xF4) { cp = b0 & 0x07; len = 4; }
        else return false;
        if (i + len > n) return false;
        for (int k = 1; k < len; ++k) {
            const uint32_t b = p[i + k];
            if ((b & 0xC0) != 0x80) return false;
            cp = (cp << 6) | (b & 0x3F);
        }
        if (len == 3 && (cp < 0x800 || (cp >= 0xD800 && cp <= 0xDFFF))) return false;
        if (len == 4 && (cp < 0x10000 || cp > 0x10FFFF)) return false;
        out.cp.push_back(cp);
        out.off.push_back((uint32_t)i);
        i += len;
    }
    out.off.push_back((uint32_t)n);
    return true;
}

void append_utf8(std::string& s, uint32_t cp) {
    if (cp < 0x80) s += (char)cp;
    else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
    else { s += (char)(0xF0 | (cp >> 18)); s += (char)(0x80 | ((cp >> 12) & 0x3F)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
}

// ---------------------------------------------------------------------------------------------------------------
// The pre-tokeniser.  One call returns the end (code point index) of the piece that starts at i, trying the
// alternatives of the pattern in their written order, each with the backtracking a regex engine would do:
//   1  (?i:'s|'t|'re|'ve|'m|'ll|'d)
//   2  [^\r\n\p{L}\p{N}]?\p{L}+
//   3  \p{N}
//   4   ?[^\s\p{L}\p{N}]+[\r\n]*
//   5  \s*[\r\n]+
//   6  \s+(?!\S)
//   7  \s+
// Every code point is a letter, a number, white space or "other", so one of 2, 3, 4, 7 always matches: the scan
// never has to skip input.
// ---------------------------------------------------------------------------------------------------------------
inline bool is_crlf(uint32_t c) { return c == '\r' || c == '\n'; }

// caseless comparison against an ASCII lower-case letter; U+017F (long s) folds to 's' under Unicode caseless matching
inline bool ci_eq(uint32_t c, char lower) {
    if (c == (uint32_t)lower || c == (uint32_t)(lower - 32)) return true;
    return lower == 's' && c == 0x17F;
}

size_t next_piece(const std::vector<uint32_t>& cp, size_t i) {
    const size_t n = cp.size();
    const uint32_t c0 = cp[i];
    // 1: contractions
    if (c0 == '\'' && i + 1 < n) {
        const uint32_t c1 = cp[i + 1];
        if (ci_eq(c1, 's') || ci_eq(c1, 't')) return i + 2;
        if (i + 2 < n && ci_eq(c1, 'r') && ci_eq(cp[i + 2], 'e')) return i + 3;
        if (i + 2 < n && ci_eq(c1, 'v') && ci_eq(cp[i + 2], 'e')) return i + 3;
        if (ci_eq(c1, 'm')) return i + 2;
        if (i + 2 < n && ci_eq(c1, 'l') && ci_eq(cp[i + 2], 'l')) return i + 3;
        if (ci_eq(c1, 'd')) return i + 2;
    }
    const uint8_t k0 = classify(c0);
    // 2: an optional leading character that is no letter, number, CR or LF, then letters
    {
        size_t j = i;
        if (k0 != C_LETTER && k0 != C_NUMBER && !is_crlf(c0) && i + 1 < n && classify(cp[i + 1]) == C_LETTER) j = i + 1;
        if (classify(cp[j]) == C_LETTER) {
            while (j < n && classify(cp[j]) == C_LETTER) ++j;
            return j;
        }
    }
    // 3: a single number character
    if (k0 == C_NUMBER) return i + 1;
    // 4: an optional space, then characters that are neither white space, letters nor numbers, then CR/LF
    {
        size_t j = i;
        if (c0 == ' ' && i + 1 < n && classify(cp[i + 1]) == C_OTHER) j = i + 1;
        if (classify(cp[j]) == C_OTHER) {
            while (j < n && classify(cp[j]) == C_OTHER) ++j;
            while (j < n && is_crlf(cp[j])) ++j;
            return j;
        }
    }
    // here c0 is white space
    size_t e = i;
    while (e < n && classify(cp[e]) == C_SPACE) ++e;
    // 5: white space up to and including its last CR/LF
    for (size_t j = e; j > i; --j)
        if (is_crlf(cp[j - 1])) return j;
    // 6: white space not followed by a non-space: the whole run at the end of the text, else all but its last character
    if (e == n) return e;
    if (e - i >= 2) return e - 1;
    // 7
    return e;
}

// ---------------------------------------------------------------------------------------------------------------
// Minimal JSON reader: enough for the ranks file (objects, arrays, strings with all escapes, numbers, literals).
// ---------------------------------------------------------------------------------------------------------------
struct JsonReader {
    const char* p;
    const char* end;

    [[noreturn]] void bad(const char* what) const { throw std::runtime_error(std::string("JSON: ") + what); }
    void ws() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p;
    }
    char peek() {
        ws();
        if (p >= end) bad("unexpected end of file");
        return *p;
    }
    void expect(char c) {
        if (peek() != c) bad("unexpected character");
        ++p;
    }
    static int hex(char c) {
        if (c >= '0' && c <= '9') return c - '0';
        if (c >= 'a' && c <= 'f') return c - 'a' + 10;
        if (c >= 'A' && c <= 'F') return c - 'A' + 10;
        return -1;
    }
    uint32_t hex4() {
        if (end - p < 4) bad("short \\u escape");
        uint32_t v = 0;
        for (int k = 0; k < 4; ++k) {
            const int h = hex(p[k]);
            if (h < 0) bad("bad \\u escape");
            v = v * 16 + (uint32_t)h;
        }
        p += 4;
        return v;
    }
    std::string string() {
        expect('"');
        std::string s;
        for (;;) {
            if (p >= end) bad("unterminated string");
            const char c = *p++;
            if (c == '"') return s;
            if (c != '\\') { s += c; continue; }
            if (p >= end) bad("unterminated escape");
            const char e = *p++;
            switch (e) {
                case '"': s += '"'; break;
                case '\\': s += '\\'; break;
                case '/': s += '/'; break;
                case 'b': s += '\b'; break;
                case 'f': s += '\f'; break;
                case 'n': s += '\n'; break;
                case 'r': s += '\r'; break;
                case 't': s += '\t'; break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp <= 0xDBFF) {
                        if (end - p < 6 || p[0] != '\\' || p[1] != 'u') bad("lone surrogate");
                        p += 2;
                        const uint32_t lo = hex4();
                        if (lo < 0xDC00 || lo > 0xDFFF) bad("bad surrogate pair");
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
                        bad("lone surrogate");
                    }
                    append_utf8(s, cp);
                    break;
                }
                default: bad("unknown escape");
            }
        }
    }
    // a number as a double (the ids of the ranks file are small integers)
    double number() {
        ws();
        const char* s = p;
        if (p < end && (*p == '-' || *p == '+')) ++p;
        while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) ++p;
        if (p == s) bad("number expected");
        return std::stod(std::string(s, p));
    }
    void skip_value() {
        const char c = peek();
        if (c == '"') { string(); return; }
        if (c == '{') {
            ++p;
            if (peek() == '}') { ++p; return; }
            for (;;) {
                string();
                expect(':');
                skip_value();
                if (peek() == ',') { ++p; continue; }
                expect('}');
                return;
            }
        }
        if (c == '[') {
            ++p;
            if (peek() == ']') { ++p; return; }
            for (;;) {
                skip_value();
                if (peek() == ',') { ++p; continue; }
                expect(']');
                return;
            }
        }
        if (c == 't' && end - p >= 4 && !memcmp(p, "true", 4)) { p += 4; return; }
        if (c == 'f' && end - p >= 5 && !memcmp(p, "false", 5)) { p += 5; return; }
        if (c == 'n' && end - p >= 4 && !memcmp(p, "null", 4)) { p += 4; return; }
        number();
    }
    // calls f(key) for every member of an object; f must consume the value
    template <class F> void object(F f) {
        expect('{');
        if (peek() == '}') { ++p; return; }
        for (;;) {
            std::string key = string();
            expect(':');
            f(key);
            if (peek() == ',') { ++p; continue; }
            expect('}');
            return;
        }
    }
};

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// The tokenizer object
// ---------------------------------------------------------------------------------------------------------------
struct cuqwen_tokenizer {
    // token string -> id.  Open addressing over an arena of the strings, so that look-ups take a string_view of the
    // chunk being merged and allocate nothing.
    std::string arena;
    struct Slot { uint32_t off, len; int id; };
    std::vector<Slot> table;     // size is a power of two; len == UINT32_MAX marks an empty slot
    size_t n_vocab = 0;

    std::unordered_map<int, std::string> id_to_bytes;   // id -> decoded bytes (special-token strings stay literal)
    std::vector<std::pair<std::string, int>> specials;  // longest first
    std::string byte_symbol[256];                       // byte -> its symbol of the GPT-2 alphabet (UTF-8)

    static uint64_t hash(std::string_view s) {
        uint64_t h = 1469598103934665603ull;
        for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
        return h;
    }
    void reserve(size_t n) {
        size_t cap = 16;
        while (cap < n * 2 + 2) cap <<= 1;
        table.assign(cap, Slot{0, UINT32_MAX, 0});
    }
    void insert(std::string_view s, int id) {
        const size_t mask = table.size() - 1;
        size_t h = hash(s) & mask;
        while (table[h].len != UINT32_MAX) h = (h + 1) & mask;
        table[h] = Slot{(uint32_t)arena.size(), (uint32_t)s.size(), id};
        arena.append(s);
    }
    // returns the id or -1
    int find(std::string_view s) const {
        if (table.empty()) return -1;
        const size_t mask = table.size() - 1;
        size_t h = hash(s) & mask;
        while (table[h].len != UINT32_MAX) {
            const Slot& t = table[h];
            if (t.len == s.size() && !memcmp(arena.data() + t.off, s.data(), s.size())) return t.id;
            h = (h + 1) & mask;
        }
        return -1;
    }
};

namespace {

// The GPT-2 byte alphabet (reference src/tokenizer.cpp:10-38): printable Latin-1 bytes stand for themselves, the
// other 68 bytes take the code points 256, 257, ... in byte order.
void build_byte_alphabet(uint32_t (&symbol_cp)[256]) {
    bool keeps[256] = {};
    for (int b = '!'; b <= '~'; ++b) keeps[b] = true;
    for (int b = 0xA1; b <= 0xAC; ++b) keeps[b] = true;
    for (int b = 0xAE; b <= 0xFF; ++b) keeps[b] = true;
    uint32_t next = 256;
    for (int b = 0; b < 256; ++b) symbol_cp[b] = keeps[b] ? (uint32_t)b : next++;
}

// token string (symbols of the byte alphabet) -> bytes.  Anything that is not a symbol is copied through, as the
// reference does (src/tokenizer.cpp:218-238).
std::string symbols_to_bytes(const std::string& tok, const std::unordered_map<uint32_t, uint8_t>& cp_to_byte) {
    std::string out;
    const unsigned char* p = (const unsigned char*)tok.data();
    const size_t n = tok.size();
    size_t i = 0;
    while (i < n) {
        if (p[i] < 0x80) {
            auto it = cp_to_byte.find(p[i]);
            out += it != cp_to_byte.end() ? (char)it->second : (char)p[i];
            i += 1;
        } else if (i + 1 < n && (p[i] & 0xE0) == 0xC0 && (p[i + 1] & 0xC0) == 0x80) {
            const uint32_t cp = ((uint32_t)(p[i] & 0x1F) << 6) | (p[i + 1] & 0x3F);
            auto it = cp >= 0x80 ? cp_to_byte.find(cp) : cp_to_byte.end();
            if (it != cp_to_byte.end()) { out += (char)it->second; i += 2; }
            else { out += (char)p[i]; i += 1; }
        } else {
            out += (char)p[i];
            i += 1;
        }
    }
    return out;
}

// Merge loop over one pre-tokenised chunk (reference src/tokenizer.cpp:101-144): the chunk's bytes become symbols;
// while some adjacent pair concatenates to a vocabulary entry, the pair with the lowest id (leftmost on a tie) is
// merged, one occurrence per round.  Parts are spans of `sym`; pair ids are cached and only the two pairs next to a
// merge are looked up again.  A part that is not in the vocabulary becomes id 0 (the reference's operator[] default).
void bpe_chunk(const cuqwen_tokenizer& t, const char* bytes, size_t n, std::string& sym, std::vector<uint32_t>& start,
               std::vector<int>& pair_id, std::vector<int>& out) {
    sym.clear();
    start.clear();
    for (size_t i = 0; i < n; ++i) {
        start.push_back((uint32_t)sym.size());
        sym += t.byte_symbol[(unsigned char)bytes[i]];
    }
    start.push_back((uint32_t)sym.size());          // start[k]..start[k+1] is part k
    size_t parts = n;
    auto view = [&](size_t a, size_t b) { return std::string_view(sym.data() + start[a], start[b] - start[a]); };
    pair_id.assign(parts > 0 ? parts - 1 : 0, -1);
    for (size_t k = 0; k + 1 < parts; ++k) pair_id[k] = t.find(view(k, k + 2));
    while (parts >= 2) {
        int best = -1, best_id = INT32_MAX;
        for (size_t k = 0; k + 1 < parts; ++k)
            if (pair_id[k] >= 0 && pair_id[k] < best_id) { best_id = pair_id[k]; best = (int)k; }
        if (best < 0) break;
        // parts best and best+1 become one: drop boundary best+1
        start.erase(start.begin() + best + 1);
        pair_id.erase(pair_id.begin() + best);
        --parts;
        if (best > 0) pair_id[best - 1] = t.find(view(best - 1, best + 1));
        if ((size_t)best + 1 < parts) pair_id[best] = t.find(view(best, best + 2));
    }
    for (size_t k = 0; k < parts; ++k) {
        const int id = t.find(view(k, k + 1));
        out.push_back(id < 0 ? 0 : id);
    }
}

struct Scratch {
    CodePoints cps;
    std::string sym;
    std::vector<uint32_t> start;
    std::vector<int> pair_id;
};

// Pre-tokenise and merge a stretch of text that holds no special token (reference src/tokenizer.cpp:146-167).
void encode_plain(const cuqwen_tokenizer& t, const char* s, size_t n, Scratch& w, std::vector<int>& out) {
    if (n == 0 || !decode_utf8(s, n, w.cps)) return;
    const size_t ncp = w.cps.cp.size();
    size_t i = 0;
    while (i < ncp) {
        const size_t j = next_piece(w.cps.cp, i);
        bpe_chunk(t, s + w.cps.off[i], w.cps.off[j] - w.cps.off[i], w.sym, w.start, w.pair_id, out);
        i = j;
    }
}

template <class T> int copy_out(const std::vector<T>& v, T* dst, size_t cap, size_t* n_out) {
    if (n_out) *n_out = v.size();
    if (v.size() > cap) return fail(CUQWEN_TOK_E_SPACE, "output buffer too small");
    if (!v.empty()) memcpy(dst, v.data(), v.size() * sizeof(T));
    return CUQWEN_TOK_OK;
}

int copy_out(const std::string& v, char* dst, size_t cap, size_t* n_out) {
    if (n_out) *n_out = v.size();
    if (v.size() > cap) return fail(CUQWEN_TOK_E_SPACE, "output buffer too small");
    if (!v.empty()) memcpy(dst, v.data(), v.size());
    return CUQWEN_TOK_OK;
}

bool read_file(const char* path, std::string& out) {
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    char buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) out.append(buf, n);
    fclose(f);
    return true;
}

// Fills a tokenizer from the text of a ranks file; throws std::runtime_error on malformed input.
void load_ranks(cuqwen_tokenizer& t, const std::string& text) {
    std::map<std::string, int> vocab;          // byte-wise key order, later duplicates overwrite earlier ones
    std::map<std::string, std::string> added;  // id (as written) -> literal
    JsonReader r{text.data(), text.data() + text.size()};
    if (text.size() >= 3 && !memcmp(text.data(), "\xEF\xBB\xBF", 3)) r.p += 3;
    r.object([&](const std::string& key) {
        if (key == "vocab" && r.peek() == '{') {
            r.object([&](const std::string& tok) { vocab[tok] = (int)r.number(); });
        } else if (key == "added_tokens" && r.peek() == '{') {
            r.object([&](const std::string& id) { added[id] = r.string(); });
        } else {
            r.skip_value();
        }
    });
    r.ws();
    if (r.p != r.end) r.bad("trailing characters");

    uint32_t symbol_cp[256];
    build_byte_alphabet(symbol_cp);
    std::unordered_map<uint32_t, uint8_t> cp_to_byte;
    for (int b = 0; b < 256; ++b) {
        append_utf8(t.byte_symbol[b], symbol_cp[b]);
        cp_to_byte[symbol_cp[b]] = (uint8_t)b;
    }

    std::unordered_map<std::string, int> special_ids;
    for (const auto& kv : added) {
        int id;
        try {
            id = std::stoi(kv.first);
        } catch (const std::exception&) {
            throw std::runtime_error("added_tokens: key '" + kv.first + "' is not an integer");
        }
        if (kv.second.empty()) continue;   // an empty literal would match everywhere
        if (special_ids.emplace(kv.second, id).second) t.specials.emplace_back(kv.second, id);
        else {
            special_ids[kv.second] = id;
            for (auto& s : t.specials) if (s.first == kv.second) s.second = id;
        }
    }
    std::stable_sort(t.specials.begin(), t.specials.end(),
                     [](const auto& a, const auto& b) { return a.first.size() > b.first.size(); });

    t.n_vocab = vocab.size();
    t.reserve(vocab.size());
    size_t bytes = 0;
    for (const auto& kv : vocab) bytes += kv.first.size();
    t.arena.reserve(bytes);
    for (const auto& kv : vocab) {
        t.insert(kv.first, kv.second);
        // several strings with one id: the last in key order wins, as in the reference's decoder map
        t.id_to_bytes[kv.second] = special_ids.count(kv.first) ? kv.first : symbols_to_bytes(kv.first, cp_to_byte);
    }
}

}  // namespace

extern "C" {

const char* cuqwen_tok_last_error(void) { return g_error.c_str(); }

int cuqwen_tok_open(const char* ranks_json_path, cuqwen_tokenizer** out) {
    if (!ranks_json_path || !out) return fail(CUQWEN_TOK_E_ARG, "null argument");
    *out = nullptr;
    std::string text;
    if (!read_file(ranks_json_path, text)) return fail(CUQWEN_TOK_E_IO, std::string("Cannot open JSON file: ") + ranks_json_path);
    cuqwen_tokenizer* t = nullptr;
    try {
        t = new cuqwen_tokenizer();
        load_ranks(*t, text);
    } catch (const std::exception& e) {
        delete t;
        return fail(CUQWEN_TOK_E_PARSE, std::string(ranks_json_path) + ": " + e.what());
    }
    *out = t;
    return CUQWEN_TOK_OK;
}

void cuqwen_tok_close(cuqwen_tokenizer* tok) { delete tok; }

size_t cuqwen_tok_vocab_size(const cuqwen_tokenizer* tok) { return tok ? tok->n_vocab : 0; }
size_t cuqwen_tok_special_count(const cuqwen_tokenizer* tok) { return tok ? tok->specials.size() : 0; }

int cuqwen_tok_encode(const cuqwen_tokenizer* tok, const char* text, size_t text_len, int* ids, size_t cap, size_t* n_out) {
    if (!tok || (!text && text_len) || (!ids && cap)) return fail(CUQWEN_TOK_E_ARG, "null argument");
    try {
        std::vector<int> out;
        Scratch w;
        const std::string_view s(text ? text : "", text_len);
        // next occurrence of every special token at or after the cursor; refreshed only when the cursor passes it
        const size_t ns = tok->specials.size();
        std::vector<size_t> next(ns, 0);
        for (size_t k = 0; k < ns; ++k) next[k] = s.find(tok->specials[k].first, 0);
        size_t pos = 0;
        while (pos < s.size()) {
            size_t at = std::string_view::npos, which = 0;
            for (size_t k = 0; k < ns; ++k) {
                if (next[k] != std::string_view::npos && next[k] < pos) next[k] = s.find(tok->specials[k].first, pos);
                if (next[k] < at) { at = next[k]; which = k; }   // strict: the longest wins at equal positions
            }
            if (at == std::string_view::npos) {
                encode_plain(*tok, s.data() + pos, s.size() - pos, w, out);
                break;
            }
            if (at > pos) encode_plain(*tok, s.data() + pos, at - pos, w, out);
            out.push_back(tok->specials[which].second);
            pos = at + tok->specials[which].first.size();
        }
        return copy_out(out, ids, cap, n_out);
    } catch (const std::exception& e) {
        return fail(CUQWEN_TOK_E_ARG, e.what());
    }
}

int cuqwen_tok_decode(const cuqwen_tokenizer* tok, const int* ids, size_t n, char* out, size_t cap, size_t* n_out) {
    if (!tok || (!ids && n) || (!out && cap)) return fail(CUQWEN_TOK_E_ARG, "null argument");
    try {
        std::string s;
        for (size_t i = 0; i < n; ++i) {
            auto it = tok->id_to_bytes.find(ids[i]);
            if (it != tok->id_to_bytes.end()) s += it->second;
        }
        return copy_out(s, out, cap, n_out);
    } catch (const std::exception& e) {
        return fail(CUQWEN_TOK_E_ARG, e.what());
    }
}

int cuqwen_tok_chat_template(const char* const* roles, const char* const* contents, size_t n_messages,
                             int add_generation_prompt, char* out, size_t cap, size_t* n_out) {
    if ((n_messages && (!roles || !contents)) || (!out && cap)) return fail(CUQWEN_TOK_E_ARG, "null argument");
    try {
        std::string s;
        for (size_t i = 0; i < n_messages; ++i) {
            if (!roles[i] || !contents[i]) return fail(CUQWEN_TOK_E_ARG, "null message");
            s += "<|im_start|>";
            s += roles[i];
            s += "\n";
            s += contents[i];
            s += "<|im_end|>\n";
        }
        if (add_generation_prompt) s += "<|im_start|>assistant\n";
        return copy_out(s, out, cap, n_out);
    } catch (const std::exception& e) {
        return fail(CUQWEN_TOK_E_ARG, e.what());
    }
}

int cuqwen_tok_pretokenize(const char* text, size_t text_len, size_t* ends, size_t cap, size_t* n_out) {
    if ((!text && text_len) || (!ends && cap)) return fail(CUQWEN_TOK_E_ARG, "null argument");
    try {
        std::vector<size_t> v;
        CodePoints cps;
        if (text_len && decode_utf8(text, text_len, cps)) {
            size_t i = 0;
            while (i < cps.cp.size()) {
                i = next_piece(cps.cp, i);
                v.push_back(cps.off[i]);
            }
        }
        return copy_out(v, ends, cap, n_out);
    } catch (const std::exception& e) {
        return fail(CUQWEN_TOK_E_ARG, e.what());
    }
}

}  // extern "C"
