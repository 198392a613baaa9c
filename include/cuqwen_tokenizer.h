/* C ABI of the Qwen2.5 byte-level BPE tokenizer (host only, no CUDA; library libcuqwen_tok.so).
 *
 * It replaces the reference's C++ class QwenTokenizer (include/tokenizer.h:17-42, src/tokenizer.cpp) and needs
 * neither PCRE2 nor a JSON library: the pre-tokenising pattern (src/tokenizer.cpp:72) is a hand-written scanner
 * over Unicode category tables, and the ranks file is read by a small JSON reader.
 *
 * Ranks file (written by the reference's export_weights.py:328-363): one JSON object with
 *   "vocab":        { "<token string in the GPT-2 byte alphabet>": <id>, ... }   rank of a merge == its id
 *   "added_tokens": { "<id>": "<literal special token>", ... }                   optional
 * Other keys are ignored.
 *
 * All functions return 0 on success or one of the CUQWEN_TOK_E_* codes; cuqwen_tok_last_error() gives the calling
 * thread's message.  A tokenizer object is immutable after cuqwen_tok_open and may be shared between threads.
 * Buffers are caller-owned; when one is too small the call returns CUQWEN_TOK_E_SPACE and *n_out holds the size
 * that is needed (nothing beyond `cap` is written).
 */
#ifndef CUQWEN_TOKENIZER_H
#define CUQWEN_TOKENIZER_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cuqwen_tokenizer cuqwen_tokenizer;

enum {
    CUQWEN_TOK_OK = 0,
    CUQWEN_TOK_E_IO = 1,     /* the ranks file cannot be opened (reference: std::runtime_error, src/tokenizer.cpp:42-44) */
    CUQWEN_TOK_E_PARSE = 2,  /* the file is not the JSON described above */
    CUQWEN_TOK_E_SPACE = 3,  /* output buffer too small */
    CUQWEN_TOK_E_ARG = 4     /* null pointer or similar */
};

/* QwenTokenizer::QwenTokenizer(path)  (src/tokenizer.cpp:41-83) */
int cuqwen_tok_open(const char* ranks_json_path, cuqwen_tokenizer** out);
/* QwenTokenizer::~QwenTokenizer  (src/tokenizer.cpp:85-88) */
void cuqwen_tok_close(cuqwen_tokenizer* tok);

/* QwenTokenizer::encode  (src/tokenizer.cpp:169-201): literal special tokens are cut out first (earliest
 * occurrence, longest on a tie), the text between them is pre-tokenised and merged.  `text` is `text_len` bytes of
 * UTF-8 and need not end in NUL.  A stretch between special tokens that is not valid UTF-8 yields no tokens, as in
 * the reference (its PCRE2 match fails on such a subject, src/tokenizer.cpp:152-153). */
int cuqwen_tok_encode(const cuqwen_tokenizer* tok, const char* text, size_t text_len, int* ids, size_t cap, size_t* n_out);

/* QwenTokenizer::decode / decode_single  (src/tokenizer.cpp:203-240): bytes of the tokens, concatenated; an id that
 * is not in "vocab" contributes nothing.  The output is raw bytes (not NUL-terminated, possibly a partial UTF-8
 * sequence when a character is split across tokens). */
int cuqwen_tok_decode(const cuqwen_tokenizer* tok, const int* ids, size_t n, char* out, size_t cap, size_t* n_out);

/* QwenTokenizer::apply_chat_template  (src/tokenizer.cpp:90-99): ChatML,
 * "<|im_start|>" role "\n" content "<|im_end|>\n" per message, then "<|im_start|>assistant\n" when asked. */
int cuqwen_tok_chat_template(const char* const* roles, const char* const* contents, size_t n_messages,
                             int add_generation_prompt, char* out, size_t cap, size_t* n_out);

/* The pre-tokeniser alone (the pattern of src/tokenizer.cpp:72 applied as in :146-167): writes the END byte offset
 * of every piece of `text`.  Invalid UTF-8 gives zero pieces.  Used by the parity tests. */
int cuqwen_tok_pretokenize(const char* text, size_t text_len, size_t* ends, size_t cap, size_t* n_out);

/* Number of entries of "vocab", and of "added_tokens". */
size_t cuqwen_tok_vocab_size(const cuqwen_tokenizer* tok);
size_t cuqwen_tok_special_count(const cuqwen_tokenizer* tok);

const char* cuqwen_tok_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* CUQWEN_TOKENIZER_H */
