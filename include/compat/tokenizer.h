// Source-compatible stand-in for CuQwen's include/tokenizer.h: the same two public types, `Message` and
// `QwenTokenizer`, with the same constructor and methods (include/tokenizer.h:12-42), implemented over the C ABI of
// cuqwen_tokenizer.h.  A program that says `#include "tokenizer.h"` builds unchanged with -I<this directory> and
// links libcuqwen_tok.so instead of the reference's tokenizer.cpp + PCRE2 + nlohmann::json.
//
// Error behaviour as in the reference: the constructor throws std::runtime_error when the ranks file cannot be
// opened ("Cannot open JSON file: <path>", src/tokenizer.cpp:42-44) or parsed.
#ifndef TOKENIZER_H
#define TOKENIZER_H

#include <stdexcept>
#include <string>
#include <vector>

#include "../cuqwen_tokenizer.h"

struct Message {
    std::string role;
    std::string content;
};

class QwenTokenizer {
    cuqwen_tokenizer* tok_ = nullptr;

public:
    explicit QwenTokenizer(const std::string& ranks_json_path) {
        if (cuqwen_tok_open(ranks_json_path.c_str(), &tok_) != CUQWEN_TOK_OK) throw std::runtime_error(cuqwen_tok_last_error());
    }
    ~QwenTokenizer() { cuqwen_tok_close(tok_); }
    QwenTokenizer(const QwenTokenizer&) = delete;
    QwenTokenizer& operator=(const QwenTokenizer&) = delete;

    std::string apply_chat_template(const std::vector<Message>& messages, bool add_generation_prompt = true) {
        std::vector<const char*> roles, contents;
        for (const Message& m : messages) {
            roles.push_back(m.role.c_str());
            contents.push_back(m.content.c_str());
        }
        size_t need = 0;
        cuqwen_tok_chat_template(roles.data(), contents.data(), messages.size(), add_generation_prompt, nullptr, 0, &need);
        std::string out(need, '\0');
        if (cuqwen_tok_chat_template(roles.data(), contents.data(), messages.size(), add_generation_prompt, &out[0], need, &need) != CUQWEN_TOK_OK)
            throw std::runtime_error(cuqwen_tok_last_error());
        return out;
    }

    std::vector<int> encode(const std::string& text) {
        std::vector<int> ids(text.size() + 1);   // a token covers at least one byte
        size_t n = 0;
        if (cuqwen_tok_encode(tok_, text.data(), text.size(), ids.data(), ids.size(), &n) != CUQWEN_TOK_OK)
            throw std::runtime_error(cuqwen_tok_last_error());
        ids.resize(n);
        return ids;
    }

    std::string decode(const std::vector<int>& token_ids) {
        size_t need = 0;
        cuqwen_tok_decode(tok_, token_ids.data(), token_ids.size(), nullptr, 0, &need);
        std::string out(need, '\0');
        if (cuqwen_tok_decode(tok_, token_ids.data(), token_ids.size(), &out[0], need, &need) != CUQWEN_TOK_OK)
            throw std::runtime_error(cuqwen_tok_last_error());
        return out;
    }

    std::string decode_single(int token_id) { return decode(std::vector<int>{token_id}); }
};

#endif  // TOKENIZER_H
