// A program written the way CuQwen's chat front end uses its tokenizer (src/main.cu:19-21, :64-70, :99, :123):
// it includes "tokenizer.h", builds a prompt from Messages, encodes it and decodes it back.  The test compiles it
// against include/compat/tokenizer.h and compares what it prints with the Python binding.
//
//   tokenizer_probe <ranks.json> <user text>      prints: the ids on one line, then the decoded bytes
//   tokenizer_probe <missing file>                prints the exception text, exits 3
#include <cstdio>
#include <iostream>
#include <string>
#include <vector>

#include "tokenizer.h"

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    try {
        QwenTokenizer tokenizer(argv[1]);
        std::vector<Message> conversation = {{"system", "You are a helpful assistant."}, {"user", argc > 2 ? argv[2] : ""}};
        const std::string prompt = tokenizer.apply_chat_template(conversation, true);
        const std::vector<int> ids = tokenizer.encode(prompt);
        for (size_t i = 0; i < ids.size(); ++i) std::cout << (i ? " " : "") << ids[i];
        std::cout << "\n";
        std::string pieces;
        for (int id : ids) pieces += tokenizer.decode_single(id);
        if (pieces != tokenizer.decode(ids)) return 4;
        std::cout << pieces;
    } catch (const std::runtime_error& e) {
        std::cout << e.what() << "\n";
        return 3;
    }
    return 0;
}
