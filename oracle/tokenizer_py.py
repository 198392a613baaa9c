"""CPU restatement of the reference's tokenizer - TEST INFRASTRUCTURE, not a product path.

PARITY UNPINNED: the reference holds no test or golden vector for its tokenizer, and its tokenizer does not build
on this machine (it needs PCRE2 and nlohmann::json, neither installed), so this restatement is checked only against
the reference's source text, and the pre-tokeniser additionally against the ``tokenizers`` package's Split rule
with the same pattern (tests/test_tokenizer.py).

Each function follows the reference step by step (quadratic merge loop and all), so it is slow and meant for short
inputs.  It uses the third-party ``regex`` module for the Unicode classes; white space is spelt out as the set that
PCRE2 gives ``\\s`` under PCRE2_UCP ("\\p{Z} or \\h or \\v").
"""
from __future__ import annotations

import json

import regex

# PCRE2's \s with PCRE2_UCP: category Z, horizontal space (tab, U+180E beyond Z) and vertical space (LF VT FF CR NEL)
_WS = r"\p{Z}\t\n\x0b\f\r\x85\u180e"

# reference src/tokenizer.cpp:72, with \s and \S replaced by the explicit set
PATTERN = regex.compile(
    r"(?i:'s|'t|'re|'ve|'m|'ll|'d)"
    r"|[^\r\n\p{L}\p{N}]?\p{L}+"
    r"|\p{N}"
    rf"| ?[^{_WS}\p{{L}}\p{{N}}]+[\r\n]*"
    rf"|[{_WS}]*[\r\n]+"
    rf"|[{_WS}]+(?![^{_WS}])"
    rf"|[{_WS}]+"
)


def byte_alphabet() -> dict[int, str]:
    """byte -> symbol (reference src/tokenizer.cpp:10-38)."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(161, 173)) + list(range(174, 256))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


def chat_template(messages, add_generation_prompt: bool = True) -> str:
    """reference src/tokenizer.cpp:90-99; messages are (role, content) pairs."""
    out = ""
    for role, content in messages:
        out += "<|im_start|>" + role + "\n" + content + "<|im_end|>\n"
    if add_generation_prompt:
        out += "<|im_start|>assistant\n"
    return out


def _valid_utf8(raw: bytes) -> bool:
    try:
        raw.decode("utf-8")          # strict: rejects overlong forms, surrogates and values above U+10FFFF
        return True
    except UnicodeDecodeError:
        return False


def pretokenize(raw: bytes) -> list[bytes]:
    """reference src/tokenizer.cpp:146-167: successive matches from the running offset; a subject that is not
    valid UTF-8 makes the first match fail, so nothing comes out."""
    if not _valid_utf8(raw):
        return []
    text = raw.decode("utf-8")
    out, pos = [], 0
    while pos < len(text):
        m = PATTERN.search(text, pos)
        if m is None:
            break
        out.append(m.group(0).encode("utf-8"))
        pos = m.end()
    return out


class OracleTokenizer:
    def __init__(self, ranks_json_path):
        """reference src/tokenizer.cpp:41-70."""
        with open(ranks_json_path, "rb") as f:
            j = json.loads(f.read().decode("utf-8"))
        self.encoder: dict[str, int] = {}
        self.decoder: dict[int, str] = {}
        for key in sorted(j.get("vocab", {}), key=lambda s: s.encode("utf-8")):   # the JSON library iterates keys in byte order
            self.encoder[key] = int(j["vocab"][key])
            self.decoder[int(j["vocab"][key])] = key
        self.special: dict[str, int] = {}
        ordered = []
        added = j.get("added_tokens", {})
        for key in sorted(added, key=lambda s: s.encode("utf-8")):
            self.special[added[key]] = int(key)
            ordered.append(added[key])
        self.sorted_special = sorted(ordered, key=lambda s: -len(s.encode("utf-8")))
        self.byte_encoder = byte_alphabet()
        self.byte_decoder = {v: k for k, v in self.byte_encoder.items()}

    def bpe(self, chunk: bytes) -> list[int]:
        """reference src/tokenizer.cpp:101-144."""
        parts = [self.byte_encoder[b] for b in chunk]
        while len(parts) >= 2:
            best, best_rank = -1, None
            for i in range(len(parts) - 1):
                r = self.encoder.get(parts[i] + parts[i + 1])
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best < 0:
                break
            parts = parts[:best] + [parts[best] + parts[best + 1]] + parts[best + 2:]
        return [self.encoder.get(p, 0) for p in parts]

    def encode_chunk(self, raw: bytes) -> list[int]:
        out: list[int] = []
        for piece in pretokenize(raw):
            out += self.bpe(piece)
        return out

    def encode(self, raw: bytes) -> list[int]:
        """reference src/tokenizer.cpp:169-201 (byte offsets, as std::string::find)."""
        if isinstance(raw, str):
            raw = raw.encode("utf-8")
        out: list[int] = []
        pos = 0
        while pos < len(raw):
            nxt, matched = -1, None
            for st in self.sorted_special:
                if not st:
                    continue
                f = raw.find(st.encode("utf-8"), pos)
                if f != -1 and (nxt == -1 or f < nxt):
                    nxt, matched = f, st
            if nxt == -1:
                out += self.encode_chunk(raw[pos:])
                break
            if nxt > pos:
                out += self.encode_chunk(raw[pos:nxt])
            out.append(self.special[matched])
            pos = nxt + len(matched.encode("utf-8"))
        return out

    def decode_single(self, token_id: int) -> bytes:
        """reference src/tokenizer.cpp:211-240."""
        if token_id not in self.decoder:
            return b""
        tok = self.decoder[token_id]
        if tok in self.special:
            return tok.encode("utf-8")
        out = bytearray()
        for ch in tok:
            if ch in self.byte_decoder:
                out.append(self.byte_decoder[ch])
            else:
                out += ch.encode("utf-8")
        return bytes(out)

    def decode(self, ids) -> bytes:
        return b"".join(self.decode_single(i) for i in ids)
