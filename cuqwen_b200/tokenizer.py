"""ctypes binding of ``libcuqwen_tok.so`` (declared in ``include/cuqwen_tokenizer.h``): the Qwen2.5 byte-level
BPE tokenizer.  Method names and meaning follow the reference's C++ class ``QwenTokenizer``
(include/tokenizer.h:17-42).  Loading fails loudly when the library has not been built.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Sequence

LIB_PATH = Path(__file__).resolve().parent / "libcuqwen_tok.so"

E_IO, E_PARSE, E_SPACE, E_ARG = 1, 2, 3, 4

_vp, _sz, _i = C.c_void_p, C.c_size_t, C.c_int
_psz, _pi = C.POINTER(C.c_size_t), C.POINTER(C.c_int)
_pstr = C.POINTER(C.c_char_p)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "cuqwen_tok_open": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "cuqwen_tok_close": (None, [_vp]),
    "cuqwen_tok_encode": (_i, [_vp, C.c_char_p, _sz, _pi, _sz, _psz]),
    "cuqwen_tok_decode": (_i, [_vp, _pi, _sz, C.c_char_p, _sz, _psz]),
    "cuqwen_tok_chat_template": (_i, [_pstr, _pstr, _sz, _i, C.c_char_p, _sz, _psz]),
    "cuqwen_tok_pretokenize": (_i, [C.c_char_p, _sz, _psz, _sz, _psz]),
    "cuqwen_tok_vocab_size": (_sz, [_vp]),
    "cuqwen_tok_special_count": (_sz, [_vp]),
    "cuqwen_tok_last_error": (C.c_char_p, []),
}

_lib = None


class TokenizerError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m cuqwen_b200.build` first")
        raw = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(raw, name)
            fn.restype, fn.argtypes = res, args
        _lib = raw
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise TokenizerError(rc, (lib().cuqwen_tok_last_error() or b"").decode("utf-8", "replace"))


def _as_bytes(text) -> bytes:
    return text if isinstance(text, (bytes, bytearray)) else str(text).encode("utf-8")


@dataclass
class Message:
    """One chat turn (reference include/tokenizer.h:12-15)."""
    role: str
    content: str


def apply_chat_template(messages: Iterable[Message], add_generation_prompt: bool = True) -> str:
    msgs = list(messages)
    n = len(msgs)
    roles = (C.c_char_p * max(n, 1))(*[_as_bytes(m.role) for m in msgs])
    contents = (C.c_char_p * max(n, 1))(*[_as_bytes(m.content) for m in msgs])
    need = C.c_size_t(0)
    rc = lib().cuqwen_tok_chat_template(roles, contents, n, int(add_generation_prompt), None, 0, C.byref(need))
    if rc not in (0, E_SPACE):
        _check(rc)
    buf = C.create_string_buffer(max(need.value, 1))
    _check(lib().cuqwen_tok_chat_template(roles, contents, n, int(add_generation_prompt), buf, need.value, C.byref(need)))
    return buf.raw[:need.value].decode("utf-8")


def pretokenize(text) -> list[bytes]:
    """Pieces the pre-tokenising pattern cuts ``text`` into (no vocabulary needed)."""
    raw = _as_bytes(text)
    cap = max(len(raw), 1)
    ends = (C.c_size_t * cap)()
    n = C.c_size_t(0)
    _check(lib().cuqwen_tok_pretokenize(raw, len(raw), ends, cap, C.byref(n)))
    out, a = [], 0
    for k in range(n.value):
        out.append(raw[a:ends[k]])
        a = ends[k]
    return out


class QwenTokenizer:
    """``QwenTokenizer(ranks_json_path)`` - encode / decode / decode_single / apply_chat_template."""

    def __init__(self, ranks_json_path):
        self._h = _vp()
        _check(lib().cuqwen_tok_open(str(ranks_json_path).encode(), C.byref(self._h)))

    def close(self) -> None:
        if self._h:
            lib().cuqwen_tok_close(self._h)
            self._h = _vp()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def vocab_size(self) -> int:
        return lib().cuqwen_tok_vocab_size(self._h)

    @property
    def special_count(self) -> int:
        return lib().cuqwen_tok_special_count(self._h)

    def encode(self, text) -> list[int]:
        raw = _as_bytes(text)
        cap = max(len(raw), 1)          # a token covers at least one byte
        ids = (C.c_int * cap)()
        n = C.c_size_t(0)
        _check(lib().cuqwen_tok_encode(self._h, raw, len(raw), ids, cap, C.byref(n)))
        return list(ids[:n.value])

    def decode_bytes(self, token_ids: Sequence[int]) -> bytes:
        n = len(token_ids)
        ids = (C.c_int * max(n, 1))(*token_ids)
        need = C.c_size_t(0)
        rc = lib().cuqwen_tok_decode(self._h, ids, n, None, 0, C.byref(need))
        if rc not in (0, E_SPACE):
            _check(rc)
        buf = C.create_string_buffer(max(need.value, 1))
        _check(lib().cuqwen_tok_decode(self._h, ids, n, buf, need.value, C.byref(need)))
        return buf.raw[:need.value]

    def decode(self, token_ids: Sequence[int]) -> str:
        return self.decode_bytes(token_ids).decode("utf-8", "replace")

    def decode_single(self, token_id: int) -> bytes:
        return self.decode_bytes([token_id])

    apply_chat_template = staticmethod(apply_chat_template)
