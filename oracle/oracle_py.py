"""ctypes access to the CPU oracle (oracle.c) and to the reference's own CUDA build (oracle/_ref).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke check and by the
benchmark's baseline legs; never by the package.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"

_vp, _i, _l, _f = C.c_void_p, C.c_int, C.c_long, C.c_float
_o = None


def build() -> Path:
    src = HERE / "oracle.c"
    if not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC", str(src), "-o", str(LIB), "-lm"], check=True)
    return LIB


def lib() -> C.CDLL:
    global _o
    if _o is None:
        if not LIB.exists():
            build()
        o = C.CDLL(str(LIB))
        sig = {
            "orc_h2f": (_f, [C.c_uint16]), "orc_f2h": (C.c_uint16, [_f]), "orc_threads": (_i, []), "orc_set_contract": (None, [_i]),
            "orc_unpack_int4": (None, [_vp, _l, _l, _vp]), "orc_dequant": (None, [_i, _vp, _vp, _l, _l, _vp]),
            "orc_gemv_f32": (None, [_i, _vp, _vp, _vp, _l, _l, _vp]), "orc_rmsnorm": (None, [_vp, _vp, _vp, _l, C.c_uint16]),
            "orc_rope": (None, [_vp, _vp, _i, _i, _i, _i, _f]),
            "orc_qkv": (None, [_i] + [_vp] * 13 + [_l, _l, _l]), "orc_gemv_add": (None, [_i, _vp, _vp, _vp, _vp, _l, _l]),
            "orc_mlp1": (None, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _l, _l]), "orc_logits": (None, [_i, _vp, _vp, _vp, _vp, _l, _l]),
            "orc_penalty": (None, [_vp, _vp, _i, _i, C.c_uint16]), "orc_argmax": (_i, [_vp, _i]),
            "orc_attention_exact": (None, [_vp, _vp, _vp, _vp, _i, _i, _i, _l, _i]),
            "orc_attention_ref": (None, [_vp, _vp, _vp, _vp, _i, _i, _i, _l, _i]),
            "orc_load": (_vp, [C.c_char_p, _l, C.c_char_p, _i]), "orc_free": (None, [_vp]), "orc_dims": (None, [_vp, _vp]),
            "orc_kcache": (_vp, [_vp]), "orc_vcache": (_vp, [_vp]), "orc_logits_ptr": (_vp, [_vp]), "orc_x_ptr": (_vp, [_vp]),
            "orc_step": (_i, [_vp, _i, _i, _vp, _i, _i]),
        }
        for n, (r, a) in sig.items():
            fn = getattr(o, n)
            fn.restype, fn.argtypes = r, a
        _o = o
    return _o


def _ptr(a):
    return None if a is None else a.ctypes.data


def h16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float16)


F2H = lambda v: int(np.float16(v).view(np.uint16))

# ---- thin numpy-level wrappers -------------------------------------------------------------------------------------


def gemv_f32(quant, W, S, x, rows, cols) -> np.ndarray:
    out = np.empty(rows, dtype=np.float32)
    lib().orc_gemv_f32(quant, _ptr(W), _ptr(S), _ptr(h16(x)), rows, cols, _ptr(out))
    return out


def dequant(quant, W, S, rows, cols) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.float16)
    lib().orc_dequant(quant, _ptr(W), _ptr(S), rows, cols, _ptr(out))
    return out


def rmsnorm(x, w, eps=1e-6) -> np.ndarray:
    x, w = h16(x), h16(w)
    out = np.empty_like(x)
    lib().orc_rmsnorm(_ptr(x), _ptr(w), _ptr(out), x.size, F2H(eps))
    return out


def rope(q, k, n_heads, n_kv, hd, pos, theta=1e6):
    q, k = h16(q).copy(), h16(k).copy()
    lib().orc_rope(_ptr(q), _ptr(k), n_heads, n_kv, hd, pos, theta)
    return q, k


def qkv(quant, xn, Wq, Wk, Wv, Sq, Sk, Sv, bq, bk, bv, dim, q_dim, kv_dim):
    q, k, v = np.empty(q_dim, np.float16), np.empty(kv_dim, np.float16), np.empty(kv_dim, np.float16)
    lib().orc_qkv(quant, _ptr(h16(xn)), _ptr(Wq), _ptr(Wk), _ptr(Wv), _ptr(Sq), _ptr(Sk), _ptr(Sv), _ptr(h16(bq)), _ptr(h16(bk)), _ptr(h16(bv)),
                  _ptr(q), _ptr(k), _ptr(v), dim, q_dim, kv_dim)
    return q, k, v


def gemv_add(quant, W, S, inp, x, rows, cols) -> np.ndarray:
    x = h16(x).copy()
    lib().orc_gemv_add(quant, _ptr(W), _ptr(S), _ptr(h16(inp)), _ptr(x), rows, cols)
    return x


def mlp1(quant, xn, Wg, Wu, Sg, Su, dim, inter) -> np.ndarray:
    out = np.empty(inter, np.float16)
    lib().orc_mlp1(quant, _ptr(h16(xn)), _ptr(Wg), _ptr(Wu), _ptr(Sg), _ptr(Su), _ptr(out), dim, inter)
    return out


def logits(quant, W, S, xn, vocab, dim) -> np.ndarray:
    out = np.empty(vocab, np.float16)
    lib().orc_logits(quant, _ptr(W), _ptr(S), _ptr(h16(xn)), _ptr(out), vocab, dim)
    return out


def penalty(lg, hist, vocab, pen=1.1) -> np.ndarray:
    lg = h16(lg).copy()
    hist = np.ascontiguousarray(hist, dtype=np.int32)
    lib().orc_penalty(_ptr(lg), _ptr(hist), hist.size, vocab, F2H(pen))
    return lg


def argmax(lg) -> int:
    lg = h16(lg)
    return lib().orc_argmax(_ptr(lg), lg.size)


def attention(q, K, V, n_heads, n_kv, hd, max_seq, length, ref_rounding=False) -> np.ndarray:
    q, K, V = h16(q), h16(K), h16(V)
    out = np.empty(n_heads * hd, np.float16)
    fn = lib().orc_attention_ref if ref_rounding else lib().orc_attention_exact
    fn(_ptr(q), _ptr(K), _ptr(V), _ptr(out), n_heads, n_kv, hd, max_seq, length)
    return out


class OracleModel:
    """Whole-model oracle: loads the same .bin file and runs the scalar decode step."""

    def __init__(self, path: str, ctx_cap: int):
        err = C.create_string_buffer(256)
        self._h = lib().orc_load(str(path).encode(), ctx_cap, err, 256)
        if not self._h:
            raise RuntimeError(err.value.decode())
        d = (C.c_int * 10)()
        lib().orc_dims(self._h, d)
        (self.vocab, self.dim, self.inter, self.layers, self.heads, self.kv, self.hd, self.max_seq, self.quant, self.lm_fmt) = list(d)
        self.ctx_cap = ctx_cap

    def step(self, token, pos, history=None, ref_attention=False) -> int:
        h = np.ascontiguousarray(history if history is not None else [], dtype=np.int32)
        return lib().orc_step(self._h, token, pos, _ptr(h) if h.size else None, h.size, 1 if ref_attention else 0)

    def _view(self, p, n, dtype=np.float16):
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), shape=(n,)).view(dtype)

    @property
    def logits(self):
        return self._view(lib().orc_logits_ptr(self._h), self.vocab)

    @property
    def x(self):
        return self._view(lib().orc_x_ptr(self._h), self.dim)

    def kv_views(self):
        n = self.layers * self.kv * self.ctx_cap * self.hd
        shape = (self.layers, self.kv, self.ctx_cap, self.hd)
        return self._view(lib().orc_kcache(self._h), n).reshape(shape), self._view(lib().orc_vcache(self._h), n).reshape(shape)

    def close(self):
        if self._h:
            lib().orc_free(self._h)
            self._h = None

    def __del__(self):
        self.close()


# ---- the reference's own CUDA build (oracle/_ref) ----------------------------------------------------------------------

def ref_lib_path(model: str, quant: str, tuned: bool = False) -> Path:
    return HERE / "_ref" / f"libcuqwen_ref_{model.replace('.', '_')}_{quant}{'_tuned' if tuned else ''}.so"


_ref_cache = {}


def ref_lib(model: str, quant: str, tuned: bool = False):
    """The reference compiled for (model, quant), or None when oracle/_ref was not built.  tuned: the build with the
    reference's own large-GPU launch constants (oracle/build_ref.py)."""
    key = (model, quant, tuned)
    if key not in _ref_cache:
        p = ref_lib_path(model, quant, tuned)
        if not p.exists():
            _ref_cache[key] = None
        else:
            r = C.CDLL(str(p))
            sig = {
                "ref_info": (None, [_vp]), "ref_sync": (_i, []), "ref_embedding": (None, [_vp, _vp, _vp, _i]),
                "ref_rmsnorm": (None, [_vp, _vp, _vp, _i, _f]),
                "ref_qkv": (None, [_vp] * 13 + [_i, _i, _i, _i, _vp, _f]), "ref_kv_store": (None, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
                "ref_attention": (None, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp]),
                "ref_gemv_add": (None, [_vp, _vp, _vp, _vp, _i, _i]), "ref_mlp1": (None, [_vp] * 6 + [_i, _i]),
                "ref_mlp2": (None, [_vp, _vp, _vp, _vp, _i, _i]), "ref_logits": (None, [_vp, _vp, _vp, _i, _i]),
                "ref_logits_int8": (None, [_vp, _vp, _vp, _vp, _i, _i]), "ref_penalty": (None, [_vp, _vp, _vp, _i, _f]),
                "ref_argmax": (None, [_vp, _vp, _i]), "ref_model_load": (_vp, [C.c_char_p]), "ref_lm_head_quantized": (_i, [_vp]),
                "ref_forward": (_i, [_vp, _i, _i, _vp, _i]), "ref_decode_n": (_f, [_vp, _i, _i, _i, _vp]),
                "ref_bench_attention": (_f, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _i]),
                "ref_bench_gemv_add": (_f, [_vp, _vp, _i, _vp, _vp, _i, _i, _i]),
                "ref_kv_fill_normal": (None, [_vp, _i, C.c_ulonglong]), "ref_state_ptr": (_vp, [_vp, _i]), "ref_model_free": (None, [_vp]),
            }
            for n, (res, args) in sig.items():
                fn = getattr(r, n)
                fn.restype, fn.argtypes = res, args
            _ref_cache[key] = r
    return _ref_cache[key]
