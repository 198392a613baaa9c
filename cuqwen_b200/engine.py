"""Python mirror of the host API over the C ABI.

The reference's host API is C++ (``load_weights`` / ``malloc_qwen_state`` /
``qwen_forward`` / ``launch_*``, CuQwen include/*.h); the same calls exist here
as ``Engine.load`` / ``Engine()`` / ``Engine.step`` and the functions in
``kernels``.  Nothing here computes: every method forwards to
``libcuqwen_b200.so``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _abi
from ._abi import Params, check

FP16, INT8, INT4 = 0, 1, 2
QUANT_ID = {"fp16": FP16, "int8": INT8, "int4": INT4}
MODEL_ID = {"0.5b": 0, "1.5b": 1, "3b": 2, "7b": 3, "14b": 4}
FLAG_ACCURATE_ROPE, FLAG_NO_PDL, FLAG_NO_GRAPH, FLAG_STEP_TRACE, FLAG_TP_NCCL, FLAG_NO_HANDOVER, FLAG_KV_INT8, FLAG_TP_SUM_IN_GEMV, FLAG_PREFILL_ATTN_MMA = 1, 2, 4, 16, 32, 64, 128, 256, 512

# cuqwen_get_ptr ids (include/cuqwen_b200.h)
PTR = dict(X=0, XN=1, Q=2, K=3, V=4, ATT=5, GATE=6, LOGITS=7, KEY_CACHE=8, VALUE_CACHE=9, HISTORY=10, STEP_TRACE=11, TOKEN=12, POS=13,
           HISTORY_LEN=14, SAMPLED=15, PARTIAL_O=16, PARTIAL_ML=17, UP=18, MLP_OUT=19, STREAM=20, KEY_SCALE=21, VALUE_SCALE=22,
           EMBED=32, NORM=33, LM_HEAD=34, LM_HEAD_SCALE=35,
           IN_NORM=64, WQ=65, SQ=66, BQ=67, WK=68, SK=69, BK=70, WV=71, SV=72, BV=73, WO=74, SO=75, POST_NORM=76,
           WGATE=77, SGATE=78, WUP=79, SUP=80, WDOWN=81, SDOWN=82)


class DevBuf:
    """A device allocation owned through the C ABI (no torch involved)."""

    def __init__(self, nbytes: int, device: int = 0, zero: bool = True):
        self.device, self.nbytes = device, int(nbytes)
        p = C.c_void_p()
        check(_abi.lib().cuqwen_dev_alloc(device, self.nbytes, C.byref(p)))
        self.ptr = p.value
        if zero:
            check(_abi.lib().cuqwen_dev_memset(device, self.ptr, 0, self.nbytes))

    @classmethod
    def from_numpy(cls, a: np.ndarray, device: int = 0) -> "DevBuf":
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes, device, zero=False)
        check(_abi.lib().cuqwen_dev_upload(device, b.ptr, a.ctypes.data, a.nbytes))
        return b

    def upload(self, a: np.ndarray, offset: int = 0) -> None:
        a = np.ascontiguousarray(a)
        assert offset + a.nbytes <= self.nbytes
        check(_abi.lib().cuqwen_dev_upload(self.device, self.ptr + offset, a.ctypes.data, a.nbytes))

    def numpy(self, dtype, count: int | None = None, offset: int = 0) -> np.ndarray:
        dt = np.dtype(dtype)
        n = (self.nbytes - offset) // dt.itemsize if count is None else count
        out = np.empty(n, dtype=dt)
        check(_abi.lib().cuqwen_dev_download(self.device, out.ctypes.data, self.ptr + offset, out.nbytes))
        return out

    def zero(self) -> None:
        check(_abi.lib().cuqwen_dev_memset(self.device, self.ptr, 0, self.nbytes))

    def free(self) -> None:
        if self.ptr:
            _abi.lib().cuqwen_dev_free(self.device, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def download(device: int, ptr: int, dtype, count: int) -> np.ndarray:
    out = np.empty(count, dtype=np.dtype(dtype))
    check(_abi.lib().cuqwen_dev_download(device, out.ctypes.data, ptr, out.nbytes))
    return out


def sm_count(device: int = 0) -> int:
    n = C.c_int(0)
    check(_abi.lib().cuqwen_dev_sm_count(device, C.byref(n)))
    return n.value


def sync(device: int = 0) -> None:
    check(_abi.lib().cuqwen_dev_sync(device))


def model_params(model: str | int, quant: str | int) -> Params:
    p = Params()
    mid = MODEL_ID[model] if isinstance(model, str) else model
    q = QUANT_ID[quant] if isinstance(quant, str) else quant
    check(_abi.lib().cuqwen_model_params(mid, q, C.byref(p)))
    return p


def custom_params(vocab, dim, inter, layers, heads, kv, hd, quant, max_seq_len=32768) -> Params:
    p = Params()
    p.model_id = -1
    p.vocab_size, p.dim, p.intermediate_size, p.n_layers = vocab, dim, inter, layers
    p.n_heads, p.n_kv_heads, p.head_dim = heads, kv, hd
    p.max_seq_len = max_seq_len
    p.quant = QUANT_ID[quant] if isinstance(quant, str) else quant
    p.tp_size = 1
    return p


class Engine:
    """malloc_qwen_state + load_weights + qwen_forward behind one object."""

    def __init__(self, params: Params):
        self._h = C.c_void_p()
        check(_abi.lib().cuqwen_create(C.byref(params), C.byref(self._h)))
        self.params = Params()
        check(_abi.lib().cuqwen_get_params(self._h, C.byref(self.params)))
        self.device = self.params.device

    def close(self) -> None:
        if self._h:
            _abi.lib().cuqwen_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load(self, path: str) -> None:
        check(_abi.lib().cuqwen_load(self._h, str(path).encode()))

    def tp_init(self, unique_id: bytes) -> None:
        buf = C.create_string_buffer(unique_id, len(unique_id))
        check(_abi.lib().cuqwen_tp_init(self._h, buf, len(unique_id)))

    def step(self, token: int, pos: int, history=None) -> int:
        out = C.c_int(0)
        if history is not None and len(history):
            h = np.ascontiguousarray(history, dtype=np.int32)
            check(_abi.lib().cuqwen_step(self._h, token, pos, h.ctypes.data_as(C.POINTER(C.c_int)), len(h), C.byref(out)))
        else:
            check(_abi.lib().cuqwen_step(self._h, token, pos, None, 0, C.byref(out)))
        return out.value

    def decode_n(self, first_token: int, start_pos: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.int32)
        check(_abi.lib().cuqwen_decode_n(self._h, first_token, start_pos, n, out.ctypes.data_as(C.POINTER(C.c_int))))
        return out

    def step_loop(self, first_token: int, start_pos: int, n: int) -> np.ndarray:
        """cuqwen_step_loop: n calls of cuqwen_step in a C loop, each token making the host round trip."""
        out = np.empty(n, dtype=np.int32)
        check(_abi.lib().cuqwen_step_loop(self._h, first_token, start_pos, n, out.ctypes.data_as(C.POINTER(C.c_int))))
        return out

    def prefill(self, tokens, pos0: int = 0) -> None:
        """cuqwen_prefill: the KV cache rows [pos0, pos0 + len(tokens)) of these prompt tokens, computed as batched tiles."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        check(_abi.lib().cuqwen_prefill(self._h, t.ctypes.data_as(C.POINTER(C.c_int)), int(t.size), pos0))

    @property
    def last_decode_ms(self) -> float:
        return float(_abi.lib().cuqwen_last_decode_ms(self._h))

    def kv_fill_normal(self, ctx_len: int, seed: int) -> None:
        check(_abi.lib().cuqwen_kv_fill_normal(self._h, ctx_len, seed))

    def ptr(self, which: str, layer: int = 0) -> tuple[int, int]:
        p, n = C.c_void_p(), C.c_size_t()
        check(_abi.lib().cuqwen_get_ptr(self._h, PTR[which], layer, C.byref(p), C.byref(n)))
        return (p.value or 0), n.value

    def read(self, which: str, dtype=np.float16, layer: int = 0, count: int | None = None, offset: int = 0) -> np.ndarray:
        p, n = self.ptr(which, layer)
        dt = np.dtype(dtype)
        c = (n - offset) // dt.itemsize if count is None else count
        return download(self.device, p + offset, dt, c)

    def write(self, which: str, a: np.ndarray, layer: int = 0, offset: int = 0) -> None:
        p, n = self.ptr(which, layer)
        a = np.ascontiguousarray(a)
        assert offset + a.nbytes <= n
        check(_abi.lib().cuqwen_dev_upload(self.device, p + offset, a.ctypes.data, a.nbytes))

    @property
    def lm_head_kind(self) -> int:
        return _abi.lib().cuqwen_lm_head_kind(self._h)

    def step_bytes(self, ctx: int) -> int:
        return int(_abi.lib().cuqwen_step_bytes(self._h, ctx))

    def profile_step(self, token: int, pos: int) -> np.ndarray:
        """Microseconds between consecutive launches of one step run launch by launch (cuqwen_step_profile)."""
        buf = (C.c_float * 4096)()
        n = C.c_int(0)
        check(_abi.lib().cuqwen_step_profile(self._h, token, pos, buf, 4096, C.byref(n)))
        return np.array(buf[:n.value], dtype=np.float32)

    @property
    def step_launches(self) -> int:
        return _abi.lib().cuqwen_step_launches(self._h)


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    check(_abi.lib().cuqwen_nccl_unique_id(buf, 128))
    return buf.raw
