"""ctypes binding of ``libcuqwen_b200.so`` (declared in ``include/cuqwen_b200.h``).

Loading fails loudly when the library has not been built: there is no CPU or
PyTorch fallback for any entry point.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libcuqwen_b200.so"


class Params(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "model_id", "vocab_size", "dim", "intermediate_size", "n_layers", "n_heads", "n_kv_heads", "head_dim",
        "max_seq_len", "quant", "device", "tp_rank", "tp_size", "attn_splits")] + [
        ("flags", C.c_uint32), ("norm_eps", C.c_float), ("rope_theta", C.c_float), ("repetition_penalty", C.c_float)]


_vp, _i, _f, _sz, _l = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_long
_pi = C.POINTER(C.c_int)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "cuqwen_model_params": (_i, [_i, _i, C.POINTER(Params)]),
    "cuqwen_create": (_i, [C.POINTER(Params), C.POINTER(_vp)]),
    "cuqwen_destroy": (None, [_vp]),
    "cuqwen_load": (_i, [_vp, C.c_char_p]),
    "cuqwen_step": (_i, [_vp, _i, _i, _pi, _i, _pi]),
    "cuqwen_decode_n": (_i, [_vp, _i, _i, _i, _pi]),
    "cuqwen_step_loop": (_i, [_vp, _i, _i, _i, _pi]),
    "cuqwen_prefill": (_i, [_vp, _pi, _i, _i]),
    "cuqwen_last_decode_ms": (_f, [_vp]),
    "cuqwen_kv_fill_normal": (_i, [_vp, _i, C.c_uint64]),
    "cuqwen_tp_init": (_i, [_vp, _vp, _sz]),
    "cuqwen_nccl_unique_id": (_i, [_vp, _sz]),
    "cuqwen_tp_plan": (_i, [_i] * 7 + [_pi]),
    "cuqwen_get_ptr": (_i, [_vp, _i, _i, C.POINTER(_vp), C.POINTER(_sz)]),
    "cuqwen_lm_head_kind": (_i, [_vp]),
    "cuqwen_get_params": (_i, [_vp, C.POINTER(Params)]),
    "cuqwen_step_bytes": (C.c_uint64, [_vp, _i]),
    "cuqwen_step_launches": (_i, [_vp]),
    "cuqwen_step_profile": (_i, [_vp, _i, _i, C.POINTER(C.c_float), _i, C.POINTER(_i)]),
    "cuqwen_dev_alloc": (_i, [_i, _sz, C.POINTER(_vp)]),
    "cuqwen_dev_sm_count": (_i, [_i, _pi]),
    "cuqwen_dev_free": (_i, [_i, _vp]),
    "cuqwen_dev_upload": (_i, [_i, _vp, _vp, _sz]),
    "cuqwen_dev_download": (_i, [_i, _vp, _vp, _sz]),
    "cuqwen_dev_memset": (_i, [_i, _vp, _i, _sz]),
    "cuqwen_dev_sync": (_i, [_i]),
    "cuqwen_dev_join": (_i, [_i, _vp, _i]),
    "cuqwen_capture_begin": (_i, [_i]),
    "cuqwen_capture_replay": (_i, [_i, _i, C.POINTER(_f)]),
    "cuqwen_bench_begin": (_i, [_i]),
    "cuqwen_bench_end": (_i, [_i, C.POINTER(_f)]),
    "cuqwen_k_embedding": (_i, [_i, _vp, _vp, _vp, _i]),
    "cuqwen_k_rmsnorm": (_i, [_i, _vp, _vp, _vp, _i, _f]),
    "cuqwen_k_qkv": (_i, [_i, _i, _vp, _vp, _f] + [_vp] * 14 + [_i] * 5 + [_vp, _f, _i]),
    "cuqwen_k_rope": (_i, [_i, _vp, _vp, _i, _i, _i, _vp, _f, _i]),
    "cuqwen_k_kv_store": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "cuqwen_k_attention": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "cuqwen_k_attention_kv8": (_i, [_i] + [_vp] * 9 + [_i] * 5 + [_vp, _vp]),
    "cuqwen_k_attention_static": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "cuqwen_k_attention_static_status": (_i, [_i, _vp, C.POINTER(C.c_uint)]),
    "cuqwen_k_tp_sum": (_i, [_i, _vp, _vp, _vp, _i, _i, _vp, _i, C.c_longlong]),
    "cuqwen_attn_scratch_bytes": (_i, [_i, _i, _i, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]),
    "cuqwen_k_gemv_add": (_i, [_i, _i, _vp, _vp, _vp, _vp, _i, _i]),
    "cuqwen_k_prefill_attention": (_i, [_i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i]),
    "cuqwen_k_prefill_gemm": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "cuqwen_k_gemv": (_i, [_i, _i, _vp, _vp, _vp, _vp, _f, _vp, _i, _i]),
    "cuqwen_k_gemv_f32": (_i, [_i, _i, _vp, _vp, _vp, _vp, _i, _i]),
    "cuqwen_k_mlp1": (_i, [_i, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "cuqwen_k_penalty": (_i, [_i, _vp, _vp, _vp, _i, _f, _vp]),
    "cuqwen_k_argmax": (_i, [_i, _vp, _vp, _i, _vp]),
    "cuqwen_k_dequant": (_i, [_i, _i, _vp, _vp, _vp, _l, _l]),
    "cuqwen_strerror": (C.c_char_p, [_i]),
    "cuqwen_last_error": (C.c_char_p, []),
}

_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; raise if it is missing (no fallback path exists)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cuqwen_b200.build` (nvcc, sm_100a). "
                "This package has no CPU or PyTorch fallback.")
        l = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


class CuQwenError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"cuqwen error {code}: {msg}")
        self.code = code


def check(code: int) -> None:
    if code != 0:
        raise CuQwenError(code, lib().cuqwen_last_error().decode(errors="replace"))
