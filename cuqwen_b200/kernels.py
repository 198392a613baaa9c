"""The reference's ``launch_*`` operators (CuQwen include/kernels.cuh:19-160) with run-time dims.

Arguments are device pointers (ints or ``DevBuf``); every function queues work
on the library's per-device stream and returns; ``engine.sync()`` waits.
"""
from __future__ import annotations

import ctypes as C

from . import _abi
from ._abi import check
from .engine import DevBuf


def _p(b):
    if b is None:
        return None
    return b.ptr if isinstance(b, DevBuf) else int(b)


def embedding_lookup(table, d_token, out, dim, device=0):
    check(_abi.lib().cuqwen_k_embedding(device, _p(table), _p(d_token), _p(out), dim))


def rmsnorm(x, weight, out, dim, eps, device=0):
    check(_abi.lib().cuqwen_k_rmsnorm(device, _p(x), _p(weight), _p(out), dim, eps))


def fused_attn_block(quant, x, wq, wk, wv, sq, sk, sv, bq, bk, bv, q_out, k_out, v_out, dim, n_heads, n_kv_heads, head_dim,
                     d_pos, rope_theta=1e6, rope_fast=1, norm_weight=None, eps=0.0, kcache=None, vcache=None, max_seq_len=0, device=0):
    check(_abi.lib().cuqwen_k_qkv(device, quant, _p(x), _p(norm_weight), eps, _p(wq), _p(wk), _p(wv), _p(sq), _p(sk), _p(sv),
                                  _p(bq), _p(bk), _p(bv), _p(q_out), _p(k_out), _p(v_out), _p(kcache), _p(vcache),
                                  dim, n_heads, n_kv_heads, head_dim, max_seq_len, _p(d_pos), rope_theta, rope_fast))


def rope(q, k, n_heads, n_kv_heads, head_dim, d_pos, rope_theta=1e6, rope_fast=1, device=0):
    check(_abi.lib().cuqwen_k_rope(device, _p(q), _p(k), n_heads, n_kv_heads, head_dim, _p(d_pos), rope_theta, rope_fast))


def kv_cache_store(k, v, kcache, vcache, d_pos, n_kv_heads, max_seq_len, head_dim, device=0):
    check(_abi.lib().cuqwen_k_kv_store(device, _p(k), _p(v), _p(kcache), _p(vcache), _p(d_pos), n_kv_heads, max_seq_len, head_dim))


def attn_scratch_bytes(n_kv_heads, head_dim, n_splits):
    a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
    check(_abi.lib().cuqwen_attn_scratch_bytes(n_kv_heads, head_dim, n_splits, C.byref(a), C.byref(b), C.byref(c)))
    return a.value, b.value, c.value


def gqa_attention_decode(q, kcache, vcache, out, d_pos, n_heads, n_kv_heads, head_dim, max_seq_len, n_splits,
                         scratch_o, scratch_ml, counters, device=0):
    check(_abi.lib().cuqwen_k_attention(device, _p(q), _p(kcache), _p(vcache), _p(out), _p(d_pos), n_heads, n_kv_heads, head_dim,
                                        max_seq_len, n_splits, _p(scratch_o), _p(scratch_ml), _p(counters)))


def gqa_attention_decode_kv8(q, kcache8, vcache8, kscale, vscale, k_cur, v_cur, out, d_pos, n_heads, n_kv_heads, head_dim, max_seq_len, n_splits,
                             scratch_o, scratch_ml, device=0):
    """cuqwen_k_attention_kv8: int8 caches with fp32 row scales; also stores the step's own key / value into row *d_pos."""
    check(_abi.lib().cuqwen_k_attention_kv8(device, _p(q), _p(kcache8), _p(vcache8), _p(kscale), _p(vscale), _p(k_cur), _p(v_cur), _p(out), _p(d_pos),
                                            n_heads, n_kv_heads, head_dim, max_seq_len, n_splits, _p(scratch_o), _p(scratch_ml)))


def gqa_attention_decode_static(q, kcache, vcache, out, d_pos, n_heads, n_kv_heads, head_dim, max_seq_len, n_splits,
                                stream=None, device=0):
    """cuqwen_k_attention_static: same result as gqa_attention_decode, scratch inside the library (no allocation).
    Queued on `stream` (a cudaStream_t value; None = the CUDA default stream); the caller synchronises."""
    check(_abi.lib().cuqwen_k_attention_static(device, stream, _p(q), _p(kcache), _p(vcache), _p(out), _p(d_pos), n_heads, n_kv_heads,
                                               head_dim, max_seq_len, n_splits))


PF_OUT_F16, PF_OUT_F32, PF_RESID, PF_SWIGLU = 0, 1, 2, 3


def prefill_gemm(quant, mode, x, w0, s0, out, n_tokens, rows, cols, out_stride=None, w1=None, s1=None, bias=None, device=0):
    """cuqwen_k_prefill_gemm: out[t][r] = x[t] . W[r] for n_tokens rows at once on the tcgen05 tensor cores."""
    check(_abi.lib().cuqwen_k_prefill_gemm(device, quant, mode, _p(x), _p(w0), _p(s0), _p(w1), _p(s1), _p(bias), _p(out), n_tokens, rows, cols,
                                           rows if out_stride is None else out_stride))


def prefill_attention(impl, q, kcache, vcache, out, n_tokens, pos0, n_heads, n_kv_heads, head_dim, max_seq_len, q_stride=None, device=0):
    """cuqwen_k_prefill_attention: causal attention of a tile of prompt tokens (impl 0 tcgen05, 1 mma.sync)."""
    check(_abi.lib().cuqwen_k_prefill_attention(device, impl, _p(q), _p(kcache), _p(vcache), _p(out), n_tokens, pos0, n_heads, n_kv_heads, head_dim,
                                                max_seq_len, n_heads * head_dim if q_stride is None else q_stride))


def gemv_add(quant, w, scale, inp, x_inout, rows, cols, device=0):
    check(_abi.lib().cuqwen_k_gemv_add(device, quant, _p(w), _p(scale), _p(inp), _p(x_inout), rows, cols))


def gemv(quant, w, scale, x, y, rows, cols, norm_weight=None, eps=0.0, device=0):
    check(_abi.lib().cuqwen_k_gemv(device, quant, _p(w), _p(scale), _p(x), _p(norm_weight), eps, _p(y), rows, cols))


def gemv_f32(quant, w, scale, x, y, rows, cols, device=0):
    check(_abi.lib().cuqwen_k_gemv_f32(device, quant, _p(w), _p(scale), _p(x), _p(y), rows, cols))


def fused_mlp_stage1(quant, x, wg, wu, sg, su, out, dim, inter, norm_weight=None, eps=0.0, device=0):
    check(_abi.lib().cuqwen_k_mlp1(device, quant, _p(x), _p(norm_weight), eps, _p(wg), _p(wu), _p(sg), _p(su), _p(out), dim, inter))


def apply_repetition_penalty(logits, d_history, d_history_len, vocab, penalty, bitmap, device=0):
    check(_abi.lib().cuqwen_k_penalty(device, _p(logits), _p(d_history), _p(d_history_len), vocab, penalty, _p(bitmap)))


def argmax(logits, d_token_out, vocab, scratch16, device=0):
    check(_abi.lib().cuqwen_k_argmax(device, _p(logits), _p(d_token_out), vocab, _p(scratch16)))


def dequant(quant, w, scale, out, rows, cols, device=0):
    check(_abi.lib().cuqwen_k_dequant(device, quant, _p(w), _p(scale), _p(out), rows, cols))


def bench_begin(device=0):
    check(_abi.lib().cuqwen_bench_begin(device))


def bench_end(device=0) -> float:
    ms = C.c_float()
    check(_abi.lib().cuqwen_bench_end(device, C.byref(ms)))
    return ms.value


def capture_begin(device=0):
    """From here until capture_replay the kernel calls above are recorded into a CUDA graph instead of running."""
    check(_abi.lib().cuqwen_capture_begin(device))


def capture_replay(replays: int, device=0) -> float:
    """Replays the recorded graph `replays` times between two CUDA events; returns milliseconds per replay."""
    ms = C.c_float()
    check(_abi.lib().cuqwen_capture_replay(device, replays, C.byref(ms)))
    return ms.value
