"""The allocation-free attention entry point against the ordinary one.

Collected last (file name) so that it runs after every other GPU test has used the library, and it also passes alone.
Both entry points are called through the C ABI on identical device buffers; the static one twice in a row, because
its scratch block is reused from call to call and must come back clean.
"""
from __future__ import annotations

import ctypes
import ctypes.util

import numpy as np
import pytest

from cuqwen_b200 import _abi
from cuqwen_b200 import kernels as K
from cuqwen_b200.engine import DevBuf, sync
from gpu_util import close, dev, dint, report
from oracle import oracle_py as O

pytestmark = pytest.mark.gpu


def _device_sync():
    # The static entry point queues on a caller-chosen stream (here the CUDA default stream), which the library's own
    # stream does not order with: wait for the whole device through the runtime the library is linked against.
    rt = ctypes.CDLL(_cudart_name())
    assert rt.cudaDeviceSynchronize() == 0


def _cudart_name() -> str:
    """The CUDA runtime the library itself is linked against (its NEEDED entry, resolved by the loader because the
    library is already mapped), else whatever the system's search path offers."""
    lib_path = str(_abi.LIB_PATH)
    with open("/proc/self/maps") as f:
        for line in f:
            if "libcudart" in line:
                return line.split()[-1]
    _abi.lib()
    with open("/proc/self/maps") as f:
        for line in f:
            if "libcudart" in line:
                return line.split()[-1]
    name = ctypes.util.find_library("cudart")
    assert name, f"no CUDA runtime found for {lib_path}"
    return name


def _status() -> int:
    code = ctypes.c_uint(123)
    rc = _abi.lib().cuqwen_k_attention_static_status(0, None, ctypes.byref(code))
    assert rc == 0, _abi.lib().cuqwen_last_error()
    return code.value


def _case(nh, nkv, hd, length, nsplit, seed):
    rng = np.random.default_rng(seed)
    max_seq = length + 19
    q = rng.standard_normal((nh, hd)).astype(np.float16)
    Kc = rng.standard_normal((nkv, max_seq, hd)).astype(np.float16)
    Vc = rng.standard_normal((nkv, max_seq, hd)).astype(np.float16)
    Kc[:, length:] = np.float16(np.nan); Vc[:, length:] = np.float16(np.nan)
    return q, Kc, Vc, max_seq


@pytest.mark.parametrize("nh,nkv,hd,length,nsplit", [(28, 4, 128, 777, 37), (14, 2, 64, 100, 74), (40, 8, 128, 2048, 18), (12, 2, 128, 1, 5)])
def test_static_scratch_attention_matches_the_allocating_entry(built, nh, nkv, hd, length, nsplit):
    q, Kc, Vc, max_seq = _case(nh, nkv, hd, length, nsplit, seed=nh * 1000 + length)
    dq, dk, dv, dp = dev(q), dev(Kc), dev(Vc), dint(length - 1)

    bo, bml, bc = K.attn_scratch_bytes(nkv, hd, nsplit)
    so, sml, cnt = DevBuf(bo), DevBuf(bml), DevBuf(bc)
    want_buf = DevBuf(nh * hd * 2)
    K.gqa_attention_decode(dq, dk, dv, want_buf, dp, nh, nkv, hd, max_seq, nsplit, so, sml, cnt)
    want = want_buf.numpy(np.float16)
    assert np.isfinite(want.astype(np.float32)).all()
    exact = O.attention(q, Kc, Vc, nh, nkv, hd, max_seq, length)          # the CPU oracle: softmax(q K^T / sqrt(hd)) V in fp32

    for call in range(2):
        out = DevBuf(nh * hd * 2)                  # zeroed on the library's stream ...
        sync()                                     # ... which the default stream does not wait for
        K.gqa_attention_decode_static(dq, dk, dv, out, dp, nh, nkv, hd, max_seq, nsplit)
        _device_sync()
        got = out.numpy(np.float16)
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), f"call {call}: static-scratch result differs"
        assert close(got, exact), f"call {call}: " + report(got, exact)
        assert _status() == 0, "a bounded wait ran out inside the static-scratch kernels"


def test_static_scratch_attention_rejects_shapes_beyond_its_block(built):
    nh, nkv, hd, length = 64, 8, 128, 64
    q, Kc, Vc, max_seq = _case(nh, nkv, hd, length, 128, seed=5)
    dq, dk, dv, dp, out = dev(q), dev(Kc), dev(Vc), dint(length - 1), DevBuf(nh * hd * 2)
    lib = _abi.lib()
    # 8 KV heads x 128 splits needs 8 * (128 + 16) = 1152 partial slots; the block holds 384
    rc = lib.cuqwen_k_attention_static(0, None, dq.ptr, dk.ptr, dv.ptr, out.ptr, dp.ptr, nh, nkv, hd, max_seq, 128)
    assert rc == 1 and b"fixed scratch" in lib.cuqwen_last_error()
    rc = lib.cuqwen_k_attention_static(0, None, dq.ptr, dk.ptr, dv.ptr, out.ptr, dp.ptr, nh, nkv, 96, max_seq, 8)
    assert rc == 1
    rc = lib.cuqwen_k_attention_static(0, None, None, dk.ptr, dv.ptr, out.ptr, dp.ptr, nh, nkv, hd, max_seq, 8)
    assert rc == 1
