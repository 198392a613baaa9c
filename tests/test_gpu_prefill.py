"""Batched-token prefill (no counterpart in the reference, which prefills token by token through the decode path,
src/main.cu:86-92; README.md:145 names the batched form as future work).

Kernel level: cuqwen_k_prefill_gemm (tcgen05 GEMM over a tile of tokens) against a float64 product of the same fp16
inputs and de-quantised weights, tolerance 2e-3 relative / 1e-2 absolute as for the decode GEMV."""
import numpy as np
import pytest

from cuqwen_b200 import binfmt
from cuqwen_b200 import kernels as K
from tests.gpu_util import DevBuf, close, dev, quant_mats, report, sync

pytestmark = pytest.mark.gpu


def dequant(w, s, quant, cols):
    if quant == 0:
        return w.astype(np.float64)
    q = binfmt.unpack_int4(w, cols) if quant == 2 else w
    return q.astype(np.float64) * np.repeat(s.astype(np.float64), 128, axis=1)


@pytest.mark.parametrize("quant", [2, 1, 0])
@pytest.mark.parametrize("T,R,Kc", [(1, 256, 128), (37, 512, 896), (128, 576, 3584), (300, 1024, 1536), (257, 264, 256)])
def test_prefill_gemm_plain_modes(built, quant, T, R, Kc):
    rng = np.random.default_rng(T * 131 + R + quant)
    x = rng.standard_normal((T, Kc)).astype(np.float16)
    w, s = quant_mats(rng, R, Kc, quant, full_range=False, sigma=0.05)
    want = x.astype(np.float64) @ dequant(w, s, quant, Kc).T
    dx, dw, ds = dev(x), dev(w), (dev(s) if s is not None else None)
    # fp32 output
    out = DevBuf(T * R * 4)
    K.prefill_gemm(quant, K.PF_OUT_F32, dx, dw, ds, out, T, R, Kc)
    sync()
    got = out.numpy(np.float32).reshape(T, R)
    assert close(got, want), "f32: " + report(got, want)
    # fp16 output with bias, into a wider row (out_stride > rows); the columns beside it stay untouched
    bias = rng.standard_normal(R).astype(np.float16)
    stride = R + 64
    canvas = np.full((T, stride), 7.0, np.float16)
    out = dev(canvas)
    K.prefill_gemm(quant, K.PF_OUT_F16, dx, dw, ds, out, T, R, Kc, out_stride=stride, bias=dev(bias))
    sync()
    got = out.numpy(np.float16).reshape(T, stride)
    assert close(got[:, :R], want + bias.astype(np.float64)), "f16+bias: " + report(got[:, :R], want + bias.astype(np.float64))
    assert (got[:, R:] == np.float16(7.0)).all()
    # residual add in place
    res = rng.standard_normal((T, R)).astype(np.float16)
    out = dev(res)
    K.prefill_gemm(quant, K.PF_RESID, dx, dw, ds, out, T, R, Kc)
    sync()
    got = out.numpy(np.float16).reshape(T, R)
    assert close(got, want + res.astype(np.float64)), "resid: " + report(got, want + res.astype(np.float64))


@pytest.mark.parametrize("quant", [2, 1, 0])
@pytest.mark.parametrize("T,R,Kc", [(5, 128, 256), (130, 320, 896), (256, 1024, 1536)])
def test_prefill_gemm_swiglu(built, quant, T, R, Kc):
    rng = np.random.default_rng(T + R * 3 + quant)
    x = rng.standard_normal((T, Kc)).astype(np.float16)
    wg, sg = quant_mats(rng, R, Kc, quant, full_range=False, sigma=0.05)
    wu, su = quant_mats(rng, R, Kc, quant, full_range=False, sigma=0.05)
    g = x.astype(np.float64) @ dequant(wg, sg, quant, Kc).T
    u = x.astype(np.float64) @ dequant(wu, su, quant, Kc).T
    want = g / (1.0 + np.exp(-g)) * u
    out = DevBuf(T * R * 2)
    K.prefill_gemm(quant, K.PF_SWIGLU, dev(x), dev(wg), dev(sg) if sg is not None else None, out, T, R, Kc,
                   w1=dev(wu), s1=dev(su) if su is not None else None)
    sync()
    got = out.numpy(np.float16).reshape(T, R)
    assert close(got, want), report(got, want)
