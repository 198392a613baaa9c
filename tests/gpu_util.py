"""Helpers shared by the GPU parity tests: device buffers through the C ABI, seeded inputs, comparisons."""
from __future__ import annotations

import numpy as np

from cuqwen_b200 import binfmt
from cuqwen_b200.engine import DevBuf, sync

RTOL, ATOL = 2e-3, 1e-2      # parity contract for fp16 outputs: 2e-3 relative or 1e-2 absolute
EPS_H = float(np.float16(1e-6))


def dev(a) -> DevBuf:
    return DevBuf.from_numpy(np.ascontiguousarray(a))


def dint(v: int) -> DevBuf:
    return dev(np.array([v], dtype=np.int32))


def close(got, want, rtol=RTOL, atol=ATOL):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    bad = np.abs(got - want) > atol + rtol * np.abs(want)
    return not bad.any()


def report(got, want) -> str:
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = np.abs(got - want)
    return f"max abs {d.max():.3e}, max rel {(d / (np.abs(want) + 1e-6)).max():.3e}"


def quant_mats(rng, rows, cols, quant, full_range=True, sigma=0.02):
    """Device-format weights and scales for one projection.  full_range: integers uniform over the whole
    two's-complement range with scales U(0.002, 0.02) (benchmark config 1); otherwise N(0, sigma) quantised the
    way the exporter does."""
    if quant == 0:
        return np.ascontiguousarray((sigma * rng.standard_normal((rows, cols))).astype(np.float16)), None
    if full_range:
        lo, hi = (-8, 7) if quant == 2 else (-128, 127)
        q = rng.integers(lo, hi + 1, size=(rows, cols)).astype(np.int8)
        s = rng.uniform(0.002, 0.02, size=(rows, cols // 128)).astype(np.float16)
    else:
        q, s = binfmt.quantize_groupwise((sigma * rng.standard_normal((rows, cols))).astype(np.float32), 7 if quant == 2 else 127)
    w = binfmt.pack_int4(q) if quant == 2 else q
    return np.ascontiguousarray(w), np.ascontiguousarray(s)


class Pool:
    """Uploads arrays and keeps the device buffers alive until the pool goes away; returns raw pointers."""

    def __init__(self):
        self.keep = []

    def p(self, a):
        if a is None:
            return None
        b = a if isinstance(a, DevBuf) else dev(a)
        self.keep.append(b)
        return b.ptr


QNAME = {0: "fp16", 1: "int8", 2: "int4"}

__all__ = ["dev", "dint", "close", "report", "quant_mats", "sync", "DevBuf", "RTOL", "ATOL", "EPS_H", "QNAME", "Pool"]
