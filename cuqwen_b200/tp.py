"""Host-side view of the tensor-parallel partition the engine applies (csrc/tp_plan.h through cuqwen_tp_plan).

Column-parallel: q/k/v projections (whole heads), gate/up (128-column groups of the MLP width), lm_head (16-row
tiles of the vocabulary).  Row-parallel: o_proj and down_proj, whose partial sums are added across ranks.  With
more ranks than KV heads the ranks that share a KV head split its query heads and each keeps that head's K and V.
The reference is single-GPU (its whole model sits in one QwenWeights, include/load_weights.h:17-54); this is the
multi-GPU extension of the same layouts.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _abi


@dataclass(frozen=True)
class Plan:
    q0: int
    q1: int          # query heads [q0, q1)
    kv0: int
    kv1: int         # KV heads [kv0, kv1) stored on this rank
    q_per_kv: int    # query heads per stored KV head on this rank
    i0: int
    i1: int          # MLP columns [i0, i1)
    v0: int
    v1: int          # vocabulary rows [v0, v1)


def plan(cfg: dict, rank: int, size: int) -> Plan:
    out = (C.c_int * 9)()
    _abi.check(_abi.lib().cuqwen_tp_plan(cfg["heads"], cfg["kv"], cfg["hd"], cfg["inter"], cfg["vocab"], rank, size, out))
    return Plan(*list(out))


def shard_tensors(t: dict, cfg: dict, p: Plan) -> dict:
    """The slice of a full tensor dict (names as in the HF checkpoint / binfmt.random_tensors) that rank `p` holds."""
    hd = cfg["hd"]
    qs, ks = slice(p.q0 * hd, p.q1 * hd), slice(p.kv0 * hd, p.kv1 * hd)
    out = {}
    for name, a in t.items():
        if ".q_proj." in name:
            out[name] = a[qs]
        elif ".k_proj." in name or ".v_proj." in name:
            out[name] = a[ks]
        elif name.endswith("o_proj.weight"):
            out[name] = a[:, qs]
        elif name.endswith("gate_proj.weight") or name.endswith("up_proj.weight"):
            out[name] = a[p.i0:p.i1]
        elif name.endswith("down_proj.weight"):
            out[name] = a[:, p.i0:p.i1]
        elif name == "lm_head.weight":
            out[name] = a[p.v0:p.v1]
        else:
            out[name] = a          # norms and the embedding are replicated
    return {k: np.ascontiguousarray(v) for k, v in out.items()}


def pack_argmax_key(value: float, index: int) -> int:
    """(order-preserving key of the fp32 value) << 32 | ~index: the maximum over ranks picks the largest value and,
    among equals, the smallest global index — what every rank's sampler contributes to the all-gather."""
    bits = int(np.float32(value).view(np.uint32))
    key = bits ^ 0xFFFFFFFF if bits & 0x80000000 else bits | 0x80000000
    return (key << 32) | (~index & 0xFFFFFFFF)


def unpack_argmax_index(packed: int) -> int:
    return ~packed & 0xFFFFFFFF
