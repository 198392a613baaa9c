"""Capture outputs of the reference's own CUDA kernels (oracle/_ref, built from the unmodified CuQwen sources) on
seeded inputs, so the CPU oracle can be pinned against them where no GPU is present.

Run on a machine with a CUDA device after `python oracle/build_ref.py`:
    python tests/golden/make_ref_golden.py [OUT.npz]        (default: tests/golden/ref_kernels.npz)
Shapes are small on purpose: the file is committed.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from cuqwen_b200 import binfmt  # noqa: E402
from cuqwen_b200.engine import DevBuf  # noqa: E402
from oracle import oracle_py as O  # noqa: E402

out_path = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent / "ref_kernels.npz"
rng = np.random.default_rng(20251125)
res = {}
keep = []


def up(a):
    if a is None:
        return None
    b = DevBuf.from_numpy(np.ascontiguousarray(a))
    keep.append(b)
    return b.ptr


rows, cols = 64, 896          # mlp1: dim = cols, inter = rows
for quant, tag in ((0, "fp16"), (1, "int8"), (2, "int4")):
    ref = O.ref_lib("0.5b", tag)
    if ref is None:
        raise SystemExit("oracle/_ref is not built")

    def mat():
        if quant == 0:
            return (0.02 * rng.standard_normal((rows, cols))).astype(np.float16), None
        lo, hi = (-8, 7) if quant == 2 else (-128, 127)
        q = rng.integers(lo, hi + 1, size=(rows, cols)).astype(np.int8)
        s = rng.uniform(0.002, 0.02, size=(rows, cols // 128)).astype(np.float16)
        return (binfmt.pack_int4(q) if quant == 2 else q), s

    (w, s), (wg, sg), (wu, su) = mat(), mat(), mat()
    x = rng.standard_normal(cols).astype(np.float16)
    acc = DevBuf(rows * 2)
    ref.ref_gemv_add(up(w), up(s), up(x), acc.ptr, rows, cols)
    o = DevBuf(rows * 2)
    ref.ref_mlp1(up(x), up(wg), up(wu), up(sg), up(su), o.ptr, cols, rows)
    assert ref.ref_sync() == 0
    res.update({f"{tag}_shape": np.array([rows, cols]), f"{tag}_w": w, f"{tag}_x": x, f"{tag}_wg": wg, f"{tag}_wu": wu,
                f"{tag}_gemv_out": acc.numpy(np.float16), f"{tag}_mlp1_out": o.numpy(np.float16)})
    if quant:
        res.update({f"{tag}_s": s, f"{tag}_sg": sg, f"{tag}_su": su})

ref = O.ref_lib("0.5b", "fp16")
# attention: 14 query heads / 2 KV heads, head_dim 64, 75 keys (not a multiple of 16), zero rows after the context
nh, nkv, hd, max_seq, length = 14, 2, 64, 96, 75
q = rng.standard_normal((nh, hd)).astype(np.float16)
Kc = np.zeros((nkv, max_seq, hd), np.float16); Vc = np.zeros((nkv, max_seq, hd), np.float16)
Kc[:, :length] = rng.standard_normal((nkv, length, hd)).astype(np.float16)
Vc[:, :length] = rng.standard_normal((nkv, length, hd)).astype(np.float16)
n = nkv * 16 * 64
po, pm, ps, ao = DevBuf(n * hd * 4), DevBuf(n * 4), DevBuf(n * 4), DevBuf(nh * hd * 2)
ref.ref_attention(up(q), up(Kc), up(Vc), ao.ptr, up(np.array([length - 1], np.int32)), nh, nkv, hd, max_seq, po.ptr, pm.ptr, ps.ptr)
assert ref.ref_sync() == 0
res.update({"attn_shape": np.array([nh, nkv, hd, max_seq, length]), "attn_q": q, "attn_k": Kc, "attn_v": Vc, "attn_out": ao.numpy(np.float16)})
# rmsnorm
x = (2 * rng.standard_normal(896)).astype(np.float16); w = (1 + 0.02 * rng.standard_normal(896)).astype(np.float16)
ro = DevBuf(896 * 2)
ref.ref_rmsnorm(up(x), up(w), ro.ptr, 896, 1e-6)
assert ref.ref_sync() == 0
res.update({"rms_x": x, "rms_w": w, "rms_out": ro.numpy(np.float16)})
# rope via the fused block with identity-free inputs: q/k = bias only (zero weights), position 77
dim, pos = 128, 77
zq = np.zeros((nh * hd, dim), np.float16); zk = np.zeros((nkv * hd, dim), np.float16)
bq = rng.standard_normal(nh * hd).astype(np.float16); bk = rng.standard_normal(nkv * hd).astype(np.float16); bv = rng.standard_normal(nkv * hd).astype(np.float16)
qo, ko, vo = DevBuf(nh * hd * 2), DevBuf(nkv * hd * 2), DevBuf(nkv * hd * 2)
ref.ref_qkv(up(np.zeros(dim, np.float16)), up(zq), up(zk), up(zk), None, None, None, up(bq), up(bk), up(bv), qo.ptr, ko.ptr, vo.ptr, dim, nh, nkv, hd,
            up(np.array([pos], np.int32)), 1e6)
assert ref.ref_sync() == 0
res.update({"rope_shape": np.array([nh, nkv, hd, pos]), "rope_q": bq, "rope_k": bk, "rope_q_out": qo.numpy(np.float16), "rope_k_out": ko.numpy(np.float16)})
np.savez_compressed(out_path, **res)
print("wrote", out_path, "with", len(res), "arrays")
