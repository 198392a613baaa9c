"""Per-kernel timing harness: every operator of one decoder layer (plus lm_head) in isolation, at a model's real
shapes, reported as algorithmic bytes / CUDA-event time = GB/s.

The counterpart of the reference's benchmark/kernel_profile.cu (cudaEvent timing of each launch_* on dummy buffers
at a fixed position), with two differences: each kernel rotates over several distinct copies of its weights so that
the bytes really come from HBM rather than from the 126 MB L2, and the result is expressed against the bytes the
kernel has to move.

    python -m cuqwen_b200.microbench --model 7b --quant int4 --pos 8192 [--kernels gateup,down] [--iters 50] [--json]
    python -m cuqwen_b200.microbench --quant int4 --gemv 4864x896        # one GEMV, HBM-cold and L2-warm
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import binfmt
from . import engine as E
from . import kernels as K

L2_BYTES = 126 << 20


def _weights(rng, rows, cols, quant):
    if quant == 0:
        return (0.02 * rng.standard_normal((rows, cols))).astype(np.float16), None
    lo, hi = (-8, 7) if quant == 2 else (-128, 127)
    q = rng.integers(lo, hi + 1, size=(rows, cols), dtype=np.int8)
    s = rng.uniform(0.002, 0.02, size=(rows, cols // 128)).astype(np.float16)
    return (binfmt.pack_int4(q) if quant == 2 else q), s


class Copies:
    """n device copies of one (weights, scales) pair; `next()` cycles through them."""

    def __init__(self, rng, rows, cols, quant, min_total_bytes, device):
        w, s = _weights(rng, rows, cols, quant)
        self.bytes = w.nbytes + (s.nbytes if s is not None else 0)
        n = max(2, -(-min_total_bytes // self.bytes)) if min_total_bytes > 0 else 1      # 0: a single copy (L2-warm timing)
        n = min(n, 64)
        self.w = [E.DevBuf.from_numpy(w, device) for _ in range(n)]
        self.s = [E.DevBuf.from_numpy(s, device) if s is not None else None for _ in range(n)]
        self.i = 0

    def next(self):
        self.i = (self.i + 1) % len(self.w)
        return self.w[self.i], self.s[self.i]


def graph_time(fn, iters: int, device: int = 0, per_graph: int = 16) -> float:
    """Microseconds per call of `fn` (which queues kernels through the C ABI) with the caller out of the measurement:
    `per_graph` calls are recorded into a CUDA graph (cuqwen_capture_begin) and the graph is replayed between two
    events.  `fn` should rotate over its weight copies with a period that divides `per_graph`."""
    for _ in range(per_graph):
        fn()                                # every kernel has run once before the capture; the rotation is back at its start
    E.sync(device)
    K.capture_begin(device)
    for _ in range(per_graph):
        fn()
    replays = max(1, iters // per_graph)
    return K.capture_replay(replays, device) * 1e3 / per_graph


def run(model: str, quant: str, pos: int, which, iters: int, device: int = 0, rotate_bytes: int = 3 * L2_BYTES):
    cfg, q = binfmt.MODELS[model], E.QUANT_ID[quant]
    d, I, V, hd, nh, nkv = cfg["dim"], cfg["inter"], cfg["vocab"], cfg["hd"], cfg["heads"], cfg["kv"]
    qd, kd = nh * hd, nkv * hd
    rng = np.random.default_rng(0)
    h16 = lambda n: E.DevBuf.from_numpy(rng.standard_normal(n).astype(np.float16), device)
    x, xq, xi = h16(d), h16(qd), h16(I)
    normw = E.DevBuf.from_numpy(np.ones(d, np.float16), device)
    dpos = E.DevBuf.from_numpy(np.array([pos], np.int32), device)
    eps = float(np.float16(1e-6))
    results = []

    def timed(name, alg_bytes, fn, period=1):
        us = graph_time(fn, iters, device, period * -(-16 // period))       # whole rotations, at least 16 calls per graph
        results.append({"kernel": name, "us": round(us, 3), "bytes": int(alg_bytes), "gbs": round(alg_bytes / us / 1e3, 1)})

    if "qkv" in which:
        cq, ck, cv = (Copies(rng, r, d, q, rotate_bytes // 3, device) for r in (qd, kd, kd))
        bq, bk, bv = h16(qd), h16(kd), h16(kd)
        qo, ko, vo = E.DevBuf(qd * 2, device), E.DevBuf(kd * 2, device), E.DevBuf(kd * 2, device)
        max_seq = 32768
        kc, vc = E.DevBuf(nkv * max_seq * hd * 2, device), E.DevBuf(nkv * max_seq * hd * 2, device)

        def f():
            (wq, sq), (wk, sk), (wv, sv) = cq.next(), ck.next(), cv.next()
            K.fused_attn_block(q, x, wq, wk, wv, sq, sk, sv, bq, bk, bv, qo, ko, vo, d, nh, nkv, hd, dpos, norm_weight=normw, eps=eps,
                               kcache=kc, vcache=vc, max_seq_len=max_seq, device=device)
        timed("rmsnorm+qkv+bias+rope+kvstore", cq.bytes + ck.bytes + cv.bytes + 2 * d * 2 + (qd + 2 * kd) * 2, f, max(len(cq.w), len(ck.w)))
    if "attn" in which:
        max_seq = 32768
        ncopy = max(2, -(-rotate_bytes // (2 * nkv * (pos + 1) * hd * 2)))
        ncopy = min(ncopy, 16)
        kv = []
        for _ in range(ncopy):
            kbuf, vbuf = E.DevBuf(nkv * max_seq * hd * 2, device), E.DevBuf(nkv * max_seq * hd * 2, device)
            blk = rng.standard_normal((pos + 1) * hd).astype(np.float16)
            for h in range(nkv):
                kbuf.upload(blk, h * max_seq * hd * 2); vbuf.upload(blk, h * max_seq * hd * 2)
            kv.append((kbuf, vbuf))
        sm = E.sm_count(device)
        nsplit = max(1, min(128, sm // nkv))
        bo, bml, bc = K.attn_scratch_bytes(nkv, hd, nsplit)
        so, sml, cnt = E.DevBuf(bo, device), E.DevBuf(bml, device), E.DevBuf(bc, device)
        qv, out = h16(qd), E.DevBuf(qd * 2, device)
        state = {"i": 0}

        def f():
            state["i"] = (state["i"] + 1) % ncopy
            kbuf, vbuf = kv[state["i"]]
            K.gqa_attention_decode(qv, kbuf, vbuf, out, dpos, nh, nkv, hd, max_seq, nsplit, so, sml, cnt, device=device)
        timed(f"attention(ctx {pos + 1}, {nsplit} splits)", 2 * nkv * (pos + 1) * hd * 2, f, ncopy)
    if "oproj" in which:
        c = Copies(rng, d, qd, q, rotate_bytes, device)
        xr = h16(d)

        def f():
            w, s = c.next()
            K.gemv_add(q, w, s, xq, xr, d, qd, device=device)
        timed("o_proj+residual", c.bytes + qd * 2 + d * 4, f, len(c.w))
    if "gateup" in which:
        cg, cu = Copies(rng, I, d, q, rotate_bytes // 2, device), Copies(rng, I, d, q, rotate_bytes // 2, device)
        out = E.DevBuf(I * 2, device)

        def f():
            (wg, sg), (wu, su) = cg.next(), cu.next()
            K.fused_mlp_stage1(q, x, wg, wu, sg, su, out, d, I, norm_weight=normw, eps=eps, device=device)
        timed("rmsnorm+gate/up+swiglu", cg.bytes + cu.bytes + 2 * d * 2 + I * 2, f, len(cg.w))
    if "down" in which:
        c = Copies(rng, d, I, q, rotate_bytes, device)
        xr = h16(d)

        def f():
            w, s = c.next()
            K.gemv_add(q, w, s, xi, xr, d, I, device=device)
        timed("down+residual", c.bytes + I * 2 + d * 4, f, len(c.w))
    if "lmhead" in which:
        lq = 0 if (cfg["tied"] or q == 0) else 1
        c = Copies(rng, V, d, lq, rotate_bytes, device)
        out = E.DevBuf(V * 2, device)

        def f():
            w, s = c.next()
            K.gemv(lq, w, s, x, out, V, d, norm_weight=normw, eps=eps, device=device)
        timed("rmsnorm+lm_head", c.bytes + 2 * d * 2 + V * 2, f, len(c.w))
    return results


def single_gemv(rows: int, cols: int, quant: str, iters: int, device: int = 0) -> list:
    """One W.x GEMV (fp16 out), HBM-cold (rotating over copies worth three L2 sizes) and L2-warm (one copy).
    With rows=4864, cols=896, quant=int4 this is the single W4A16 GEMV of the benchmark configurations:
    integers uniform in [-8, 7], scales U(0.002, 0.02), x ~ N(0, 1); bytes = weights + scales + x + y."""
    q = E.QUANT_ID[quant]
    rng = np.random.default_rng(1234)
    x = E.DevBuf.from_numpy(rng.standard_normal(cols).astype(np.float16), device)
    y = E.DevBuf(rows * 2, device)
    out = []
    for label, rot in (("HBM-cold", 3 * L2_BYTES), ("L2-warm", 0)):
        c = Copies(rng, rows, cols, q, rot, device)

        def f():
            w, s = c.next()
            K.gemv(q, w, s, x, y, rows, cols, device=device)
        us = graph_time(f, iters, device, len(c.w) * -(-16 // len(c.w)))
        alg = c.bytes + cols * 2 + rows * 2
        out.append({"kernel": f"gemv {rows}x{cols} {quant} ({label})", "us": round(us, 3), "bytes": int(alg), "gbs": round(alg / us / 1e3, 1)})
    return out


def attention_sweep(lens=(512, 2048, 8192, 32768), heads=((28, 4), (40, 8)), splits=(8, 16, 32, 64, 128), iters: int = 200, device: int = 0) -> list:
    """Split-KV attention alone (both launches: partials, fold) over context lengths, head layouts and split counts:
    q fp16 [n_heads, 128] ~ N(0,1), K and V fp16 N(0,1) in the head-major cache layout, rotating over copies worth
    three L2 sizes.  Algorithmic bytes = 2 * n_kv * len * 128 * 2.  The split count SMs / n_kv (one CTA per SM, what
    the engine uses) is always part of the sweep."""
    hd, max_seq = 128, 32768
    rng = np.random.default_rng(4)
    sm = E.sm_count(device)
    out = []
    for nh, nkv in heads:
        q = E.DevBuf.from_numpy(rng.standard_normal(nh * hd).astype(np.float16), device)
        o = E.DevBuf(nh * hd * 2, device)
        for n in lens:
            ncopy = max(2, min(16, -(-3 * L2_BYTES // (2 * nkv * n * hd * 2))))
            blk = rng.standard_normal(n * hd).astype(np.float16)
            kv = []
            for _ in range(ncopy):
                kb, vb = E.DevBuf(nkv * max_seq * hd * 2, device), E.DevBuf(nkv * max_seq * hd * 2, device)
                for h in range(nkv):
                    kb.upload(blk, h * max_seq * hd * 2); vb.upload(blk, h * max_seq * hd * 2)
                kv.append((kb, vb))
            dpos = E.DevBuf.from_numpy(np.array([n - 1], np.int32), device)
            alg = 2 * nkv * n * hd * 2
            for ns in sorted(set(list(splits) + [max(1, min(128, sm // nkv))])):
                bo, bml, bc = K.attn_scratch_bytes(nkv, hd, ns)
                so, sml, cnt = E.DevBuf(bo, device), E.DevBuf(bml, device), E.DevBuf(bc, device)
                st = {"i": 0}

                def f():
                    st["i"] = (st["i"] + 1) % ncopy
                    K.gqa_attention_decode(q, kv[st["i"]][0], kv[st["i"]][1], o, dpos, nh, nkv, hd, max_seq, ns, so, sml, cnt, device=device)
                us = graph_time(f, iters, device, ncopy * -(-16 // ncopy))
                out.append({"heads": f"{nh}/{nkv}", "len": n, "splits": ns, "us": round(us, 3), "bytes": alg, "gbs": round(alg / us / 1e3, 1)})
                E.sync(device)
            del kv
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="7b")
    ap.add_argument("--quant", default="int4")
    ap.add_argument("--pos", type=int, default=8191)
    ap.add_argument("--kernels", default="qkv,attn,oproj,gateup,down,lmhead")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--rotate-mb", type=int, default=3 * 126)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--gemv", default="", help="ROWSxCOLS: time one GEMV of that shape instead (e.g. 4864x896), cold and L2-warm")
    ap.add_argument("--attn-sweep", action="store_true", help="attention alone over lengths x head layouts x split counts")
    a = ap.parse_args()
    if a.attn_sweep:
        res = attention_sweep(iters=max(a.iters, 100), device=a.device)
        if a.json:
            print(json.dumps({"attention_sweep": res}))
        else:
            for r in res:
                print(f"  heads {r['heads']:<5} len {r['len']:>6} splits {r['splits']:>4} {r['us']:>9.2f} us  {r['bytes'] / 1e6:>8.2f} MB  {r['gbs']:>8.1f} GB/s")
        return
    if a.gemv:
        rows, cols = (int(v) for v in a.gemv.lower().split("x"))
        res = single_gemv(rows, cols, a.quant, max(a.iters, 200), a.device)
        if a.json:
            print(json.dumps({"quant": a.quant, "kernels": res}))
        else:
            for r in res:
                print(f"  {r['kernel']:<44} {r['us']:>9.2f} us  {r['bytes'] / 1e6:>9.3f} MB  {r['gbs']:>8.1f} GB/s")
        return
    res = run(a.model, a.quant, a.pos, set(a.kernels.split(",")), a.iters, a.device, a.rotate_mb << 20)
    if a.json:
        print(json.dumps({"model": a.model, "quant": a.quant, "pos": a.pos, "kernels": res}))
    else:
        print(f"Qwen2.5-{a.model} {a.quant}  position {a.pos}")
        for r in res:
            print(f"  {r['kernel']:<36} {r['us']:>9.2f} us  {r['bytes'] / 1e6:>9.2f} MB  {r['gbs']:>8.1f} GB/s")
        cfg = binfmt.MODELS[a.model]
        per_layer = sum(r["us"] for r in res if "lm_head" not in r["kernel"])
        print(f"  layer subtotal {per_layer:.1f} us x {cfg['layers']} layers")


if __name__ == "__main__":
    main()
