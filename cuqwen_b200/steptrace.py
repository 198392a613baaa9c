"""Where one decode step spends its time.

``python -m cuqwen_b200.steptrace --model 7b --quant int4 --ctx 8192`` prints two tables for a random-init model:

* launch by launch (``cuqwen_step_profile``): the default path run eagerly with a CUDA event after every launch, averaged
  per kind of kernel (times include launch gaps, so they bound the graph replay from above);
* phase by phase (``CUQWEN_FLAG_FUSED_STEP | CUQWEN_FLAG_STEP_TRACE``): the persistent step kernel's own stamps - for
  every phase the span from the first CTA entering it to the first CTA entering the next, the mean and longest time a
  CTA's consumers were busy in it, the time spent staging the activation vector, and the barrier that follows.

The reference's counterpart is benchmark/kernel_profile.cu, which times each kernel in isolation.
"""
from __future__ import annotations

import argparse
import os
import subprocess
from pathlib import Path

import numpy as np

from . import binfmt, build
from . import engine as E


def model_file(model: str, quant: str, seed: int = 42) -> Path:
    base = Path("/dev/shm") if os.access("/dev/shm", os.W_OK) else Path("/tmp")
    p = base / f"cuqwen_bench_{model.replace('.', '_')}_{quant}_seed{seed}.bin"
    want = binfmt.file_nbytes(binfmt.MODELS[model], binfmt.QUANT_ID[quant])
    if not p.exists() or p.stat().st_size != want:
        build.build_gen()
        tmp = p.with_suffix(f".tmp{os.getpid()}")
        subprocess.run([str(build.GEN_BIN), "--out", str(tmp), "--model", model, "--quant", quant, "--seed", str(seed)], check=True)
        os.replace(tmp, p)
    return p


def launches(model: str, quant: str, ctx: int, reps: int = 5) -> dict:
    cfg = binfmt.MODELS[model]
    eng = E.Engine(E.model_params(model, quant))
    eng.load(str(model_file(model, quant)))
    eng.kv_fill_normal(ctx, 42)
    eng.decode_n(1234, ctx, 64)
    ms_graph = eng.last_decode_ms / 64
    us = sum(eng.profile_step(5, ctx + 64 + i) for i in range(reps)) / reps
    L = cfg["layers"]
    per = (len(us) - 1 - 3) // L
    body = us[1:1 + per * L].reshape(L, per)
    names = ["qkv", "attention (2 launches)", "o_proj", "gate/up", "down"] if per == 5 else [f"k{i}" for i in range(per)]
    out = {"graph_ms_per_step": ms_graph, "eager_sum_us": float(us.sum()), "embed": float(us[0]),
           "per_layer": {n: float(v) for n, v in zip(names, body[1:].mean(0))},
           "tail": {n: float(v) for n, v in zip(["lm_head", "penalty", "argmax"], us[1 + per * L:])}}
    eng.close()
    return out


def phases(model: str, quant: str, ctx: int) -> dict:
    prm = E.model_params(model, quant)
    prm.flags = E.FLAG_FUSED_STEP | E.FLAG_STEP_TRACE
    eng = E.Engine(prm)
    eng.load(str(model_file(model, quant)))
    eng.kv_fill_normal(ctx, 42)
    eng.decode_n(1234, ctx, 64)
    ms = eng.last_decode_ms / 64
    eng.step(5, ctx + 64)
    _, nbytes = eng.ptr("STEP_TRACE")
    if nbytes == 0:
        eng.close()
        return {"ms_per_step": ms, "phases": {}}
    L = binfmt.MODELS[model]["layers"]
    nph = 6 * L + 1
    tr = eng.read("STEP_TRACE", dtype=np.uint64).astype(np.int64).reshape(nph, -1, 4)
    eng.close()
    names = ["qkv", "attn partials", "attn fold", "o_proj", "gate/up", "down"]
    agg: dict = {}
    for p in range(nph):
        name = names[p % 6] if p < nph - 1 else "lm_head"
        ent, stg, ext = tr[p, :, 0], tr[p, :, 1], tr[p, :, 2]
        nxt = tr[p + 1, :, 0].min() if p + 1 < nph else ext.max()
        staged = [(s - e) for s, e in zip(stg, ent) if s > 0]
        d = dict(span=(nxt - ent.min()) / 1e3, busy_mean=float((ext - ent).mean()) / 1e3, busy_max=float((ext - ent).max()) / 1e3,
                 stage=float(np.mean(staged)) / 1e3 if staged else 0.0, barrier=(nxt - ext.max()) / 1e3)
        if p >= 6 or name == "lm_head":          # skip the first layer (cold)
            agg.setdefault(name, []).append(d)
    return {"ms_per_step": ms, "phases": {n: {k: float(np.mean([d[k] for d in lst])) for k in lst[0]} for n, lst in agg.items()}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="7b")
    ap.add_argument("--quant", default="int4")
    ap.add_argument("--ctx", type=int, default=8192)
    a = ap.parse_args()
    la = launches(a.model, a.quant, a.ctx)
    print(f"Qwen2.5-{a.model} {a.quant}, KV context {a.ctx}")
    print(f"default path: {la['graph_ms_per_step']:.3f} ms per step as a graph; launch by launch {la['eager_sum_us'] / 1e3:.3f} ms")
    print(f"  embedding {la['embed']:.2f} us")
    for n, v in la["per_layer"].items():
        print(f"  {n:<22s} {v:7.2f} us per layer")
    for n, v in la["tail"].items():
        print(f"  {n:<22s} {v:7.2f} us")
    ph = phases(a.model, a.quant, a.ctx)
    print(f"persistent step kernel: {ph['ms_per_step']:.3f} ms per step")
    print(f"  {'phase':<14s} {'span':>7s} {'busy':>7s} {'longest':>7s} {'staging':>7s} {'barrier':>7s}   (us)")
    for n, d in ph["phases"].items():
        print(f"  {n:<14s} {d['span']:7.2f} {d['busy_mean']:7.2f} {d['busy_max']:7.2f} {d['stage']:7.2f} {d['barrier']:7.2f}")


if __name__ == "__main__":
    main()
