"""Where one decode step spends its time.

``python -m cuqwen_b200.steptrace --model 7b --quant int4 --ctx 8192`` prints two tables for a random-init model:

* launch by launch (``cuqwen_step_profile``): the default path run eagerly with a CUDA event after every launch, averaged
  per kind of kernel (times include launch gaps, so they bound the graph replay from above);
* inside the graph (``CUQWEN_FLAG_STEP_TRACE``): every GEMV / attention launch stamps its own timeline while the step
  replays as a CUDA graph with programmatic dependent launch - relative to the moment the launch before it finished:
  when its first / last CTA started, when the dependency wait returned, when the input vector was staged, when the
  main loop and the kernel ended.  The last column is what the launch adds to the step.

The reference's counterpart is benchmark/kernel_profile.cu, which times each kernel in isolation.
"""
from __future__ import annotations

import argparse
import os
import subprocess
from pathlib import Path

import numpy as np

from . import _abi, binfmt, build
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


def timeline(model: str, quant: str, ctx: int, reps: int = 8) -> dict:
    prm = E.model_params(model, quant)
    prm.flags = E.FLAG_STEP_TRACE
    eng = E.Engine(prm)
    eng.load(str(model_file(model, quant)))
    eng.kv_fill_normal(ctx, 42)
    eng.decode_n(1234, ctx, 64)
    ms = eng.last_decode_ms / 64
    L = binfmt.MODELS[model]["layers"]
    ptr, nbytes = eng.ptr("STEP_TRACE")
    acc = None
    for r in range(reps):
        _abi.check(_abi.lib().cuqwen_dev_memset(eng.device, ptr, 0, nbytes))
        E.sync(eng.device)
        eng.step(5, ctx + 64 + r)                               # one graph replay
        t = eng.read("STEP_TRACE", dtype=np.uint64).reshape(-1, 16).copy()
        for c in (0, 2):
            t[:, c] = ~t[:, c]                                  # "first" stamps are stored complemented
        t = t.astype(np.int64)[1:1 + 6 * L + 1]                 # launch 0 is the embedding copy (no stamps)
        prev_end = np.concatenate([[t[0, 0]], t[:-1, 5]])
        rel = (t[:, :6] - prev_end[:, None]) / 1e3
        acc = rel if acc is None else acc + rel
    eng.close()
    rel = acc / reps
    body = rel[:6 * L].reshape(L, 6, 6)[1:].mean(0)             # skip the first layer (it follows the embedding copy)
    names = ["qkv", "attn partials", "attn fold", "o_proj", "gate/up", "down"]
    rows = {n: body[i].tolist() for i, n in enumerate(names)}
    rows["lm_head"] = rel[6 * L].tolist()
    return {"ms_per_step": ms, "rows": rows, "layer_us": float(body[:, 5].sum())}


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
    tl = timeline(a.model, a.quant, a.ctx)
    print(f"inside the graph ({tl['ms_per_step']:.3f} ms per step with the stamps on), us after the previous launch ended:")
    print(f"  {'launch':<14s} {'1st CTA':>8s} {'last CTA':>8s} {'wait ret':>8s} {'staged':>8s} {'loop end':>8s} {'end':>8s}")
    for n, v in tl["rows"].items():
        print(f"  {n:<14s} " + " ".join(f"{x:8.2f}" if abs(x) < 1e6 else f"{'-':>8s}" for x in v))
    print(f"  one layer: {tl['layer_us']:.2f} us")


if __name__ == "__main__":
    main()
