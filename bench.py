#!/usr/bin/env python
"""Headline benchmark: batch-1 greedy decode of random-init Qwen2.5-7B W4A16 at an 8K-token KV context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model 7b] [--quant int4] [--ctx 8192]

One "step" is one decode token (one pass of the hot path).  Rank 0 prints ONE JSON line:
  value   tokens/s with the token fed back on the device (cuqwen_decode_n: K graph replays between two CUDA events)
  e2e     tokens/s through cuqwen_step, the call a host makes per token: host token in (H2D), sampled token out (D2H)
  roofline    the dominant kernel (gate/up W4A16 GEMV + SwiGLU) timed alone over all layers' weights, algorithmic
              bytes / CUDA-event time against the measured HBM copy bandwidth; `step` gives the same for the whole step
  cpu_baseline  the scalar CPU oracle of the same step on the host cores (N=1, rank 0, bounded sample)
--impl reference times the reference's own CUDA build (oracle/_ref, its qwen_forward loop) on the same file and context.
Under torchrun (N>1) the model is tensor-parallel over the N GPUs (strong scaling: the work per token is fixed).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "B=1 decode tok/s (7B W4A16, 1/2/4/8 B200); GEMV HBM GB/s vs peak"
SEED = 42
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel from an ncu capture (see profiles/);
# None until a capture exists for the shape.  7B int4: 70,102,016 read + 1,697,792 written
# (profiles/gemv_kernel_int4_swiglu_7b_gateup_ncu.md).
NCU_TRAFFIC_BYTES = {("7b", "int4"): 71799808}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def model_path(model: str, quant: str, layers: int = 0) -> Path:
    base = Path("/dev/shm") if os.access("/dev/shm", os.W_OK) else Path("/tmp")
    return base / f"cuqwen_bench_{model.replace('.', '_')}_{quant}{f'_L{layers}' if layers else ''}_seed{SEED}.bin"


def model_config(model: str, layers: int = 0) -> dict:
    """The model's dimensions; layers > 0 cuts the depth (same matrices, fewer of them) for profiler captures, which
    must keep the memory held on the device small."""
    from cuqwen_b200 import binfmt
    cfg = dict(binfmt.MODELS[model])
    if layers:
        cfg["layers"] = layers
    return cfg


def ensure_model_file(model: str, quant: str, layers: int = 0) -> Path:
    from cuqwen_b200 import binfmt, build
    p = model_path(model, quant, layers)
    cfg = model_config(model, layers)
    want = binfmt.file_nbytes(cfg, binfmt.QUANT_ID[quant])
    if not p.exists() or p.stat().st_size != want:
        build.build_gen()
        tmp = p.with_suffix(f".tmp{os.getpid()}")
        if layers:
            dims = [str(cfg[k]) for k in ("vocab", "dim", "inter", "layers", "heads", "kv", "hd")]
            cmd = [str(build.GEN_BIN), "--out", str(tmp), "--dims", *dims, "--quant", quant, "--seed", str(SEED)] + ([] if cfg["tied"] else ["--untied"])
        else:
            cmd = [str(build.GEN_BIN), "--out", str(tmp), "--model", model, "--quant", quant, "--seed", str(SEED)]
        subprocess.run(cmd, check=True)
        os.replace(tmp, p)
    return p


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc = device, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.device)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill(); out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def workload_config(a, cfg, qid: int, steps: int) -> dict:
    """The `config` object: identical in both arms (what differs between them is reported under `arm`)."""
    from cuqwen_b200 import binfmt
    kv8 = getattr(a, "kv", "fp16") == "int8" and getattr(a, "impl", "ours") == "ours"
    gb = binfmt.step_bytes(cfg, qid, int(a.ctx + steps / 2), kv8) / 1e9
    cut = f" CUT TO {a.layers} LAYERS (profiler-sized, not a benchmark value)" if getattr(a, "layers", 0) else ""
    return {"workload": f"Qwen2.5-{a.model.upper()}{cut} {a.quant} random-init (N(0,0.02) weights, seed {SEED}), B=1 greedy decode, "
                        f"KV context {a.ctx} prefilled with N(0,1) fp16{' (stored as int8 rows + scales)' if kv8 else ''}, {steps} steps",
            "l2": f"no flush needed: every step streams {gb:.2f} GB of weights and KV, far beyond the 126 MB L2"}


def dist_setup(n: int):
    """Returns (rank, world, local_rank, torch.distributed or None)."""
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world == 1:
        return 0, 1, 0, None
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local, dist


def max_over_ranks(dist, local: int, v: float) -> float:
    if dist is None:
        return v
    import torch
    t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{local}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(dist, local: int):
    if dist is not None:
        import torch
        dist.barrier()
        torch.cuda.synchronize(local)


def dominant_kernel_roofline(eng, E, K, model_cfg, quant_id: int, iters: int = 20):
    """gate/up GEMV + SwiGLU alone, cycling over every layer's weights (inputs far larger than L2)."""
    dim, inter_l = model_cfg["dim"], eng.ptr("GATE")[1] // 2
    L = model_cfg["layers"]
    x = E.DevBuf.from_numpy(np.random.default_rng(0).standard_normal(dim).astype(np.float16), eng.device)
    out = E.DevBuf(inter_l * 2, eng.device)
    ptrs = [(eng.ptr("WGATE", l)[0], eng.ptr("WUP", l)[0], eng.ptr("SGATE", l)[0] or None, eng.ptr("SUP", l)[0] or None, eng.ptr("POST_NORM", l)[0])
            for l in range(L)]
    wbytes = eng.ptr("WGATE", 0)[1] + eng.ptr("SGATE", 0)[1]
    eps = float(np.float16(1e-6))               # the reference narrows eps to fp16 (src/model.cu:131-134)

    def sweep():      # the kernel exactly as the step launches it: fused RMSNorm prologue with the layer's own weight
        for wg, wu, sg, su, nw in ptrs:
            K.fused_mlp_stage1(quant_id, x, wg, wu, sg, su, out, dim, inter_l, norm_weight=nw, eps=eps, device=eng.device)

    for _ in range(3):
        sweep()
    E.sync(eng.device)
    K.bench_begin(eng.device)
    for _ in range(iters):
        sweep()
    ms = K.bench_end(eng.device)
    per_launch_s = ms / 1e3 / (iters * L)
    alg = 2 * wbytes + dim * 2 + dim * 2 + inter_l * 2          # weights + scales, x, the RMSNorm weight, the output
    return alg, per_launch_s


PARITY_RTOL, PARITY_ATOL, PARITY_TIE = 2e-3, 1e-2, 1e-3      # per-operator fp16 contract: 2e-3 relative or 1e-2 absolute
PARITY_RMS = 1.5e-2                                          # whole step: rms(logit difference) / rms(logits); measured 0.6 % (7B, 8K keys) to 1.0 % (14B, 32,000 keys)


def parity_leg(eng, a, cfg, path, rank, world, local, dist, steps: int = 32):
    """UNTIMED check of what the timed legs computed.  Rank 0 runs the reference's own CUDA build (oracle/_ref, the
    checker) on the same model file with the same seeded KV fill; both engines are fed the reference's token stream
    (teacher forcing) for `steps` tokens at the benchmark's context.  Every rank's slice of the logits is gathered and
    compared with the reference's logits.  Pass = (a) greedy top-1 agreement >= 99 % (the same token, or one the
    reference itself holds within the fp16 contract of its own choice - random-init logits are nearly flat) and (b)
    rms(difference) <= 1.5 % of rms(logits).  The per-operator contract (2e-3 relative / 1e-2 absolute) is what the
    kernel tests hold every GEMV and attention output to; after 28 or 48 layers the two engines' fp16 roundings (the
    reference also rounds scores and probabilities to fp16) have accumulated, so the line reports how many logits still
    sit inside it instead of requiring all of them to.  Returns the JSON object (rank 0) or None."""
    import ctypes as C
    from cuqwen_b200 import engine as E
    from cuqwen_b200 import tp as TP
    V, ctx = cfg["vocab"], a.ctx
    ref = rm = None
    why = ""
    if rank == 0:
        from oracle import oracle_py as O
        ref = O.ref_lib(a.model, a.quant)
        if ref is None:
            why = f"oracle/_ref/{O.ref_lib_path(a.model, a.quant).name} not built"
        else:
            rm = ref.ref_model_load(str(path).encode())
            ref.ref_kv_fill_normal(rm, ctx, SEED)
    have = 1 if rm else 0
    if dist is not None:
        import torch
        t = torch.tensor([have], dtype=torch.int32, device=f"cuda:{local}")
        dist.broadcast(t, 0)
        have = int(t.item())
    if not have:
        return {"vs": "unavailable", "why": why, "pass": None} if rank == 0 else None
    eng.kv_fill_normal(ctx, SEED)              # the timed legs wrote rows ctx .. ctx+K; start from the same cache as the reference
    pl = TP.plan(cfg, rank, world)
    tok = 1234 % V
    agree = strict = 0
    worst_abs = worst_rms = 0.0
    inside = total = 0
    for i in range(steps):
        tok_r, lr = 0, None
        if rank == 0:
            tok_r = int(ref.ref_forward(rm, tok, ctx + i, None, 0))
            lr = E.download(local, ref.ref_state_ptr(rm, 0), np.float16, V).astype(np.float32)
        tok_e = eng.step(tok, ctx + i)
        mine = eng.read("LOGITS").astype(np.float32)
        if dist is not None:
            import torch
            parts = [None] * world
            dist.all_gather_object(parts, (pl.v0, mine))
            t = torch.tensor([tok_r], dtype=torch.int64, device=f"cuda:{local}")
            dist.broadcast(t, 0)
            tok_r = int(t.item())
        else:
            parts = [(pl.v0, mine)]
        if rank == 0:
            le = np.zeros(V, dtype=np.float32)
            for v0, sl in parts:
                le[v0:v0 + len(sl)] = sl
            d = np.abs(le - lr)
            worst_abs = max(worst_abs, float(d.max()))
            worst_rms = max(worst_rms, float(np.sqrt((d * d).mean()) / max(np.sqrt((lr * lr).mean()), 1e-12)))
            inside += int((d <= PARITY_ATOL + PARITY_RTOL * np.abs(lr)).sum()); total += V
            strict += tok_e == tok_r
            agree += (tok_e == tok_r) or abs(lr[tok_r] - lr[tok_e]) <= PARITY_RTOL * abs(lr[tok_r]) + PARITY_TIE
        tok = tok_r
    if rank != 0:
        return None
    ref.ref_model_free(rm)
    kv8 = a.kv == "int8"     # the 8-bit cache is outside the parity contract: compared with the same reference, looser bar
    ok = bool(np.isfinite(worst_rms) and worst_rms <= (1e-1 if kv8 else PARITY_RMS) and agree / steps >= (0.85 if kv8 else 0.99))
    return {"vs": f"reference CUDA build oracle/_ref (qwen_forward, teacher-forced), same file, same KV seed, context {ctx}",
            "steps": steps, "top1_agree": round(agree / steps, 4), "top1_identical": round(strict / steps, 4),
            "max_abs_logit": round(worst_abs, 6), "rel_rms_logit": round(worst_rms, 6),
            "logits_inside_2e-3rel_1e-2abs": round(inside / max(total, 1), 6),
            "criterion": "int8 KV cache, outside the parity contract (sanity bound only): top1_agree >= 0.85 and rel_rms_logit <= 0.1" if kv8 else "top1_agree >= 0.99 and rel_rms_logit <= 0.015",
            "pass": ok}


def run_ours(a):
    rank, world, local, dist = dist_setup(a.gpus)
    from cuqwen_b200 import binfmt
    from cuqwen_b200 import engine as E
    from cuqwen_b200 import kernels as K
    qid = E.QUANT_ID[a.quant]
    cfg = model_config(a.model, a.layers)
    if rank == 0:
        path = ensure_model_file(a.model, a.quant, a.layers)
    barrier(dist, local)
    path = model_path(a.model, a.quant, a.layers)
    if a.layers:       # profiler-sized variant: explicit dims, and a KV cache just long enough for the run
        prm = E.custom_params(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], a.quant,
                              max_seq_len=(a.ctx + a.steps + max(a.warmup, 3) + 64 + 15) // 16 * 16)
    else:
        prm = E.model_params(a.model, a.quant)
    prm.device, prm.tp_rank, prm.tp_size = local, rank, world
    kv8 = a.kv == "int8"
    if kv8:
        prm.flags |= E.FLAG_KV_INT8
    prm.flags |= a.flags
    eng = E.Engine(prm)
    eng.load(str(path))
    if world > 1:
        import torch
        idt = torch.zeros(128, dtype=torch.uint8, device=f"cuda:{local}")
        if rank == 0:
            idt = torch.tensor(list(E.nccl_unique_id()), dtype=torch.uint8, device=f"cuda:{local}")
        dist.broadcast(idt, 0)
        eng.tp_init(bytes(idt.cpu().tolist()))
    ctx, Kst, W = a.ctx, a.steps, max(a.warmup, 3)
    eng.kv_fill_normal(ctx, SEED)
    first = 1234 % cfg["vocab"]

    # ---- value: device-resident token feedback, K graph replays between two events ----
    eng.decode_n(first, ctx, W)
    barrier(dist, local)
    with ClockSampler(local) as cs:
        eng.decode_n(first, ctx, Kst)
        ms = eng.last_decode_ms
    barrier(dist, local)
    ms = max_over_ranks(dist, local, ms)
    value = Kst / (ms / 1e3)

    # ---- e2e: one cuqwen_step per token, host token in, sampled token out ----
    # (cuqwen_step_loop: the per-token calls in a C loop, as the reference arm's loop is; no Python between the tokens)
    eng.step_loop(first, ctx, W)
    barrier(dist, local)
    t0 = time.perf_counter()
    eng.step_loop(first, ctx, Kst)
    e2e_s = time.perf_counter() - t0
    barrier(dist, local)
    e2e_s = max_over_ranks(dist, local, e2e_s)
    e2e = Kst / e2e_s

    peak, peak_src = peaks()
    mean_ctx = ctx + Kst / 2
    step_bytes_total = binfmt.step_bytes(cfg, qid, int(mean_ctx), kv8)
    out = {
        "metric": METRIC, "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": Kst, "warmup": W,
        "ms_per_step": round(ms / Kst, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int4 weights x fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": workload_config(a, cfg, qid, Kst),
        "arm": {"parallelism": f"tp{world}", "attn_splits": eng.params.attn_splits, "kv_cache": a.kv},
        "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 12,
                "how": "cuqwen_step per token (C loop, cuqwen_step_loop): the host writes token / position into a pinned mailbox that the step's first kernel reads over PCIe (16 B), the last kernel writes token + status + sequence number back (12 B) and the host polls for it"},
        "gpu_launches": Kst * eng.step_launches,
        "clocks": cs.result,
    }
    step_gbs = step_bytes_total / (ms / 1e3 / Kst) / 1e9
    out["step"] = {"algorithmic_bytes": step_bytes_total, "achieved_gbs_all_gpus": round(step_gbs, 1), "frac_of_n_x_peak": round(step_gbs / (peak * world), 4),
                   "launches_per_step": eng.step_launches}
    if rank == 0:
        alg, sec = dominant_kernel_roofline(eng, E, K, cfg, qid)
        ach = alg / sec / 1e9
        out["roofline"] = {"bound": "hbm", "kernel": "gemv_kernel<int4, SWIGLU> (gate/up GEMV + SwiGLU)", "achieved": round(ach, 1), "peak": peak,
                           "unit": "GB/s", "frac": round(ach / peak, 4), "peak_source": peak_src + ", of measured", "frac_of_nominal_8tbs": round(ach / 8000.0, 4), "bytes_per_launch": alg,
                           "us_per_launch": round(sec * 1e6, 3), "traffic": NCU_TRAFFIC_BYTES.get((a.model, a.quant))}
    par = None if (a.no_parity or a.layers) else parity_leg(eng, a, cfg, path, rank, world, local, dist)
    if rank == 0 and par is not None:
        out["parity"] = par
    if rank == 0 and world == 1 and not kv8 and cfg["hd"] in (64, 128):
        # the step before the hot path (the "next" row the prefill kernels cover): one prompt through cuqwen_prefill,
        # after everything timed above (it overwrites the first rows of the synthetic KV fill)
        n = min(2048, ctx)
        toks = np.random.default_rng(SEED).integers(0, cfg["vocab"], size=n).astype(np.int32)
        eng.prefill(toks[:min(512, n)], 0)
        eng.prefill(toks, 0)
        pms = eng.last_decode_ms
        d, I, nl, qd, kd = cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"] * cfg["hd"], cfg["kv"] * cfg["hd"]
        flop = 2.0 * n * (nl * d * (qd + 2 * kd) + (nl - 1) * (qd * d + 3 * d * I)) + 4.0 * cfg["heads"] * cfg["hd"] * (n * (n + 1) / 2) * (nl - 1)
        # its dominant kernel alone, the way the dominant decode kernel is reported above: the gate/up + SwiGLU GEMM of
        # every layer in turn over the prompt's activations (weights 1.9 GB in all: nothing stays in L2), CUDA events
        gate_ptrs = [(eng.ptr("WGATE", l)[0], eng.ptr("WUP", l)[0], eng.ptr("SGATE", l)[0] or None, eng.ptr("SUP", l)[0] or None) for l in range(nl)]
        xa = E.DevBuf.from_numpy(np.random.default_rng(1).standard_normal((n, d)).astype(np.float16), eng.device)
        ga = E.DevBuf(n * I * 2, eng.device)

        def gemm_sweep():
            for wg, wu, sg, su in gate_ptrs:
                K.prefill_gemm(qid, K.PF_SWIGLU, xa, wg, sg, ga, n, I, d, w1=wu, s1=su, device=eng.device)
        gemm_sweep()
        E.sync(eng.device)
        K.bench_begin(eng.device)
        for _ in range(3):
            gemm_sweep()
        gsec = K.bench_end(eng.device) / 1e3 / (3 * nl)
        gflop = 2.0 * n * d * 2 * I
        tpeak = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        burst, sustained = float(tpeak.get("bf16_tflops", 1590.0)), float(tpeak.get("bf16_tflops_sustained", 1400.0))
        out["prefill"] = {"prompt_tokens": n, "ms": round(pms, 3), "prompt_tok_s": round(n / (pms / 1e3), 1), "tflops": round(flop / (pms / 1e3) / 1e12, 1),
                          "roofline": {"bound": "tensor", "kernel": f"prefill_gemm_kernel<{a.quant}> (gate/up GEMM + SwiGLU, {n} x {d} x {2 * I}, tcgen05)",
                                       "achieved": round(gflop / gsec / 1e12, 1), "peak": burst, "unit": "TFLOP/s", "frac": round(gflop / gsec / 1e12 / burst, 4),
                                       "frac_of_sustained": round(gflop / gsec / 1e12 / sustained, 4), "us_per_launch": round(gsec * 1e6, 1),
                                       "peak_source": ("measured (MEASURED_PEAKS.json bf16_tflops: cuBLAS burst; bf16_tflops_sustained for the second fraction), of measured"
                                                       if tpeak else "fallback (1590 / 1400 TFLOP/s), of fallback")},
                          "what": "cuqwen_prefill: batched tcgen05 GEMMs and attention filling the KV cache for a prompt; the reference does this with one "
                                  "qwen_forward per token (bench.py --sweep prefill [--impl reference] compares them)"}
    eng.close()
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline(path, cfg, ctx)
    if rank == 0:
        emit(out)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and par is not None and par.get("pass") is False:
        sys.stderr.write("bench: PARITY FAILED " + json.dumps(par) + "\n")
        sys.exit(3)


def cpu_baseline(path: Path, cfg: dict, ctx: int, steps: int = 2):
    """Scalar CPU oracle of the same step on the host cores: a bounded sample (1 untimed + `steps` timed tokens)."""
    from oracle import oracle_py as O
    m = O.OracleModel(str(path), ctx + steps + 2)
    Kc, Vc = m.kv_views()
    rng = np.random.default_rng(SEED)
    blk = rng.standard_normal((cfg["kv"], 512, cfg["hd"])).astype(np.float16)
    for l in range(cfg["layers"]):
        for s in range(0, ctx, 512):
            n = min(512, ctx - s)
            Kc[l, :, s:s + n] = blk[:, :n]; Vc[l, :, s:s + n] = blk[:, :n]
    tok = m.step(1234 % cfg["vocab"], ctx)
    t0 = time.perf_counter()
    for i in range(steps):
        tok = m.step(tok, ctx + 1 + i)
    dt = time.perf_counter() - t0
    cores = O.lib().orc_threads()
    m.close()
    return {"value": round(steps / dt, 4), "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{steps} decode steps (after 1 untimed) of the same model file at KV context {ctx}, scalar C oracle, OpenMP over output rows"}


_JSON_OUT = None


def emit(obj):
    out = _JSON_OUT or sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle_py as O
    from cuqwen_b200 import binfmt
    from cuqwen_b200 import engine as E
    ref = O.ref_lib(a.model, a.quant)
    if ref is None:
        emit({"impl": "reference", "unavailable": f"oracle/_ref/{O.ref_lib_path(a.model, a.quant).name} was not built (needs the CuQwen sources at build time)"})
        return
    cfg = binfmt.MODELS[a.model]
    path = ensure_model_file(a.model, a.quant)
    ctx, Kst, W = a.ctx, a.steps, max(a.warmup, 3)
    first = 1234 % cfg["vocab"]
    import ctypes as C

    def timed(lib):
        m = lib.ref_model_load(str(path).encode())
        lib.ref_kv_fill_normal(m, ctx, SEED)
        toks = (C.c_int * max(Kst, W))()
        lib.ref_decode_n(m, first, ctx, W, toks)       # first call also captures the reference's CUDA graph
        with ClockSampler(0) as cs:
            t0 = time.perf_counter()
            ms = lib.ref_decode_n(m, first, ctx, Kst, toks)
            wall = time.perf_counter() - t0
        lib.ref_model_free(m)
        return ms, wall, cs

    ms, wall, cs = timed(ref)
    value, e2e = Kst / (ms / 1e3), Kst / wall
    # the same sources with the two launch constants the reference's config.h asks users to retune per GPU set to its
    # large-GPU values (oracle/build_ref.py): reported beside the stock build, the faster of the two is the bar
    tuned = None
    rt = O.ref_lib(a.model, a.quant, tuned=True)
    if rt is not None:
        ms_t, wall_t, _ = timed(rt)
        tuned = {"value": round(Kst / (ms_t / 1e3), 2), "e2e": round(Kst / wall_t, 2), "unit": "tok/s", "knobs": {"ATTN_PARTITIONS": 128, "ARGMAX_BLOCKS": 256},
                 "source": "include/config.h:140-146,178-185 of the reference: its own per-GPU guidance, largest values listed"}
    qid = E.QUANT_ID[a.quant]
    nl = 1 + 10 * cfg["layers"] + 5
    out = {
        "impl": "reference", "metric": METRIC, "value": round(value, 2), "unit": "tok/s", "n_gpus": 1, "steps": Kst, "warmup": W,
        "ms_per_step": round(ms / Kst, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int4 weights x fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": workload_config(a, cfg, qid, Kst),
        "arm": {"parallelism": "tp1 (the reference is single-GPU)",
                "build": "CuQwen src/kernels.cu + model.cu + load_weights.cpp, nvcc -O3 --use_fast_math sm_100a, stock tuning constants"},
        "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 4},
        "gpu_launches": Kst * nl, "clocks": cs.result,
        "cpu_baseline": {"value": round(value, 2), "unit": "tok/s", "cores": 0, "kind": "reference",
                         "sample": "the reference has no CPU implementation of this path; this arm is its own CUDA build run on the GPU "
                                   f"({Kst} qwen_forward calls)"},
        "step": {"algorithmic_bytes": binfmt.step_bytes(cfg, qid, int(ctx + Kst / 2))},
    }
    if tuned is not None:
        out["tuned"] = tuned
    emit(out)


def run_sweep(a):
    """Kernel-level measurements of the other benchmark configurations, one JSON line each:
      --sweep gemv       the single W4A16 GEMV at the Qwen2.5-0.5B MLP shape (4864 x 896), HBM-cold and L2-warm
      --sweep attention  split-KV attention alone over lengths {512, 2K, 8K, 32K} x heads {28/4, 40/8} x split counts
      --sweep prefill    a prompt of --prompt tokens through cuqwen_prefill (batched tiles) against the token-by-token path
    --impl reference times the reference's own kernels (launch_gemv_add_fp16 on a zeroed accumulator, src/kernels.cu:640-687;
    launch_gqa_attention_decode with its fixed 64 partitions, :290-323) in C loops inside oracle/_ref."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from cuqwen_b200 import binfmt
    from cuqwen_b200 import engine as E
    from cuqwen_b200 import microbench as MB
    rng = np.random.default_rng(1234)
    L2 = 126 << 20
    if a.sweep == "prefill":
        run_prefill_sweep(a, rng)
        return
    if a.impl == "ours":
        if a.sweep == "gemv":
            rows = MB.single_gemv(4864, 896, "int4", 2000)
        else:
            rows = MB.attention_sweep(iters=200)
        emit({"sweep": a.sweep, "impl": "ours", "timing": "CUDA events around replays of a CUDA graph of the launches (no caller in the measurement)", "rows": rows})
        return
    from oracle import oracle_py as O
    import ctypes as C
    if a.sweep == "gemv":
        ref = O.ref_lib("0.5b", "int4")
        if ref is None:
            emit({"sweep": a.sweep, "impl": "reference", "unavailable": "oracle/_ref not built"}); return
        r, c = 4864, 896
        q = rng.integers(-8, 8, size=(r, c), dtype=np.int8)
        w, sc = binfmt.pack_int4(q), rng.uniform(0.002, 0.02, size=(r, c // 128)).astype(np.float16)
        x = E.DevBuf.from_numpy(rng.standard_normal(c).astype(np.float16))
        y = E.DevBuf(r * 2)
        rows = []
        for label, n in (("HBM-cold", -(-3 * L2 // w.nbytes)), ("L2-warm", 1)):
            ws = [E.DevBuf.from_numpy(w) for _ in range(n)]; ss = [E.DevBuf.from_numpy(sc) for _ in range(n)]
            E.sync()
            pw, ps = (C.c_void_p * n)(*[b.ptr for b in ws]), (C.c_void_p * n)(*[b.ptr for b in ss])
            us = ref.ref_bench_gemv_add(pw, ps, n, x.ptr, y.ptr, r, c, 2000) * 1e3
            alg = w.nbytes + sc.nbytes + c * 2 + r * 2
            rows.append({"kernel": f"launch_gemv_add_fp16 {r}x{c} int4 ({label})", "us": round(us, 3), "bytes": alg, "gbs": round(alg / us / 1e3, 1)})
        emit({"sweep": a.sweep, "impl": "reference", "timing": "CUDA events around a C loop of launches", "rows": rows})
        return
    rows, hd, max_seq = [], 128, 32768
    for (nh, nkv), model in (((28, 4), "7b"), ((40, 8), "14b")):
        ref = O.ref_lib(model, "fp16")
        if ref is None:
            continue
        qv, out = E.DevBuf.from_numpy(rng.standard_normal(nh * hd).astype(np.float16)), E.DevBuf(nh * hd * 2)
        npart = nkv * 16 * 64                                   # partial buffers as src/model.cu:40-43 sizes them
        po, pm, ps_ = E.DevBuf(npart * hd * 4), E.DevBuf(npart * 4), E.DevBuf(npart * 4)
        for n in (512, 2048, 8192, 32768):
            ncopy = max(2, min(16, -(-3 * L2 // (2 * nkv * n * hd * 2))))
            blk = rng.standard_normal(n * hd).astype(np.float16)
            kv = []
            for _ in range(ncopy):
                kb, vb = E.DevBuf(nkv * max_seq * hd * 2), E.DevBuf(nkv * max_seq * hd * 2)      # zero past the context, as the reference relies on
                for h in range(nkv):
                    kb.upload(blk, h * max_seq * hd * 2); vb.upload(blk, h * max_seq * hd * 2)
                kv.append((kb, vb))
            dpos = E.DevBuf.from_numpy(np.array([n - 1], np.int32))
            E.sync()
            pk, pv = (C.c_void_p * ncopy)(*[k.ptr for k, _ in kv]), (C.c_void_p * ncopy)(*[v.ptr for _, v in kv])
            us = ref.ref_bench_attention(qv.ptr, pk, pv, ncopy, out.ptr, dpos.ptr, nh, nkv, hd, max_seq, po.ptr, pm.ptr, ps_.ptr, 200) * 1e3
            alg = 2 * nkv * n * hd * 2
            rows.append({"heads": f"{nh}/{nkv}", "len": n, "splits": 64, "us": round(us, 3), "bytes": alg, "gbs": round(alg / us / 1e3, 1)})
            del kv
    emit({"sweep": a.sweep, "impl": "reference", "timing": "CUDA events around a C loop of launches", "rows": rows})


def run_prefill_sweep(a, rng):
    """Time to fill the KV cache for a prompt of a.prompt tokens (model a.model / a.quant, random token ids).
    ours: cuqwen_prefill (device time between CUDA events, and wall clock around the call with the ids in host memory),
    beside the same engine's token-by-token path.  --impl reference: the reference's only prefill, qwen_forward once per
    prompt token (src/main.cu:86-92).  The token-by-token figures are estimates: 32 steps at each of four evenly spaced
    positions, mean time per step times the prompt length."""
    from cuqwen_b200 import binfmt
    from cuqwen_b200 import engine as E
    cfg = model_config(a.model, a.layers)            # --layers cuts the depth for profiler captures (not a benchmark value)
    path = ensure_model_file(a.model, a.quant, a.layers)
    n = a.prompt
    spots = [n // 8, 3 * n // 8, 5 * n // 8, 7 * n // 8]
    qid = E.QUANT_ID[a.quant]
    d, I, nl, qd, kd = cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"] * cfg["hd"], cfg["kv"] * cfg["hd"]
    # the last layer stops once its keys and values are stored: it has no attention, o_proj or MLP in a prefill
    gemm_flop = 2.0 * n * (nl * d * (qd + 2 * kd) + (nl - 1) * (qd * d + 3 * d * I))
    attn_flop = 4.0 * cfg["heads"] * cfg["hd"] * (n * (n + 1) / 2) * (nl - 1)
    if a.impl == "ours":
        if a.layers:
            prm = E.custom_params(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], a.quant, max_seq_len=max(n + 64, 1024))
        else:
            prm = E.model_params(a.model, a.quant)
            prm.max_seq_len = max(n + 64, 1024)
        eng = E.Engine(prm)
        eng.load(str(path))
        toks = rng.integers(0, cfg["vocab"], size=n).astype(np.int32)
        eng.prefill(toks[:512], 0)                      # warm-up: workspace allocation, kernel attributes
        with ClockSampler(0) as cs:
            t0 = time.perf_counter()
            eng.prefill(toks, 0)
            wall = time.perf_counter() - t0
        ms = eng.last_decode_ms
        per_tok = []
        for pos in spots:
            eng.decode_n(1234 % cfg["vocab"], pos, 8)
            eng.decode_n(1234 % cfg["vocab"], pos, 32)
            per_tok.append(eng.last_decode_ms / 32)
        est = float(np.mean(per_tok)) * n
        emit({"sweep": "prefill", "impl": "ours", "model": a.model + (f" cut to {a.layers} layers" if a.layers else ""), "quant": a.quant, "prompt_tokens": n,
              "prefill_ms": round(ms, 3), "prefill_wall_ms": round(wall * 1e3, 3), "prompt_tok_s": round(n / (ms / 1e3), 1),
              "tflops": round((gemm_flop + attn_flop) / (ms / 1e3) / 1e12, 1), "gemm_flop": gemm_flop, "attention_flop": attn_flop,
              "token_by_token_ms_estimate": round(est, 1), "token_by_token_ms_per_step_at": dict(zip(map(str, spots), [round(v, 4) for v in per_tok])),
              "speedup_over_token_by_token": round(est / ms, 1), "clocks": cs.result})
        eng.close()
        return
    from oracle import oracle_py as O
    import ctypes as C
    ref = O.ref_lib(a.model, a.quant)
    if ref is None:
        emit({"sweep": "prefill", "impl": "reference", "unavailable": "oracle/_ref not built"}); return
    m = ref.ref_model_load(str(path).encode())
    ref.ref_kv_fill_normal(m, n, SEED)
    toks = (C.c_int * 64)()
    per_tok = []
    for pos in spots:
        ref.ref_decode_n(m, 1234 % cfg["vocab"], pos, 8, toks)
        per_tok.append(ref.ref_decode_n(m, 1234 % cfg["vocab"], pos, 32, toks) / 32)
    ref.ref_model_free(m)
    est = float(np.mean(per_tok)) * n
    emit({"sweep": "prefill", "impl": "reference", "model": a.model, "quant": a.quant, "prompt_tokens": n,
          "prefill_ms_estimate": round(est, 1), "prompt_tok_s": round(n / (est / 1e3), 1),
          "ms_per_step_at": dict(zip(map(str, spots), [round(v, 4) for v in per_tok])),
          "how": "qwen_forward once per prompt token (src/main.cu:86-92): 32 calls at each of four positions, mean x prompt length"})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prompt", type=int, default=8192, help="--sweep prefill: prompt length in tokens")
    ap.add_argument("--model", default="7b")
    ap.add_argument("--quant", default="int4")
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--flags", type=int, default=0, help="extra CUQWEN_FLAG_* bits for the engine (comparison variants)")
    ap.add_argument("--kv", default="fp16", choices=["fp16", "int8"], help="KV cache format (int8: opt-in 8-bit cache, outside the parity contract)")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (profiler captures only; the JSON line says so)")
    ap.add_argument("--sweep", default="", choices=["", "gemv", "attention", "prefill"], help="kernel-level sweeps of the other benchmark configurations")
    a = ap.parse_args()
    # Libraries (NCCL's version banner, for one) write to file descriptor 1.  Keep the real stdout aside for the one
    # JSON line and send everything else to stderr.
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if a.sweep:
        run_sweep(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
