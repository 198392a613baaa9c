"""Build the UNMODIFIED CuQwen CUDA sources into oracle/_ref/ (test / baseline infrastructure).

The reference picks model and quantisation at compile time, so one shared
library is produced per (model, quant): ``oracle/_ref/libcuqwen_ref_<model>_<quant>.so``.
Sources are compiled where they lie under the reference checkout with plain
nvcc (the reference's CMake needs libpcre2 / nlohmann-json for a tokenizer this
path never calls); only ``ref_wrap.cu`` of this repository is added.  Flags
follow the reference's CMakeLists.txt:105 (``-O3 --use_fast_math``), the
architecture is sm_100a.

It also builds the reference's own PROGRAMS into oracle/_ref/apps/, each from its unmodified source file:
  chat_b200_<m>_<q>, benchmark_b200_<m>_<q>, kernel_profile_b200_<m>_<q>
      src/main.cu, benchmark/cuqwen_benchmark.cu, benchmark/kernel_profile.cu compiled against this repository's
      source-compatible headers (include/compat) and linked to libcuqwen_b200.so / libcuqwen_tok.so: the drop-in check;
  benchmark_ref_<m>_<q>
      benchmark/cuqwen_benchmark.cu with the reference's own kernels.cu, model.cu, load_weights.cpp: the stock
      program, for a like-for-like run under the reference's own measuring protocol.

For a few (model, quant) pairs a second library ``..._tuned.so`` is built from the same sources with the two launch
constants the reference's config.h asks users to retune per GPU set to its large-GPU values (see TUNED_KNOBS).

Usage: python oracle/build_ref.py [--ref <CuQwen checkout>] [--only 7b:int4,0.5b:fp16] [--no-apps]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
OUT = HERE / "_ref"
MODEL_DEF = {"0.5b": "QWEN_MODEL_0_5B", "1.5b": "QWEN_MODEL_1_5B", "3b": "QWEN_MODEL_3B", "7b": "QWEN_MODEL_7B", "14b": "QWEN_MODEL_14B"}
QUANT_DEF = {"fp16": None, "int8": "QUANT_INT8", "int4": "QUANT_INT4"}
DEFAULT = [(m, q) for m in ("0.5b", "7b", "14b") for q in ("fp16", "int8", "int4")]


# The reference's config.h tells users to retune two launch constants per GPU (include/config.h:140-146 and :178-185;
# the shipped 64 / 128 are its RTX 3090 values, 128 / 256 its values for the widest part it lists).  The "tuned"
# libraries are the same unmodified sources with exactly that edit made.
TUNED_KNOBS = {"ATTN_PARTITIONS": 128, "ARGMAX_BLOCKS": 256}
TUNED = [("7b", "int4"), ("14b", "int8"), ("0.5b", "int4")]


def lib_path(model: str, quant: str, tuned: bool = False) -> Path:
    return OUT / f"libcuqwen_ref_{model.replace('.', '_')}_{quant}{'_tuned' if tuned else ''}.so"


def tuned_config(ref: Path) -> Path:
    """A generated copy of the reference's config.h with the two constants of TUNED_KNOBS changed and nothing else.
    It is pre-included, so the include guard makes the sources' own #include "config.h" a no-op."""
    import re
    text = (ref / "include" / "config.h").read_text()
    for name, value in TUNED_KNOBS.items():
        text, n = re.subn(rf"(constexpr\s+int\s+{name}\s*=\s*)\d+(\s*;)", rf"\g<1>{value}\g<2>", text)
        if n != 1:
            raise RuntimeError(f"config.h: expected exactly one definition of {name}, found {n}")
    d = OUT / "tuned_include"
    d.mkdir(parents=True, exist_ok=True)
    out = d / "config.h"
    if not out.exists() or out.read_text() != text:
        out.write_text(text)
    return out


def build_one(ref: Path, model: str, quant: str, tuned: bool = False) -> Path:
    out = lib_path(model, quant, tuned)
    srcs = [ref / "src" / "kernels.cu", ref / "src" / "model.cu", ref / "src" / "load_weights.cpp", HERE / "ref_wrap.cu"]
    deps = srcs + [ROOT / "cuqwen_b200" / "csrc" / "rng.cuh", ref / "include" / "config.h"]
    if out.exists() and all(out.stat().st_mtime > d.stat().st_mtime for d in deps):
        return out
    cmd = ["nvcc", "-O3", "--use_fast_math", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-shared", "-Xcompiler", "-fPIC", "-x", "cu", f"-D{MODEL_DEF[model]}"]
    if tuned:
        cmd += ["-include", str(tuned_config(ref))]
    if QUANT_DEF[quant]:
        cmd.append(f"-D{QUANT_DEF[quant]}")
    cmd += ["-I", str(ref / "include"), "-I", str(ROOT / "cuqwen_b200" / "csrc"), *map(str, srcs), "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"reference build failed for {model}/{quant}")
    return out


APPS = [("0.5b", "int4"), ("7b", "int4")]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def app_path(kind: str, model: str, quant: str) -> Path:
    return OUT / "apps" / f"{kind}_{model.replace('.', '_')}_{quant}"


def _nvcc(cmd, what: str) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"reference program build failed: {what}")


def build_apps(ref: Path, model: str, quant: str) -> list[Path]:
    """The reference's programs for one (model, quant); skipped when this repository's libraries are not built yet."""
    libdir = ROOT / "cuqwen_b200"
    if not (libdir / "libcuqwen_b200.so").exists() or not (libdir / "libcuqwen_tok.so").exists():
        return []
    (OUT / "apps").mkdir(parents=True, exist_ok=True)
    defs = [f"-D{MODEL_DEF[model]}"] + ([f"-D{QUANT_DEF[quant]}"] if QUANT_DEF[quant] else [])
    compat = [ROOT / "include" / "cuqwen_compat.hpp", ROOT / "include" / "cuqwen_b200.h", ROOT / "include" / "cuqwen_tokenizer.h",
              ROOT / "include" / "compat" / "tokenizer.h"]
    built = []
    ours = {"chat_b200": ref / "src" / "main.cu", "benchmark_b200": ref / "benchmark" / "cuqwen_benchmark.cu",
            "kernel_profile_b200": ref / "benchmark" / "kernel_profile.cu"}
    for kind, src in ours.items():
        out = app_path(kind, model, quant)
        if not (out.exists() and all(out.stat().st_mtime > d.stat().st_mtime for d in [src, *compat])):
            _nvcc(["nvcc", "-O2", "-std=c++17", *ARCH, "-diag-suppress", "177", *defs, "-I", str(ROOT / "include" / "compat"), str(src), "-o", str(out),
                   "-L", str(libdir), "-lcuqwen_b200", "-lcuqwen_tok", "-Xlinker", "-rpath=$ORIGIN/../../../cuqwen_b200"], out.name)
        built.append(out)
    out = app_path("benchmark_ref", model, quant)
    srcs = [ref / "src" / "kernels.cu", ref / "src" / "model.cu", ref / "src" / "load_weights.cpp", ref / "benchmark" / "cuqwen_benchmark.cu"]
    if not (out.exists() and all(out.stat().st_mtime > d.stat().st_mtime for d in srcs)):
        _nvcc(["nvcc", "-O3", "--use_fast_math", "-std=c++17", *ARCH, "-x", "cu", *defs, "-I", str(ref / "include"), *map(str, srcs), "-o", str(out)], out.name)
    built.append(out)
    return built


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CUQWEN_REFERENCE_DIR") or str(ROOT.parent / "reference"))
    ap.add_argument("--only", default="")
    ap.add_argument("--no-apps", action="store_true")
    a = ap.parse_args()
    ref = Path(a.ref)
    if not (ref / "src" / "kernels.cu").exists():
        print(f"reference sources not found under {ref}; nothing built")
        return
    OUT.mkdir(exist_ok=True)
    todo = [tuple(x.split(":")) for x in a.only.split(",") if x] or DEFAULT
    with ThreadPoolExecutor(max_workers=4) as ex:
        for p in ex.map(lambda mq: build_one(ref, *mq), todo):
            print("built", p.name)
        for p in ex.map(lambda mq: build_one(ref, *mq, tuned=True), [mq for mq in TUNED if mq in todo]):
            print("built", p.name)
        if not a.no_apps:
            for ps in ex.map(lambda mq: build_apps(ref, *mq), APPS):
                for p in ps:
                    print("built", p.name)


if __name__ == "__main__":
    main()
