"""Build the UNMODIFIED CuQwen CUDA sources into oracle/_ref/ (test / baseline infrastructure).

The reference picks model and quantisation at compile time, so one shared
library is produced per (model, quant): ``oracle/_ref/libcuqwen_ref_<model>_<quant>.so``.
Sources are compiled where they lie under the reference checkout with plain
nvcc (the reference's CMake needs libpcre2 / nlohmann-json for a tokenizer this
path never calls); only ``ref_wrap.cu`` of this repository is added.  Flags
follow the reference's CMakeLists.txt:105 (``-O3 --use_fast_math``), the
architecture is sm_100a.

Usage: python oracle/build_ref.py [--ref <CuQwen checkout>] [--only 7b:int4,0.5b:fp16]
"""
from __future__ import annotations

import argparse
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


def lib_path(model: str, quant: str) -> Path:
    return OUT / f"libcuqwen_ref_{model.replace('.', '_')}_{quant}.so"


def build_one(ref: Path, model: str, quant: str) -> Path:
    out = lib_path(model, quant)
    srcs = [ref / "src" / "kernels.cu", ref / "src" / "model.cu", ref / "src" / "load_weights.cpp", HERE / "ref_wrap.cu"]
    deps = srcs + [ROOT / "cuqwen_b200" / "csrc" / "rng.cuh"]
    if out.exists() and all(out.stat().st_mtime > d.stat().st_mtime for d in deps):
        return out
    cmd = ["nvcc", "-O3", "--use_fast_math", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-shared", "-Xcompiler", "-fPIC", "-x", "cu", f"-D{MODEL_DEF[model]}"]
    if QUANT_DEF[quant]:
        cmd.append(f"-D{QUANT_DEF[quant]}")
    cmd += ["-I", str(ref / "include"), "-I", str(ROOT / "cuqwen_b200" / "csrc"), *map(str, srcs), "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"reference build failed for {model}/{quant}")
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default="/root/reference")
    ap.add_argument("--only", default="")
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


if __name__ == "__main__":
    main()
