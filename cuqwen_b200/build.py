"""In-tree build of the CUDA library (sm_100a) and of the CPU oracle.

``build_all()`` compiles every ``csrc/*.cu`` with nvcc for ``sm_100a`` and links
``cuqwen_b200/libcuqwen_b200.so`` and the host-only tokenizer into
``cuqwen_b200/libcuqwen_tok.so``; it also builds ``oracle/liboracle.so`` (the
scalar C checker) and, when the CuQwen sources are present on this machine, the
reference's own CUDA kernels into ``oracle/_ref/`` (see ``oracle/build_ref.py``).
Objects go to ``build/`` and are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "cuqwen_b200" / "csrc"
OBJ = ROOT / "build" / "obj"
LIB = ROOT / "cuqwen_b200" / "libcuqwen_b200.so"
ORACLE_SRC = ROOT / "oracle" / "oracle.c"
ORACLE_LIB = ROOT / "oracle" / "liboracle.so"
TOK_SRC = CSRC / "tokenizer.cpp"
TOK_LIB = ROOT / "cuqwen_b200" / "libcuqwen_tok.so"
GEN_SRC = CSRC / "gen_random_bin.cpp"
GEN_BIN = ROOT / "cuqwen_b200" / "gen_random_bin"

def reference_dir() -> Path:
    """Where a checkout of the reference (CuQwen) lies: $CUQWEN_REFERENCE_DIR, else a directory named `reference`
    beside this repository.  Only build-time and test-time tooling looks there; nothing at run time does."""
    return Path(os.environ.get("CUQWEN_REFERENCE_DIR") or ROOT.parent / "reference")


def cuda_home() -> Path:
    """The CUDA toolkit root: $CUDA_HOME / $CUDA_PATH, else the directory two levels above the nvcc on PATH."""
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            return Path(os.environ[var])
    import shutil
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parent.parent
    raise RuntimeError("CUDA toolkit not found: set CUDA_HOME")


NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, log: Path | None = None):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)))
    return r


def build_cuda(verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + [h for h in CSRC.glob("*.h") if h.name != "unicode_tables.h"] + [ROOT / "include" / "cuqwen_b200.h"]
    srcs = sorted(CSRC.glob("*.cu"))
    jobs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if _newer(o, [s] + headers):
            jobs.append((s, o))

    def cc(job):
        s, o = job
        _run(["nvcc", *NVCC_FLAGS, "-c", str(s), "-o", str(o)], log=OBJ / (s.stem + ".ptxas.txt"))
        return s.name

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for name in ex.map(cc, jobs):
            if verbose:
                print("compiled", name)
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if _newer(LIB, objs):
        tmp = LIB.with_suffix(".so.tmp")     # link aside and rename: a reader never sees a half-written library
        _run(["nvcc", "-shared", "-o", str(tmp), *map(str, objs), "-lcudart", "-ldl"])
        os.replace(tmp, LIB)
    return LIB


def build_oracle() -> Path:
    if _newer(ORACLE_LIB, [ORACLE_SRC]):
        _run(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC", str(ORACLE_SRC), "-o", str(ORACLE_LIB), "-lm"])
    return ORACLE_LIB


def build_tokenizer() -> Path:
    """The tokenizer is host code with no CUDA in it: a library of its own (include/cuqwen_tokenizer.h)."""
    deps = [TOK_SRC, CSRC / "unicode_tables.h", ROOT / "include" / "cuqwen_tokenizer.h"]
    if _newer(TOK_LIB, deps):
        _run(["g++", "-O2", "-std=c++17", "-Wall", "-shared", "-fPIC", str(TOK_SRC), "-o", str(TOK_LIB)])
    return TOK_LIB


def build_gen() -> Path:
    if GEN_SRC.exists() and _newer(GEN_BIN, [GEN_SRC]):
        _run(["g++", "-O3", "-std=c++17", "-pthread", str(GEN_SRC), "-o", str(GEN_BIN)])
    return GEN_BIN


def build_all(verbose: bool = False) -> None:
    build_cuda(verbose)
    build_gen()
    build_tokenizer()
    build_oracle()
    ref = ROOT / "oracle" / "build_ref.py"
    if ref.exists() and (reference_dir() / "src" / "kernels.cu").exists():
        subprocess.run([sys.executable, str(ref), "--ref", str(reference_dir())], check=True)


if __name__ == "__main__":
    build_all(verbose=True)
