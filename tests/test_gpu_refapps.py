"""CuQwen's own programs, built from their unmodified source files against include/compat and linked to this
repository's libraries (oracle/build_ref.py puts them in oracle/_ref/apps where the CuQwen checkout is available),
run on the GPU: the chat front end produces the engine's tokens, the benchmark program completes its protocol."""
import json
import os
import re
import shutil
import subprocess
from pathlib import Path

import pytest

from cuqwen_b200 import build
from cuqwen_b200 import engine as E
from cuqwen_b200 import tokenizer as T
from oracle import tokenizer_py as O

ROOT = Path(__file__).resolve().parent.parent
APPS = ROOT / "oracle" / "_ref" / "apps"
VOCAB = 151936


def full_vocab_ranks(path: Path) -> None:
    """A ranks file in which every id of the model's vocabulary decodes to visible text: ids 0..255 are the byte
    symbols, id i >= 256 is "<i in base 36>" (no two entries concatenate to a third, so nothing merges)."""
    alpha = O.byte_alphabet()
    vocab = {alpha[b]: i for i, b in enumerate(sorted(alpha))}
    digits = "0123456789abcdefghijklmnopqrstuvwxyz"
    for i in range(256, VOCAB):
        s, v = "", i
        while v:
            s = digits[v % 36] + s
            v //= 36
        vocab[f"<{s}>"] = i
    added = {"151643": "<|endoftext|>", "151644": "<|im_start|>", "151645": "<|im_end|>"}
    path.write_text(json.dumps({"vocab": vocab, "special_tokens": {}, "added_tokens": added}, ensure_ascii=False), encoding="utf-8")


@pytest.fixture(scope="module")
def workdir(built):
    if not (APPS / "chat_b200_0_5b_int4").exists():
        pytest.skip("the reference's programs were not built on this machine (oracle/build_ref.py)")
    build.build_tokenizer()
    base = Path("/dev/shm") if Path("/dev/shm").is_dir() and os.access("/dev/shm", os.W_OK) else Path("/tmp")
    d = base / f"cuqwen_refapps_{os.getpid()}"
    (d / "weights").mkdir(parents=True, exist_ok=True)
    (d / "build").mkdir(exist_ok=True)
    subprocess.run([str(build.GEN_BIN), "--out", str(d / "weights" / "model_int4_0_5b.bin"), "--model", "0.5b", "--quant", "int4", "--seed", "11"], check=True)
    full_vocab_ranks(d / "weights" / "qwen25_bpe_ranks.json")
    yield d
    shutil.rmtree(d, ignore_errors=True)


@pytest.mark.gpu
def test_chat_program_prints_the_engines_tokens(workdir):
    user = "Hello there, what's 2+2?"
    r = subprocess.run([str(APPS / "chat_b200_0_5b_int4")], input=(user + "\nexit\n").encode(), capture_output=True, cwd=workdir, timeout=600)
    assert r.returncode == 0, r.stderr.decode(errors="replace")[-2000:]
    out = r.stdout
    assert b"Engine Initialized and Ready" in out and b"Cleaning up CUDA resources... Done." in out
    m = re.search(rb"\[(\d+) tokens generated \| [\d.]+ tok/s \| Context: (\d+)/32768\]", out)
    assert m, out[-500:]
    said = out.split(b"Qwen > ", 1)[1]

    # the same conversation through the Python binding (src/main.cu:57-112: prefill without history, then decode with
    # the generated tokens as penalty history)
    with T.QwenTokenizer(workdir / "weights" / "qwen25_bpe_ranks.json") as tok:
        prompt = tok.encode(T.apply_chat_template([T.Message("user", user)], True))
        assert prompt[0] == 151644 and 151645 in prompt
        eng = E.Engine(E.model_params("0.5b", 2))
        eng.load(str(workdir / "weights" / "model_int4_0_5b.bin"))
        pos, nxt = 0, 0
        for t in prompt:
            nxt = eng.step(t, pos)
            pos += 1
        gen = []
        while nxt not in (151643, 151645) and len(gen) < 300:
            gen.append(nxt)
            nxt = eng.step(nxt, pos, history=gen)
            pos += 1
        eng.close()
        want = tok.decode_bytes(gen)
    assert len(want) > 300 and said.startswith(want), (said[:200], want[:200])
    n_generated, context = int(m.group(1)), int(m.group(2))
    assert context == len(prompt) + n_generated and (n_generated >= len(gen))


@pytest.mark.gpu
def test_benchmark_program_completes_its_protocol(workdir):
    r = subprocess.run([str(APPS / "benchmark_b200_0_5b_int4")], capture_output=True, text=True, cwd=workdir / "build", timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    samples = re.findall(r"\[Sample\] Context\s+(\d+)K .*Speed: ([\d.]+) tok/s", r.stdout)
    assert [int(k) for k, _ in samples] == [1, 5, 9, 13, 17, 21, 25, 29, 32]
    assert all(float(v) > 100 for _, v in samples)
    assert "Average Speed" in r.stdout
    print(r.stdout[r.stdout.index("OVERALL METRICS") - 80:])


@pytest.mark.gpu
def test_kernel_profile_program_runs_every_operator(workdir):
    r = subprocess.run([str(APPS / "kernel_profile_b200_0_5b_int4"), "1000"], capture_output=True, text=True, cwd=workdir, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    for label in ("rmsnorm", "fused_attn_block(qkv+rope)", "kv_cache_store", "gqa_attention_decode", "o_proj gemv_add", "mlp_stage1(gate+up)",
                  "mlp_stage2(down)", "embedding_lookup", "compute_logits(lm_head)", "repetition_penalty", "argmax"):
        assert re.search(re.escape(label) + r"\s+[\d.]+ us", r.stdout), label
    assert "est/token" in r.stdout
    # the program times with events on ITS stream (the default stream); the wrappers order the library's stream
    # against it, so the lm_head (272 MB of fp16 for this model) cannot come out faster than the memory allows
    lm_head_us = float(re.search(r"compute_logits\(lm_head\)\s+([\d.]+) us", r.stdout).group(1))
    assert lm_head_us > 272e6 / 8e12 * 1e6, lm_head_us
