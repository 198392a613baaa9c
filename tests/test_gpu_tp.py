"""Tensor parallelism on 2, 4 and 8 GPUs of one node: one process per GPU (tests/tp_worker.py), compared with the
single-GPU engine on the same model.  Both exchange paths are covered: partials pushed with peer stores (default) and
NCCL all-reduce calls (CUQWEN_FLAG_TP_NCCL).  A case is skipped on a box with fewer GPUs than it has ranks."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from cuqwen_b200 import binfmt
from cuqwen_b200 import engine as E
from tests.gpu_util import close, report

pytestmark = pytest.mark.gpu

CFG = dict(vocab=2048, dim=384, inter=768, layers=3, heads=6, kv=2, hd=128, tied=False)
# the head layout of Qwen2.5-7B (28 query heads over 4 KV heads) at small widths: at 8 ranks two ranks share a KV head and
# split its seven query heads 3 + 4; MLP groups (8) and vocabulary tiles spread one or more per rank
CFG_7B_HEADS = dict(vocab=4096, dim=512, inter=1024, layers=2, heads=28, kv=4, hd=128, tied=False)


def gpu_count() -> int:
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for ln in out.splitlines() if ln.startswith("GPU "))
    except Exception:
        return 0


def run_ranks(tmp_path, cfg, n_ranks, quant, flags):
    path = tmp_path / "m.bin"
    binfmt.write_model(path, cfg, quant, binfmt.random_tensors(cfg, 4))
    (tmp_path / "cfg.json").write_text(json.dumps(cfg))
    worker = Path(__file__).with_name("tp_worker.py")
    procs = [subprocess.Popen([sys.executable, str(worker), str(r), str(n_ranks), str(tmp_path), str(path), str(quant), str(flags)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(n_ranks)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)

    prm = E.custom_params(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], quant, max_seq_len=128)
    one = E.Engine(prm)
    one.load(str(path))
    one.kv_fill_normal(64, seed=9)
    toks = [one.step(3 + i, 64 + i) for i in range(12)]
    toks += one.decode_n(toks[-1], 76, 10).tolist()
    want = one.read("LOGITS")
    one.close()
    ranks = [np.load(tmp_path / f"rank{r}.npz") for r in range(n_ranks)]
    return ranks, toks, want


def check_ranks(ranks, toks, want):
    for r in ranks[1:]:
        assert r["toks"].tolist() == ranks[0]["toks"].tolist()               # every rank learns the same token
    got = np.concatenate([r["logits"] for r in ranks])                        # vocabulary slices in rank order
    assert got.shape == want.shape
    assert close(got, want), report(got, want)
    same = sum(a == b for a, b in zip(ranks[0]["toks"].tolist()[:12], toks[:12]))   # teacher-forced steps are independent of one another
    assert same >= 10, (ranks[0]["toks"].tolist(), toks)


@pytest.mark.parametrize("flags", [E.FLAG_TP_SUM_IN_GEMV, 0, E.FLAG_TP_NCCL], ids=["peer_stores_sum_in_gemv", "peer_stores_sum_kernel", "nccl_allreduce"])
@pytest.mark.parametrize("quant", [2, 0])
def test_two_ranks_match_one_gpu(built, tmp_path, quant, flags):
    if gpu_count() < 2:
        pytest.skip("needs two GPUs")
    ranks, toks, want = run_ranks(tmp_path, CFG, 2, quant, flags)
    per_layer = 10 if flags == E.FLAG_TP_NCCL else 8 if flags == 0 else 6                       # 6 = qkv, attention x2, o_proj, gate/up, down; NCCL adds an all-reduce and a residual kernel twice, the sum kernel adds 2
    tail = 3 + (2 if flags == E.FLAG_TP_NCCL else 1)                                            # lm_head, penalty, sampler + (key all-gather and merge | merge of the pushed keys)
    assert int(ranks[0]["launches"]) == 1 + per_layer * CFG["layers"] + tail
    check_ranks(ranks, toks, want)


@pytest.mark.parametrize("n_ranks", [2, 4, 8])
@pytest.mark.parametrize("quant", [2, 1])
def test_7b_head_layout_over_2_4_8_ranks(built, tmp_path, n_ranks, quant):
    """28 query heads over 4 KV heads: whole KV groups per rank at 2 and 4 ranks, a KV head shared by two ranks (query
    heads 3 + 4) at 8; uneven MLP and vocabulary shares.  Default exchange path (peer stores + sum kernel, pushed keys)."""
    if gpu_count() < n_ranks:
        pytest.skip(f"needs {n_ranks} GPUs")
    ranks, toks, want = run_ranks(tmp_path, CFG_7B_HEADS, n_ranks, quant, 0)
    check_ranks(ranks, toks, want)


@pytest.mark.parametrize("n_ranks", [4])
def test_small_model_over_4_ranks_more_ranks_than_kv_heads(built, tmp_path, n_ranks):
    """6 query heads over 2 KV heads on 4 ranks: each KV head is shared by two ranks (query heads 1 + 2)."""
    if gpu_count() < n_ranks:
        pytest.skip(f"needs {n_ranks} GPUs")
    ranks, toks, want = run_ranks(tmp_path, CFG, n_ranks, 2, 0)
    check_ranks(ranks, toks, want)
