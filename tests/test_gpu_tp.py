"""Tensor parallelism on two GPUs of one node: one process per GPU (tests/tp_worker.py), compared with the single-GPU
engine on the same model.  Both exchange paths are covered: partials pushed with peer stores (default) and NCCL
all-reduce calls (CUQWEN_FLAG_TP_NCCL).  Skipped on a box with one GPU."""
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


def gpu_count() -> int:
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for ln in out.splitlines() if ln.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.parametrize("flags,sum_kernel", [(0, 0), (0, 1), (E.FLAG_TP_NCCL, 0)], ids=["peer_stores", "peer_stores_sum_kernel", "nccl_allreduce"])
@pytest.mark.parametrize("quant", [2, 0])
def test_two_ranks_match_one_gpu(built, tmp_path, monkeypatch, quant, flags, sum_kernel):
    if gpu_count() < 2:
        pytest.skip("needs two GPUs")
    path = tmp_path / "m.bin"
    binfmt.write_model(path, CFG, quant, binfmt.random_tensors(CFG, 4))
    (tmp_path / "cfg.json").write_text(json.dumps(CFG))
    monkeypatch.setenv("CUQWEN_TP_SUM_KERNEL", str(sum_kernel))      # 1: the many-rank variant (slots summed once by a small kernel)
    worker = Path(__file__).with_name("tp_worker.py")
    procs = [subprocess.Popen([sys.executable, str(worker), str(r), "2", str(tmp_path), str(path), str(quant), str(flags)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)

    prm = E.custom_params(CFG["vocab"], CFG["dim"], CFG["inter"], CFG["layers"], CFG["heads"], CFG["kv"], CFG["hd"], quant, max_seq_len=128)
    one = E.Engine(prm)
    one.load(str(path))
    one.kv_fill_normal(64, seed=9)
    toks = [one.step(3 + i, 64 + i) for i in range(12)]
    toks += one.decode_n(toks[-1], 76, 10).tolist()
    want = one.read("LOGITS")
    one.close()

    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    assert r0["toks"].tolist() == r1["toks"].tolist()                       # every rank learns the same token
    per_layer = 10 if flags else 8 if sum_kernel else 6                       # 6 = qkv, attention x2, o_proj, gate/up, down; NCCL adds an all-reduce and a residual kernel twice, the sum kernel adds 2
    assert int(r0["launches"]) == 1 + per_layer * CFG["layers"] + 3 + 2       # ... + key all-gather and merge
    got = np.concatenate([r0["logits"], r1["logits"]])
    assert close(got, want), report(got, want)
    same = sum(a == b for a, b in zip(r0["toks"].tolist()[:12], toks[:12]))   # teacher-forced steps are independent of one another
    assert same >= 10, (r0["toks"].tolist(), toks)
