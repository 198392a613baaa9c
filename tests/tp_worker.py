"""One tensor-parallel rank for tests/test_gpu_tp.py: python tp_worker.py <rank> <size> <dir> <model.bin> <quant> <flags>.

Rank 0 publishes the NCCL id through a file in <dir>; every rank runs the same teacher-forced steps and leaves its
tokens and its slice of the last logits in <dir>/rank<r>.npz."""
import json
import os
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from cuqwen_b200 import engine as E  # noqa: E402


def main():
    rank, size, d, path, quant, flags = int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3]), sys.argv[4], int(sys.argv[5]), int(sys.argv[6])
    cfg = json.loads((d / "cfg.json").read_text())
    prm = E.custom_params(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], quant, max_seq_len=128)
    prm.device, prm.tp_rank, prm.tp_size, prm.flags = rank, rank, size, flags
    eng = E.Engine(prm)
    eng.load(path)
    idf = d / "nccl_id.bin"
    if rank == 0:
        tmp = d / "nccl_id.tmp"
        tmp.write_bytes(E.nccl_unique_id())
        tmp.rename(idf)
    else:
        t0 = time.time()
        while not idf.exists():
            if time.time() - t0 > 60:
                raise RuntimeError("no NCCL id from rank 0")
            time.sleep(0.05)
    eng.tp_init(idf.read_bytes())
    eng.kv_fill_normal(64, seed=9)
    toks = [eng.step(3 + i, 64 + i) for i in range(12)]                       # teacher-forced, host round trip per step
    toks += eng.decode_n(toks[-1], 76, 10).tolist()                           # device-side feedback
    np.savez(d / f"rank{rank}.npz", toks=np.array(toks), logits=eng.read("LOGITS"), launches=eng.step_launches)
    eng.close()


if __name__ == "__main__":
    main()
