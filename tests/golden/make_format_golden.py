"""Generate tests/golden/format_golden.npz by importing the reference's own export_weights.py.

Run where the CuQwen checkout is available:  python tests/golden/make_format_golden.py [<CuQwen checkout>]
The fixture pins the quantiser and the serialised byte layout (write_fp16 / write_int8 / write_int4) on small
seeded matrices, including an all-zero group, exact half-way cases and values that clip.
"""
import io
import os
import sys
import types
from pathlib import Path

import numpy as np

ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CUQWEN_REFERENCE_DIR") or Path(__file__).resolve().parents[3] / "reference")
sys.modules.setdefault("huggingface_hub", types.SimpleNamespace(snapshot_download=None))   # network helper, unused here
sys.path.insert(0, str(ref))
import export_weights as ew  # noqa: E402

rng = np.random.default_rng(20251125)
cases = {}
for name, (rows, cols, sigma) in {"a": (8, 256, 0.02), "b": (16, 896, 0.02), "c": (3, 128, 1.0)}.items():
    w = (sigma * rng.standard_normal((rows, cols))).astype(np.float32)
    if name == "a":
        w[1, :128] = 0.0                                  # all-zero group -> scale 0
        w[2, 128:] = np.float32(0.07) * np.sign(w[2, 128:])  # every |w| equal: q = +-qmax
        w[3, :128] = np.linspace(-1, 1, 128, dtype=np.float32) * np.float32(3.5)   # exact .5 multiples of scale 0.5 (int4)
    cases[name] = w
out = {}
for name, w in cases.items():
    out[f"{name}_w"] = w
    for tag, fn in (("fp16", ew.write_fp16), ("int8", ew.write_int8), ("int4", ew.write_int4)):
        buf = io.BytesIO()
        fn(buf, w)
        out[f"{name}_{tag}_bytes"] = np.frombuffer(buf.getvalue(), dtype=np.uint8)
    q8, s8 = ew.quantize_int8_groupwise(w)
    q4, s4 = ew.quantize_int4_groupwise(w)
    out[f"{name}_q8"], out[f"{name}_s8"], out[f"{name}_q4"], out[f"{name}_s4"] = q8, s8, q4, s4
out["magic"] = np.array([ew.MAGIC_NUMBER, ew.QUANT_GROUP, ew.QUANT_FP16, ew.QUANT_INT8, ew.QUANT_INT4], dtype=np.int64)
np.savez_compressed(Path(__file__).resolve().parent / "format_golden.npz", **out)
print("wrote format_golden.npz with", len(out), "arrays")
