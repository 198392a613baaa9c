"""Generate tests/golden/export_golden.json by running the reference's own export_weights.py (its export_weights and
export_tokenizer functions, unmodified) on the synthetic checkpoint directories of export_case.py.

Run where the CuQwen checkout is available:  python tests/golden/make_export_golden.py [<CuQwen checkout>]
The fixture holds, per case and precision, the SHA-256, size and first 64 bytes of the reference's .bin, and the
SHA-256 of its tokenizer JSON, plus the SHA-256 of every input file so a test can tell that it rebuilt the same
checkpoint.
"""
import contextlib
import hashlib
import io
import json
import os
import sys
import tempfile
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import export_case  # noqa: E402

ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CUQWEN_REFERENCE_DIR") or Path(__file__).resolve().parents[3] / "reference")
sys.modules.setdefault("huggingface_hub", types.SimpleNamespace(snapshot_download=None))   # network helper, unused here
sys.path.insert(0, str(ref))
import export_weights as ew  # noqa: E402


def sha(path) -> str:
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


golden = {}
with tempfile.TemporaryDirectory() as tmp:
    os.chdir(tmp)                       # the reference writes to ./weights
    for case in export_case.CASES:
        model_dir = export_case.write_case(case, Path(tmp) / "ckpt")
        entry = {"inputs": {p.name: sha(p) for p in sorted(model_dir.iterdir())}, "bins": {}}
        for quant in ("fp16", "int8", "int4"):
            with contextlib.redirect_stdout(io.StringIO()):
                ew.export_weights(str(model_dir), "0.5b", quant)
            out = Path("weights") / f"model_{quant}_0_5b.bin"
            raw = out.read_bytes()
            entry["bins"][quant] = {"sha256": hashlib.sha256(raw).hexdigest(), "size": len(raw), "head": raw[:64].hex()}
            out.unlink()
        with contextlib.redirect_stdout(io.StringIO()):
            ew.export_tokenizer(str(model_dir))
        entry["tokenizer_sha256"] = sha(ew.OUTPUT_BPE_PATH)
        entry["tokenizer_size"] = Path(ew.OUTPUT_BPE_PATH).stat().st_size
        golden[case] = entry
    os.chdir(HERE)

(HERE / "export_golden.json").write_text(json.dumps(golden, indent=1) + "\n")
print("wrote export_golden.json:", {k: {q: v["size"] for q, v in e["bins"].items()} for k, e in golden.items()})
