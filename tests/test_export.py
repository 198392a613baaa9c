"""The streaming exporter (cuqwen_b200/export.py) writes, byte for byte, what the reference's export_weights.py wrote
for the same checkpoint directory: tests/golden/export_golden.json holds the hashes of the reference's outputs
(made by tests/golden/make_export_golden.py with the reference's own functions)."""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import pytest

from cuqwen_b200 import binfmt, export

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN_DIR))
import export_case  # noqa: E402

GOLDEN = json.loads((GOLDEN_DIR / "export_golden.json").read_text())


def sha(path) -> str:
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


@pytest.fixture(scope="module")
def checkpoints(tmp_path_factory):
    root = tmp_path_factory.mktemp("ckpt")
    dirs = {name: export_case.write_case(name, root) for name in export_case.CASES}
    for name, d in dirs.items():
        assert {p.name: sha(p) for p in sorted(d.iterdir())} == GOLDEN[name]["inputs"], "the synthetic checkpoint differs from the one the golden was made from"
    return dirs


@pytest.mark.parametrize("case", sorted(export_case.CASES))
@pytest.mark.parametrize("quant", ["fp16", "int8", "int4"])
@pytest.mark.parametrize("block", [64 << 20, 4096])
def test_model_file_is_byte_identical_to_the_reference_exporters(checkpoints, tmp_path, monkeypatch, case, quant, block):
    monkeypatch.setattr(export, "ROW_BLOCK_BYTES", block)      # small blocks: many partial row blocks per tensor
    out = tmp_path / "m.bin"
    n = export.export_weights(checkpoints[case], out, quant)
    want = GOLDEN[case]["bins"][quant]
    assert n == out.stat().st_size == want["size"]
    assert out.read_bytes()[:64].hex() == want["head"]
    assert sha(out) == want["sha256"]


@pytest.mark.parametrize("case", sorted(export_case.CASES))
def test_tokenizer_json_is_byte_identical(checkpoints, tmp_path, case):
    out = tmp_path / "ranks.json"
    export.export_tokenizer(checkpoints[case], out)
    assert out.stat().st_size == GOLDEN[case]["tokenizer_size"] and sha(out) == GOLDEN[case]["tokenizer_sha256"]


def test_exported_ranks_file_loads_in_the_tokenizer(checkpoints, tmp_path):
    from cuqwen_b200 import build
    from cuqwen_b200 import tokenizer as T
    build.build_tokenizer()
    out = tmp_path / "ranks.json"
    export.export_tokenizer(checkpoints["tied_bf16"], out)
    with T.QwenTokenizer(out) as t:
        assert t.special_count == 3
        ids = t.encode("hello world<|im_end|>\n\n")
        vocab = json.loads((checkpoints["tied_bf16"] / "vocab.json").read_text(encoding="utf-8"))
        assert ids[0] == vocab["hello"] and ids[1] == vocab["Ġw"] and (len(vocab) + 1) in ids
        assert t.decode_bytes(ids[:2]) == b"hello w"


def test_exported_file_matches_the_header_and_size_rules(checkpoints, tmp_path):
    c = export_case.CASES["untied_mixed"]
    out = tmp_path / "m.bin"
    export.export_weights(checkpoints["untied_mixed"], out, "int4")
    h = binfmt.Header.unpack(out.read_bytes()[:256])
    assert (h.vocab, h.dim, h.inter, h.layers, h.heads, h.kv, h.hd) == (c["vocab"], c["dim"], c["inter"], c["layers"], c["heads"], c["kv"], c["dim"] // c["heads"])
    assert h.quant == binfmt.INT4 and h.lm_head_fmt == 1 and h.max_seq_len == 32768
    cfg = dict(vocab=c["vocab"], dim=c["dim"], inter=c["inter"], layers=c["layers"], heads=c["heads"], kv=c["kv"], hd=h.hd, tied=False)
    assert out.stat().st_size == binfmt.file_nbytes(cfg, binfmt.INT4)


def test_reader_converts_like_the_reference(checkpoints):
    with export.SafetensorsDir(checkpoints["untied_mixed"]) as st:
        table = dict(export_case.tensor_table(export_case.CASES["untied_mixed"]))
        seen = set()
        for key, (_, dtype, shape, _, _) in st.entries.items():
            src = table[key]
            if dtype == "BF16":
                want = ((src.view(np.uint32) >> 16) << 16).view(np.float32).astype(np.float16)
            else:
                want = src.astype(np.float16)
            got = st.rows(key)
            assert got.dtype == np.float16 and list(got.shape) == shape and np.array_equal(got, want), key
            if len(shape) == 2:
                assert np.array_equal(st.rows(key, 3, 7), want[3:7])
            seen.add(dtype)
        assert seen == {"BF16", "F16", "F32"}
        assert st.contains("lm_head") and not st.contains("rotary")
        with pytest.raises(KeyError):
            st.rows("model.layers.99.mlp.up_proj.weight")


def test_errors(tmp_path, checkpoints):
    with pytest.raises(FileNotFoundError):
        export.SafetensorsDir(tmp_path)
    with pytest.raises(KeyError):
        export.export_weights(checkpoints["tied_bf16"], tmp_path / "x.bin", "int3")


def test_cli(checkpoints, tmp_path, monkeypatch, capsys):
    monkeypatch.chdir(tmp_path)
    assert export.main(["--model-dir", str(checkpoints["tied_bf16"]), "--model", "0.5b", "--quantization", "int8"]) == 0
    assert sha(tmp_path / "weights" / "model_int8_0_5b.bin") == GOLDEN["tied_bf16"]["bins"]["int8"]["sha256"]
    assert sha(tmp_path / "weights" / "qwen25_bpe_ranks.json") == GOLDEN["tied_bf16"]["tokenizer_sha256"]
