"""Weight-file format and quantiser: this repo's writers against the reference's export_weights.py.

The golden file tests/golden/format_golden.npz was produced by importing the reference's own functions
(tests/golden/make_format_golden.py); nothing here needs the reference checkout or a GPU.
"""
import os
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest

from cuqwen_b200 import binfmt, build

GOLD = np.load(Path(__file__).parent / "golden" / "format_golden.npz")
CASES = ("a", "b", "c")


def test_constants_match_reference():
    magic, group, fp16, int8, int4 = GOLD["magic"].tolist()
    assert (magic, group, fp16, int8, int4) == (binfmt.MAGIC, binfmt.GROUP, binfmt.FP16, binfmt.INT8, binfmt.INT4)


@pytest.mark.parametrize("case", CASES)
def test_quantisers_bit_identical(case):
    w = GOLD[f"{case}_w"]
    q8, s8 = binfmt.quantize_groupwise(w, 127)
    q4, s4 = binfmt.quantize_groupwise(w, 7)
    assert np.array_equal(q8, GOLD[f"{case}_q8"]) and np.array_equal(s8.view(np.uint16), GOLD[f"{case}_s8"].view(np.uint16))
    assert np.array_equal(q4, GOLD[f"{case}_q4"]) and np.array_equal(s4.view(np.uint16), GOLD[f"{case}_s4"].view(np.uint16))


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("quant,tag", [(0, "fp16"), (1, "int8"), (2, "int4")])
def test_serialised_bytes_identical(case, quant, tag):
    w = GOLD[f"{case}_w"]
    assert binfmt.proj_bytes(w, quant) == GOLD[f"{case}_{tag}_bytes"].tobytes()
    assert len(binfmt.proj_bytes(w, quant)) == binfmt.proj_nbytes(w.shape[0], w.shape[1], quant)


def test_zero_group_and_clipping_cases():
    q4, s4 = GOLD["a_q4"], GOLD["a_s4"]
    assert s4[1, 0] == 0 and not q4[1, :128].any()              # all-zero group
    assert set(np.unique(q4[2, 128:])) <= {-7, 7}               # every |w| equal -> +-qmax
    assert q4.min() >= -7 and q4.max() <= 7                     # exporter never emits -8


@pytest.mark.parametrize("case", CASES)
def test_int4_pack_unpack_roundtrip(case):
    q4 = GOLD[f"{case}_q4"]
    packed = binfmt.pack_int4(q4)
    assert np.array_equal(binfmt.unpack_int4(packed, q4.shape[1]), q4)
    full = np.arange(-8, 8, dtype=np.int8).repeat(16).reshape(2, 128)   # the decoder handles -8 too
    assert np.array_equal(binfmt.unpack_int4(binfmt.pack_int4(full), 128), full)


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("tag", ["int8", "int4"])
def test_cxx_generator_quantiser_identical(case, tag, built, tmp_path):
    """The C++ writer used for full-size random models quantises exactly like export_weights.py."""
    from cuqwen_b200 import build
    w = GOLD[f"{case}_w"]
    src, dst = tmp_path / "w.f32", tmp_path / "out.bin"
    w.tofile(src)
    subprocess.run([str(build.GEN_BIN), "--quantize", str(src), str(w.shape[0]), str(w.shape[1]), tag, str(dst)], check=True)
    assert dst.read_bytes() == GOLD[f"{case}_{tag}_bytes"].tobytes()


def test_header_roundtrip_and_padding():
    h = binfmt.Header(151936, 896, 4864, 24, 14, 2, 64, 32768, 2, 0)
    raw = h.pack()
    assert len(raw) == 256 and raw[44:] == b"\x00" * 212
    assert struct.unpack("<i", raw[:4])[0] == 0x5157454E
    assert binfmt.Header.unpack(raw) == h
    with pytest.raises(ValueError):
        binfmt.Header.unpack(b"\x00" * 256)


def test_lm_head_format_rule():
    assert binfmt.lm_head_fmt(binfmt.FP16, tied=False) == 0
    assert binfmt.lm_head_fmt(binfmt.INT4, tied=False) == 1 and binfmt.lm_head_fmt(binfmt.INT8, tied=False) == 1
    assert binfmt.lm_head_fmt(binfmt.INT4, tied=True) == 0


@pytest.mark.parametrize("quant", [0, 1, 2])
def test_written_file_layout_and_size(quant, tmp_path):
    cfg = dict(vocab=256, dim=128, inter=256, layers=2, heads=2, kv=1, hd=64, tied=(quant != 1))
    t = binfmt.random_tensors(cfg, seed=3)
    p = tmp_path / "m.bin"
    binfmt.write_model(p, cfg, quant, t)
    raw = p.read_bytes()
    assert len(raw) == binfmt.file_nbytes(cfg, quant)
    hdr = binfmt.Header.unpack(raw)
    assert (hdr.vocab, hdr.dim, hdr.quant, hdr.lm_head_fmt) == (256, 128, quant, binfmt.lm_head_fmt(quant, cfg["tied"]))
    emb = np.frombuffer(raw, dtype=np.float16, count=256 * 128, offset=256).reshape(256, 128)
    assert np.array_equal(emb, t["model.embed_tokens.weight"].astype(np.float16))
    off = 256 + 256 * 128 * 2 + 128 * 2            # first q_proj
    blob = binfmt.proj_bytes(t["model.layers.0.self_attn.q_proj.weight"], quant)
    assert raw[off:off + len(blob)] == blob


def test_cxx_generator_file_size_and_header(built, tmp_path):
    from cuqwen_b200 import build
    p = tmp_path / "g.bin"
    subprocess.run([str(build.GEN_BIN), "--out", str(p), "--dims", "512", "256", "512", "2", "4", "2", "64", "--quant", "int4", "--untied", "--seed", "7"], check=True)
    cfg = dict(vocab=512, dim=256, inter=512, layers=2, heads=4, kv=2, hd=64, tied=False)
    assert os.path.getsize(p) == binfmt.file_nbytes(cfg, 2)
    hdr = binfmt.Header.unpack(p.read_bytes()[:256])
    assert (hdr.quant, hdr.lm_head_fmt, hdr.max_seq_len) == (2, 1, 32768)
    q = tmp_path / "g2.bin"
    subprocess.run([str(build.GEN_BIN), "--out", str(q), "--dims", "512", "256", "512", "2", "4", "2", "64", "--quant", "int4", "--untied", "--seed", "7", "--threads", "3"], check=True)
    assert p.read_bytes() == q.read_bytes()         # independent of the thread count


def test_step_byte_model_matches_published_table():
    """Algorithmic bytes per decode step for the reference's model table (weights + one embedding row + KV)."""
    expect = {("0.5b", 0): 988067328, ("0.5b", 1): 635831808, ("0.5b", 2): 456918528, ("7b", 0): 14141245440, ("7b", 1): 7181432832,
              ("7b", 2): 3918788608, ("14b", 0): 27982942208, ("14b", 1): 14210920448, ("14b", 2): 7604891648}
    for (m, q), v in expect.items():
        assert binfmt.step_bytes(binfmt.MODELS[m], q, 0) == v
    assert binfmt.step_bytes(binfmt.MODELS["7b"], 2, 8192) == 4388550656
    assert binfmt.step_bytes(binfmt.MODELS["7b"], 2, 1) - binfmt.step_bytes(binfmt.MODELS["7b"], 2, 0) == 57344


@pytest.mark.skipif(not (build.reference_dir() / "export_weights.py").exists(), reason="reference checkout not on this machine")
def test_against_reference_import_random_shapes():
    import sys
    sys.path.insert(0, str(build.reference_dir()))
    import export_weights as ew
    rng = np.random.default_rng(11)
    for rows, cols in ((5, 128), (32, 512), (7, 1152)):
        w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float32)
        for qmax, fn in ((127, ew.quantize_int8_groupwise), (7, ew.quantize_int4_groupwise)):
            q, s = binfmt.quantize_groupwise(w, qmax)
            rq, rs = fn(w)
            assert np.array_equal(q, rq) and np.array_equal(s.view(np.uint16), rs.view(np.uint16))
