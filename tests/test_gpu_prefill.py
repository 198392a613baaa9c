"""Batched-token prefill (no counterpart in the reference, which prefills token by token through the decode path,
src/main.cu:86-92; README.md:145 names the batched form as future work).

Kernel level: cuqwen_k_prefill_gemm (tcgen05 GEMM over a tile of tokens) against a float64 product of the same fp16
inputs and de-quantised weights, tolerance 2e-3 relative / 1e-2 absolute as for the decode GEMV."""
import numpy as np
import pytest

from cuqwen_b200 import binfmt
from cuqwen_b200 import kernels as K
from tests.gpu_util import DevBuf, close, dev, quant_mats, report, sync

pytestmark = pytest.mark.gpu


def dequant(w, s, quant, cols):
    if quant == 0:
        return w.astype(np.float64)
    q = binfmt.unpack_int4(w, cols) if quant == 2 else w
    return q.astype(np.float64) * np.repeat(s.astype(np.float64), 128, axis=1)


@pytest.mark.parametrize("quant", [2, 1, 0])
# the launcher takes 64- or 128-row tiles while 256-row tiles would fill less than a quarter / half of the SMs: the last
# two cases are wide enough for 128 and for 256
@pytest.mark.parametrize("T,R,Kc", [(1, 256, 128), (37, 512, 896), (128, 576, 3584), (300, 1024, 1536), (257, 264, 256), (300, 6408, 256), (600, 6408, 256)])
def test_prefill_gemm_plain_modes(built, quant, T, R, Kc):
    rng = np.random.default_rng(T * 131 + R + quant)
    x = rng.standard_normal((T, Kc)).astype(np.float16)
    w, s = quant_mats(rng, R, Kc, quant, full_range=False, sigma=0.05)
    want = x.astype(np.float64) @ dequant(w, s, quant, Kc).T
    dx, dw, ds = dev(x), dev(w), (dev(s) if s is not None else None)
    # fp32 output
    out = DevBuf(T * R * 4)
    K.prefill_gemm(quant, K.PF_OUT_F32, dx, dw, ds, out, T, R, Kc)
    sync()
    got = out.numpy(np.float32).reshape(T, R)
    assert close(got, want), "f32: " + report(got, want)
    # fp16 output with bias, into a wider row (out_stride > rows); the columns beside it stay untouched
    bias = rng.standard_normal(R).astype(np.float16)
    stride = R + 64
    canvas = np.full((T, stride), 7.0, np.float16)
    out = dev(canvas)
    K.prefill_gemm(quant, K.PF_OUT_F16, dx, dw, ds, out, T, R, Kc, out_stride=stride, bias=dev(bias))
    sync()
    got = out.numpy(np.float16).reshape(T, stride)
    assert close(got[:, :R], want + bias.astype(np.float64)), "f16+bias: " + report(got[:, :R], want + bias.astype(np.float64))
    assert (got[:, R:] == np.float16(7.0)).all()
    # residual add in place
    res = rng.standard_normal((T, R)).astype(np.float16)
    out = dev(res)
    K.prefill_gemm(quant, K.PF_RESID, dx, dw, ds, out, T, R, Kc)
    sync()
    got = out.numpy(np.float16).reshape(T, R)
    assert close(got, want + res.astype(np.float64)), "resid: " + report(got, want + res.astype(np.float64))


@pytest.mark.parametrize("quant", [2, 1, 0])
@pytest.mark.parametrize("T,R,Kc", [(5, 128, 256), (130, 320, 896), (256, 1024, 1536), (130, 4872, 256), (300, 4872, 256)])
def test_prefill_gemm_swiglu(built, quant, T, R, Kc):
    rng = np.random.default_rng(T + R * 3 + quant)
    x = rng.standard_normal((T, Kc)).astype(np.float16)
    wg, sg = quant_mats(rng, R, Kc, quant, full_range=False, sigma=0.05)
    wu, su = quant_mats(rng, R, Kc, quant, full_range=False, sigma=0.05)
    g = x.astype(np.float64) @ dequant(wg, sg, quant, Kc).T
    u = x.astype(np.float64) @ dequant(wu, su, quant, Kc).T
    want = g / (1.0 + np.exp(-g)) * u
    out = DevBuf(T * R * 2)
    K.prefill_gemm(quant, K.PF_SWIGLU, dev(x), dev(wg), dev(sg) if sg is not None else None, out, T, R, Kc,
                   w1=dev(wu), s1=dev(su) if su is not None else None)
    sync()
    got = out.numpy(np.float16).reshape(T, R)
    assert close(got, want), report(got, want)


CFGS = {
    "hd128": dict(vocab=2048, dim=512, inter=1280, layers=3, heads=4, kv=2, hd=128, tied=False),
    "hd64": dict(vocab=1024, dim=256, inter=768, layers=4, heads=4, kv=2, hd=64, tied=True),
}


@pytest.mark.parametrize("quant", [2, 1, 0])
@pytest.mark.parametrize("name", ["hd128", "hd64"])
def test_prefill_fills_the_cache_like_token_by_token_steps(built, tmp_path, quant, name):
    """Engine level: cuqwen_prefill over a prompt (two calls, the second continuing at pos0 > 0 over the first one's
    rows) against the same prompt fed through cuqwen_step: cache rows close, and the decode step that follows sees
    the same distribution."""
    from cuqwen_b200 import engine as E
    cfg = CFGS[name]
    path = tmp_path / "m.bin"
    binfmt.write_model(path, cfg, quant, binfmt.random_tensors(cfg, 11))
    max_seq = 512

    def make():
        prm = E.custom_params(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], quant, max_seq_len=max_seq)
        e = E.Engine(prm)
        e.load(str(path))
        return e

    rng = np.random.default_rng(5)
    n1, n2 = 200, 77
    toks = rng.integers(0, cfg["vocab"], size=n1 + n2 + 1).astype(np.int32)
    a, b = make(), make()
    for i in range(n1 + n2):
        a.step(int(toks[i]), i)
    b.prefill(toks[:n1], 0)
    b.prefill(toks[n1:n1 + n2], n1)
    n = n1 + n2
    shape = (cfg["layers"], cfg["kv"], max_seq, cfg["hd"])
    for which in ("KEY_CACHE", "VALUE_CACHE"):
        ca = a.read(which).reshape(shape).astype(np.float64)
        cb = b.read(which).reshape(shape).astype(np.float64)
        assert np.isfinite(cb).all()
        assert not cb[:, :, n:].any(), "rows past the prompt were written"
        for l in range(cfg["layers"]):
            rms = np.sqrt(((ca[l, :, :n] - cb[l, :, :n]) ** 2).mean()) / np.sqrt((ca[l, :, :n] ** 2).mean())
            print(f"{which} layer {l}: rel rms {rms:.2e}")
            assert rms < 6e-3, f"{which} layer {l}: rel rms {rms:.3e}"
        assert close(cb[:, :, :n], ca[:, :, :n], rtol=2e-2, atol=3e-2), report(cb[:, :, :n], ca[:, :, :n])
    ta, tb = a.step(int(toks[n]), n), b.step(int(toks[n]), n)
    la, lb = a.read("LOGITS").astype(np.float64), b.read("LOGITS").astype(np.float64)
    rms = np.sqrt(((la - lb) ** 2).mean()) / np.sqrt((la ** 2).mean())
    print(f"logits after the prompt: rel rms {rms:.2e}, tokens {ta} / {tb}")
    assert rms < 1.5e-2
    assert ta == tb or abs(la[ta] - la[tb]) <= 2e-3 * abs(la[ta]) + 1e-2
    a.close(); b.close()


def test_prefill_rejects_what_it_cannot_do(built, tmp_path):
    from cuqwen_b200 import engine as E
    from cuqwen_b200._abi import CuQwenError
    cfg = CFGS["hd128"]
    path = tmp_path / "m.bin"
    binfmt.write_model(path, cfg, 2, binfmt.random_tensors(cfg, 11))
    prm = E.custom_params(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], 2, max_seq_len=256)
    e = E.Engine(prm)
    e.load(str(path))
    with pytest.raises(CuQwenError):
        e.prefill(np.zeros(300, np.int32), 0)            # runs past the cache
    with pytest.raises(CuQwenError):
        e.prefill(np.array([cfg["vocab"]], np.int32), 0)  # token out of range
    with pytest.raises(CuQwenError):
        e.prefill(np.array([1, 2], np.int32), -1)
    e.prefill(np.array([1, 2, 3], np.int32), 0)           # and the engine still works
    e.close()


@pytest.mark.parametrize("model,quant,n", [("0.5b", "int4", 300), ("0.5b", "fp16", 130), ("7b", "int4", 384)])
def test_prefill_vs_reference_build_token_by_token(built, tmpdir_big, model, quant, n):
    """Against the reference's own CUDA build at full model size: the reference prefills by n calls of qwen_forward
    (src/main.cu:86-92), this engine by one cuqwen_prefill; both then decode eight teacher-forced steps.  Bar: the
    whole-step criterion (top-1 agreement within the fp16 contract on every step, rms logit difference <= 1.5 %)."""
    import shutil
    import subprocess
    from cuqwen_b200 import build
    from cuqwen_b200 import engine as E
    from oracle import oracle_py as O
    from tests.gpu_util import RTOL
    ref = O.ref_lib(model, quant)
    if ref is None:
        pytest.skip("oracle/_ref not built")
    cfg = binfmt.MODELS[model]
    if shutil.disk_usage(tmpdir_big).free < binfmt.file_nbytes(cfg, binfmt.QUANT_ID[quant]) + (2 << 30):
        pytest.skip("not enough room for the model file")
    path = tmpdir_big / f"pf_{model}_{quant}.bin"
    subprocess.run([str(build.GEN_BIN), "--out", str(path), "--model", model, "--quant", quant, "--seed", "42"], check=True)
    V = cfg["vocab"]
    rng = np.random.default_rng(9)
    toks = rng.integers(0, V, size=n).astype(np.int32)
    try:
        prm = E.model_params(model, quant)
        prm.max_seq_len = 1024
        eng = E.Engine(prm)
        eng.load(str(path))
        rm = ref.ref_model_load(str(path).encode())
        for i in range(n - 1):
            ref.ref_forward(rm, int(toks[i]), i, None, 0)
        eng.prefill(toks[:n - 1], 0)
        tok, agree, worst = int(toks[n - 1]), 0, 0.0
        steps = 8
        for i in range(steps):
            tok_r = ref.ref_forward(rm, tok, n - 1 + i, None, 0)
            tok_e = eng.step(tok, n - 1 + i)
            lr = E.download(0, ref.ref_state_ptr(rm, 0), np.float16, V).astype(np.float32)
            le = eng.read("LOGITS").astype(np.float32)
            assert np.isfinite(le).all()
            d = le - lr
            worst = max(worst, float(np.sqrt((d * d).mean()) / np.sqrt((lr * lr).mean())))
            agree += tok_e == tok_r or abs(lr[tok_r] - lr[tok_e]) <= RTOL * abs(lr[tok_r]) + 1e-3
            tok = tok_r
        ref.ref_model_free(rm)
        eng.close()
    finally:
        path.unlink()
    print(f"{model} {quant}, prompt {n}: top-1 agreement {agree}/{steps}, rel rms of the logits {worst:.2e}")
    assert agree == steps and worst <= 1.5e-2


def test_prefill_longer_than_one_chunk_and_single_token(built, tmp_path):
    """A prompt longer than the 2048-token chunk the engine works in (the second chunk attends to the first one's
    rows), and the smallest call (one token at an odd position), against the token-by-token path."""
    from cuqwen_b200 import engine as E
    cfg = dict(vocab=512, dim=256, inter=512, layers=2, heads=2, kv=1, hd=128, tied=True)
    path = tmp_path / "m.bin"
    binfmt.write_model(path, cfg, 2, binfmt.random_tensors(cfg, 3))
    max_seq = 2432

    def make():
        e = E.Engine(E.custom_params(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], 2, max_seq_len=max_seq))
        e.load(str(path))
        return e

    rng = np.random.default_rng(2)
    n = 2048 + 331
    toks = rng.integers(0, cfg["vocab"], size=n + 2).astype(np.int32)
    a, b = make(), make()
    for i in range(n + 1):
        a.step(int(toks[i]), i)
    b.prefill(toks[:n], 0)
    b.prefill(toks[n:n + 1], n)
    shape = (cfg["layers"], cfg["kv"], max_seq, cfg["hd"])
    for which in ("KEY_CACHE", "VALUE_CACHE"):
        ca = a.read(which).reshape(shape).astype(np.float64)[:, :, :n + 1]
        cb = b.read(which).reshape(shape).astype(np.float64)[:, :, :n + 1]
        rms = np.sqrt(((ca - cb) ** 2).mean()) / np.sqrt((ca ** 2).mean())
        tail = np.sqrt(((ca[:, :, 2048:] - cb[:, :, 2048:]) ** 2).mean()) / np.sqrt((ca[:, :, 2048:] ** 2).mean())
        print(f"{which}: rel rms {rms:.2e} (rows of the second chunk {tail:.2e})")
        assert rms < 5e-3 and tail < 5e-3
    ta, tb = a.step(int(toks[n + 1]), n + 1), b.step(int(toks[n + 1]), n + 1)
    la, lb = a.read("LOGITS").astype(np.float64), b.read("LOGITS").astype(np.float64)
    rms = np.sqrt(((la - lb) ** 2).mean()) / np.sqrt((la ** 2).mean())
    print(f"logits: rel rms {rms:.2e}, tokens {ta} / {tb}")
    assert rms < 1.5e-2
    a.close(); b.close()


def attn_oracle(q, Kc, Vc, pos0, nh, nkv, hd):
    """float64 causal attention: q [T][nh*hd], caches [nkv][max_seq][hd]; query t sees keys [0, pos0 + t]."""
    T = q.shape[0]
    grp = nh // nkv
    out = np.empty((T, nh * hd))
    for h in range(nh):
        kv = h // grp
        qh = q[:, h * hd:(h + 1) * hd].astype(np.float64)
        s = qh @ Kc[kv, :pos0 + T].astype(np.float64).T / np.sqrt(hd)
        mask = np.arange(pos0 + T)[None, :] > (pos0 + np.arange(T))[:, None]
        s[mask] = -np.inf
        p = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h * hd:(h + 1) * hd] = (p / p.sum(axis=1, keepdims=True)) @ Vc[kv, :pos0 + T].astype(np.float64)
    return out


@pytest.mark.parametrize("impl,hd", [(0, 128), (0, 64), (1, 128), (1, 64)])
@pytest.mark.parametrize("T,pos0,nh,nkv", [(1, 0, 4, 2), (37, 0, 4, 2), (128, 5, 2, 1), (300, 0, 7, 1), (200, 333, 4, 4), (513, 129, 2, 2)])
def test_prefill_attention_kernels(built, impl, hd, T, pos0, nh, nkv):
    rng = np.random.default_rng(T * 7 + pos0 + nh + hd)
    max_seq = (pos0 + T + 70) // 8 * 8
    q = rng.standard_normal((T, nh * hd)).astype(np.float16)
    Kc = rng.standard_normal((nkv, max_seq, hd)).astype(np.float16)
    Vc = rng.standard_normal((nkv, max_seq, hd)).astype(np.float16)
    want = attn_oracle(q, Kc, Vc, pos0, nh, nkv, hd)
    # rows past the last query are never attended to: huge values there must not leak into any output
    Kp, Vp = Kc.copy(), Vc.copy()
    Kp[:, pos0 + T:] = 60000.0; Vp[:, pos0 + T:] = -60000.0
    out = DevBuf(T * nh * hd * 2)
    K.prefill_attention(impl, dev(q), dev(Kp), dev(Vp), out, T, pos0, nh, nkv, hd, max_seq)
    sync()
    got = out.numpy(np.float16).reshape(T, nh * hd)
    assert np.isfinite(got.astype(np.float32)).all()
    assert close(got, want), report(got, want)
