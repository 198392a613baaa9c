"""The 8-bit KV cache (CUQWEN_FLAG_KV_INT8; opt-in, outside the reference's parity contract - its roadmap names it,
README.md:147).  The cache holds int8 rows with one fp32 scale per token and KV head, scale = max|row| / 127.

Kernel level: cuqwen_k_attention_kv8 against a float64 softmax(q K^T / sqrt(d)) V over the de-quantised rows (the
same quantiser in numpy), tolerance 2e-3 relative / 1e-2 absolute as for the fp16 kernel; the row the kernel stores
for the step's own key / value must equal the numpy quantiser's output bit for bit.
Engine level: a small model decoded with the 8-bit cache stays close to the same model with the fp16 cache."""
import numpy as np
import pytest

from cuqwen_b200 import binfmt
from cuqwen_b200 import engine as E
from cuqwen_b200 import kernels as K
from tests.gpu_util import DevBuf, close, dev, dint, report, sync

pytestmark = pytest.mark.gpu


def quantise_rows(x):
    """x [..., hd] fp16 -> (int8 rows, fp32 scales): what kv8_store_row / fill_normal_q8_kernel compute."""
    v = x.astype(np.float32)
    m = np.abs(v).max(axis=-1)
    inv = np.where(m > 0, np.float32(127.0) / np.where(m > 0, m, 1).astype(np.float32), np.float32(0)).astype(np.float32)
    q = np.rint(v * inv[..., None]).astype(np.int8)
    return q, (m / np.float32(127.0)).astype(np.float32)


def oracle(q, Kd, Vd, nh, nkv, hd, length):
    """float64 attention; Kd / Vd [nkv][length][hd] already de-quantised (float64)."""
    grp = nh // nkv
    out = np.empty((nh, hd))
    for h in range(nh):
        kv = h // grp
        s = Kd[kv, :length] @ q[h].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ Vd[kv, :length]
    return out.reshape(-1)


@pytest.mark.parametrize("nh,nkv,hd", [(28, 4, 128), (40, 8, 128), (14, 2, 64)])
@pytest.mark.parametrize("length", [1, 2, 17, 64, 65, 300, 2048])
def test_attention_over_int8_cache(built, nh, nkv, hd, length):
    rng = np.random.default_rng(length * 7 + nh)
    max_seq = (length + 40) // 4 * 4
    q = rng.standard_normal((nh, hd)).astype(np.float16)
    Kf = rng.standard_normal((nkv, max_seq, hd)).astype(np.float16)
    Vf = rng.standard_normal((nkv, max_seq, hd)).astype(np.float16)
    pos = length - 1
    K8, Ks = quantise_rows(Kf)
    V8, Vs = quantise_rows(Vf)
    # rows from pos on are not in the cache: poison them (scales NaN, bytes arbitrary) - the kernel must not read them
    K8c, V8c, Ksc, Vsc = K8.copy(), V8.copy(), Ks.copy(), Vs.copy()
    K8c[:, pos:] = 77; V8c[:, pos:] = -77; Ksc[:, pos:] = np.nan; Vsc[:, pos:] = np.nan
    pad = np.full((nkv, 4), np.nan, np.float32)             # the scale arrays have room past the last row
    dk, dv = dev(K8c), dev(V8c)
    dks, dvs = dev(np.concatenate([Ksc.reshape(-1), pad.reshape(-1)])), dev(np.concatenate([Vsc.reshape(-1), pad.reshape(-1)]))
    kcur, vcur = np.ascontiguousarray(Kf[:, pos]), np.ascontiguousarray(Vf[:, pos])
    Kd = K8.astype(np.float64) * Ks[..., None].astype(np.float64)
    Vd = V8.astype(np.float64) * Vs[..., None].astype(np.float64)
    Kd[:, pos] = kcur.astype(np.float64); Vd[:, pos] = vcur.astype(np.float64)      # the step's own key / value are attended to in fp16
    want = oracle(q, Kd, Vd, nh, nkv, hd, length)
    for nsplit in (1, 18, 37):
        bo, bml, _ = K.attn_scratch_bytes(nkv, hd, nsplit)
        so, sml, out = DevBuf(bo), DevBuf(bml), DevBuf(nh * hd * 2)
        K.gqa_attention_decode_kv8(dev(q), dk, dv, dks, dvs, dev(kcur), dev(vcur), out, dint(pos), nh, nkv, hd, max_seq, nsplit, so, sml)
        sync()
        got = out.numpy(np.float16)
        assert np.isfinite(got.astype(np.float32)).all(), f"nsplit {nsplit}"
        assert close(got, want), f"nsplit {nsplit}: " + report(got, want)
        # the stored row: exactly the quantiser's output, and nothing else touched
        k_after = dk.numpy(np.int8).reshape(nkv, max_seq, hd)
        v_after = dv.numpy(np.int8).reshape(nkv, max_seq, hd)
        ks_after = dks.numpy(np.float32)[:nkv * max_seq].reshape(nkv, max_seq)
        assert np.array_equal(k_after[:, pos], K8[:, pos]) and np.array_equal(v_after[:, pos], V8[:, pos])
        assert np.array_equal(ks_after[:, pos].view(np.uint32), Ks[:, pos].view(np.uint32))
        assert (k_after[:, pos + 1:] == 77).all() and (v_after[:, :pos] == V8[:, :pos]).all()


def test_small_model_with_int8_cache_tracks_the_fp16_cache(built, tmp_path):
    cfg = dict(vocab=2048, dim=384, inter=768, layers=3, heads=6, kv=2, hd=128, tied=False)
    path = tmp_path / "m.bin"
    binfmt.write_model(path, cfg, 2, binfmt.random_tensors(cfg, 3))

    def make(flags):
        prm = E.custom_params(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], 2, max_seq_len=256)
        prm.flags = flags
        e = E.Engine(prm)
        e.load(str(path))
        e.kv_fill_normal(100, seed=5)
        return e

    a, b = make(0), make(E.FLAG_KV_INT8)
    assert b.step_bytes(100) < a.step_bytes(100)
    worst, same = 0.0, 0
    for i in range(24):
        ta, tb = a.step(7 + i, 100 + i), b.step(7 + i, 100 + i)
        la, lb = a.read("LOGITS").astype(np.float32), b.read("LOGITS").astype(np.float32)
        assert np.isfinite(lb).all()
        worst = max(worst, float(np.sqrt(((la - lb) ** 2).mean()) / np.sqrt((la ** 2).mean())))
        same += ta == tb
    print(f"int8 KV cache vs fp16: rel rms of the logits {worst:.2e}, identical greedy token {same}/24")
    assert worst < 3e-2 and same >= 20
    # rows written during the steps are int8 with a positive scale; rows never written stay zero
    k8 = b.read("KEY_CACHE", dtype=np.int8).reshape(cfg["layers"], cfg["kv"], 256, cfg["hd"])
    ks = b.read("KEY_SCALE", dtype=np.float32).reshape(cfg["layers"], cfg["kv"], 256)
    assert (ks[:, :, :124] > 0).all() and not k8[:, :, 124:].any() and not ks[:, :, 124:].any()
    assert (np.abs(k8[:, :, 100:124].astype(np.int32)).max(axis=-1) == 127).all()        # every stored row uses the full range
    toks = b.decode_n(3, 124, 16)
    assert len(toks) == 16
    a.close(); b.close()
