"""CuQwen's binary weight format: header, tensor order, quantisers, byte model.

File layout (CuQwen export_weights.py:267-323, src/load_weights.cpp:46-161),
little-endian: 11 int32 {magic 0x5157454E, vocab, dim, inter, n_layers, n_heads,
n_kv_heads, head_dim, max_seq_len, quant_type, lm_head_fmt} zero-padded to 256
bytes; embed_tokens [V,d] fp16; per layer input_layernorm, q_proj P, q_bias,
k_proj P, k_bias, v_proj P, v_bias, o_proj P, post_attention_layernorm,
gate_proj P, up_proj P, down_proj P; norm; lm_head (int8 P if lm_head_fmt == 1,
fp16 [V,d] if untied, absent if tied).  P = fp16 [out,in] | int8 [out,in] +
fp16 scales [out,in/128] | packed int4 [out,in/2] + scales.

This module is host-side tooling (numpy); it does not run on the decode path.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

MAGIC = 0x5157454E
GROUP = 128
FP16, INT8, INT4 = 0, 1, 2
QUANT_ID = {"fp16": FP16, "int8": INT8, "int4": INT4}

MODELS = {  # CuQwen include/config.h:55-113
    "0.5b": dict(vocab=151936, dim=896, inter=4864, layers=24, heads=14, kv=2, hd=64, tied=True),
    "1.5b": dict(vocab=151936, dim=1536, inter=8960, layers=28, heads=12, kv=2, hd=128, tied=True),
    "3b": dict(vocab=151936, dim=2048, inter=11008, layers=36, heads=16, kv=2, hd=128, tied=True),
    "7b": dict(vocab=152064, dim=3584, inter=18944, layers=28, heads=28, kv=4, hd=128, tied=False),
    "14b": dict(vocab=152064, dim=5120, inter=13824, layers=48, heads=40, kv=8, hd=128, tied=False),
}


@dataclass
class Header:
    vocab: int
    dim: int
    inter: int
    layers: int
    heads: int
    kv: int
    hd: int
    max_seq_len: int
    quant: int
    lm_head_fmt: int

    def pack(self) -> bytes:
        h = struct.pack("<11i", MAGIC, self.vocab, self.dim, self.inter, self.layers, self.heads, self.kv, self.hd,
                        self.max_seq_len, self.quant, self.lm_head_fmt)
        return h + b"\x00" * (256 - len(h))

    @classmethod
    def unpack(cls, raw: bytes) -> "Header":
        f = struct.unpack("<11i", raw[:44])
        if f[0] != MAGIC:
            raise ValueError(f"magic mismatch: 0x{f[0] & 0xffffffff:x}")
        return cls(*f[1:])


def quantize_groupwise(w: np.ndarray, qmax: int):
    """Symmetric per-row, per-128-column quantisation (export_weights.py:123-183).

    scale = max|w| / qmax in fp32; q = clip(round_half_even(w / scale_fp32)); the stored scale is the fp16
    rounding of scale_fp32; an all-zero group gets scale 0 and q 0.
    """
    w = np.asarray(w, dtype=np.float32)
    rows, cols = w.shape
    if cols % GROUP:
        raise ValueError(f"in_features={cols} not divisible by {GROUP}")
    g = w.reshape(rows, cols // GROUP, GROUP)
    scale = np.abs(g).max(axis=2) / np.float32(qmax)
    safe = np.where(scale > 0, scale, np.float32(1.0)).astype(np.float32)
    q = np.clip(np.rint(g / safe[:, :, None]), -qmax, qmax).astype(np.int8)
    return q.reshape(rows, cols), scale.astype(np.float16)


def pack_int4(q: np.ndarray) -> np.ndarray:
    """Two 4-bit two's-complement values per byte: element 2p low nibble, 2p+1 high (export_weights.py:198-199)."""
    n = (q.astype(np.int16) & 0xF).astype(np.uint8)
    return (n[:, 0::2] | (n[:, 1::2] << 4)).astype(np.uint8)


def unpack_int4(packed: np.ndarray, cols: int) -> np.ndarray:
    lo = (packed & 0xF).astype(np.int8)
    hi = (packed >> 4).astype(np.int8)
    lo = ((lo ^ 8) - 8).astype(np.int8)
    hi = ((hi ^ 8) - 8).astype(np.int8)
    out = np.empty((packed.shape[0], cols), dtype=np.int8)
    out[:, 0::2], out[:, 1::2] = lo, hi
    return out


def proj_bytes(w: np.ndarray, quant: int) -> bytes:
    """Serialise one projection matrix the way export_weights.write_fp16/int8/int4 do."""
    if quant == FP16:
        return np.asarray(w).astype(np.float16).tobytes()
    if quant == INT8:
        q, s = quantize_groupwise(w, 127)
        return q.tobytes() + s.tobytes()
    q, s = quantize_groupwise(w, 7)
    return pack_int4(q).tobytes() + s.tobytes()


def proj_nbytes(rows: int, cols: int, quant: int) -> int:
    w = rows * cols * 2 if quant == FP16 else rows * cols if quant == INT8 else rows * cols // 2
    return w + (rows * (cols // GROUP) * 2 if quant else 0)


def lm_head_fmt(quant: int, tied: bool) -> int:
    """INT8 head iff the build is quantised and the head is a separate tensor (export_weights.py:261)."""
    return 1 if (quant != FP16 and not tied) else 0


def file_nbytes(cfg: dict, quant: int) -> int:
    d, qd, kd, I, V = cfg["dim"], cfg["heads"] * cfg["hd"], cfg["kv"] * cfg["hd"], cfg["inter"], cfg["vocab"]
    layer = (2 * d * 2 + proj_nbytes(qd, d, quant) + qd * 2 + 2 * (proj_nbytes(kd, d, quant) + kd * 2) + proj_nbytes(d, qd, quant)
             + 2 * proj_nbytes(I, d, quant) + proj_nbytes(d, I, quant))
    n = 256 + V * d * 2 + cfg["layers"] * layer + d * 2
    if not cfg["tied"]:
        n += proj_nbytes(V, d, INT8) if quant else V * d * 2
    return n


def step_bytes(cfg: dict, quant: int, ctx: int, kv_int8: bool = False) -> int:
    """Algorithmic bytes of one decode step: every weight/scale/bias/norm byte once, one embedding row, and the
    K and V rows [0, ctx) of every layer (fp16, or int8 plus one fp32 scale per row and KV head).  Activations,
    partials, logits and the KV write are not counted."""
    d, I, V = cfg["dim"], cfg["inter"], cfg["vocab"]
    qd, kd = cfg["heads"] * cfg["hd"], cfg["kv"] * cfg["hd"]
    layer = (2 * d * 2 + proj_nbytes(qd, d, quant) + qd * 2 + 2 * (proj_nbytes(kd, d, quant) + kd * 2) + proj_nbytes(d, qd, quant)
             + 2 * proj_nbytes(I, d, quant) + proj_nbytes(d, I, quant))
    head = V * d * 2 if (cfg["tied"] or quant == FP16) else proj_nbytes(V, d, INT8)
    kv_row = cfg["kv"] * (cfg["hd"] + 4) if kv_int8 else kd * 2
    return cfg["layers"] * layer + d * 2 + head + d * 2 + 2 * cfg["layers"] * kv_row * ctx


def write_model(path, cfg: dict, quant: int, tensors: dict, max_seq_len: int = 32768) -> None:
    """Write a model file from fp32/fp16 numpy tensors named like the HF checkpoint (export_weights.py:283-321)."""
    fmt = lm_head_fmt(quant, cfg["tied"])
    hdr = Header(cfg["vocab"], cfg["dim"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv"], cfg["hd"], max_seq_len, quant, fmt)
    with open(path, "wb") as f:
        f.write(hdr.pack())
        f.write(tensors["model.embed_tokens.weight"].astype(np.float16).tobytes())
        for l in range(cfg["layers"]):
            p = f"model.layers.{l}"
            f.write(tensors[f"{p}.input_layernorm.weight"].astype(np.float16).tobytes())
            for n in ("q", "k", "v"):
                f.write(proj_bytes(tensors[f"{p}.self_attn.{n}_proj.weight"], quant))
                f.write(tensors[f"{p}.self_attn.{n}_proj.bias"].astype(np.float16).tobytes())
            f.write(proj_bytes(tensors[f"{p}.self_attn.o_proj.weight"], quant))
            f.write(tensors[f"{p}.post_attention_layernorm.weight"].astype(np.float16).tobytes())
            for n in ("gate", "up", "down"):
                f.write(proj_bytes(tensors[f"{p}.mlp.{n}_proj.weight"], quant))
        f.write(tensors["model.norm.weight"].astype(np.float16).tobytes())
        if not cfg["tied"]:
            f.write(proj_bytes(tensors["lm_head.weight"], INT8 if fmt == 1 else FP16))


def random_tensors(cfg: dict, seed: int) -> dict:
    """Random-init tensors for a (small) config: N(0, 0.02) everywhere, RMSNorm weights 1 + N(0, 0.02)."""
    rng = np.random.default_rng(seed)
    d, qd, kd, I, V = cfg["dim"], cfg["heads"] * cfg["hd"], cfg["kv"] * cfg["hd"], cfg["inter"], cfg["vocab"]
    n = lambda *s: (0.02 * rng.standard_normal(s)).astype(np.float32)
    t = {"model.embed_tokens.weight": n(V, d), "model.norm.weight": 1 + n(d)}
    for l in range(cfg["layers"]):
        p = f"model.layers.{l}"
        t[f"{p}.input_layernorm.weight"] = 1 + n(d)
        t[f"{p}.post_attention_layernorm.weight"] = 1 + n(d)
        for nm, rows in (("q", qd), ("k", kd), ("v", kd)):
            t[f"{p}.self_attn.{nm}_proj.weight"] = n(rows, d)
            t[f"{p}.self_attn.{nm}_proj.bias"] = n(rows)
        t[f"{p}.self_attn.o_proj.weight"] = n(d, qd)
        t[f"{p}.mlp.gate_proj.weight"] = n(I, d)
        t[f"{p}.mlp.up_proj.weight"] = n(I, d)
        t[f"{p}.mlp.down_proj.weight"] = n(d, I)
    if not cfg["tied"]:
        t["lm_head.weight"] = n(V, d)
    return t
