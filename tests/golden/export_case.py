"""Synthetic Hugging Face-style checkpoint directories for the exporter tests.  Every byte is a pure function of the
case name (integer hashing only, no library random generator), so the directory built on one machine is identical
to the one the golden hashes in export_golden.json were made from."""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

CASES = {
    # name: (config, tied, shards, dtype of tensor number i)
    "tied_bf16": dict(vocab=320, dim=256, inter=384, layers=2, heads=4, kv=2, tied=True, shards=1, dtypes=("BF16",)),
    "untied_mixed": dict(vocab=300, dim=128, inter=256, layers=3, heads=2, kv=1, tied=False, shards=2, dtypes=("F16", "BF16", "F32")),
}


def _hash64(idx: np.ndarray, seed: int) -> np.ndarray:
    z = idx.astype(np.uint64) + np.uint64((seed * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def values(shape, seed: int, scale: float, offset: float = 0.0) -> np.ndarray:
    n = int(np.prod(shape))
    u = (_hash64(np.arange(n, dtype=np.uint64), seed) >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)
    return ((u - np.float32(0.5)) * np.float32(2 * scale) + np.float32(offset)).reshape(shape)


def tensor_table(c: dict):
    """[(name, fp32 array)] in checkpoint order."""
    d, hd = c["dim"], c["dim"] // c["heads"]
    qd, kd, I = c["heads"] * hd, c["kv"] * hd, c["inter"]
    out, seed = [], [1]

    def add(name, shape, scale=0.05, offset=0.0):
        seed[0] += 1
        out.append((name, values(shape, seed[0], scale, offset)))

    add("model.embed_tokens.weight", (c["vocab"], d))
    for l in range(c["layers"]):
        p = f"model.layers.{l}"
        add(f"{p}.input_layernorm.weight", (d,), 0.1, 1.0)
        add(f"{p}.self_attn.q_proj.weight", (qd, d))
        add(f"{p}.self_attn.q_proj.bias", (qd,), 0.5)
        add(f"{p}.self_attn.k_proj.weight", (kd, d))
        add(f"{p}.self_attn.k_proj.bias", (kd,), 0.5)
        add(f"{p}.self_attn.v_proj.weight", (kd, d))
        add(f"{p}.self_attn.v_proj.bias", (kd,), 0.5)
        add(f"{p}.self_attn.o_proj.weight", (d, qd))
        add(f"{p}.post_attention_layernorm.weight", (d,), 0.1, 1.0)
        add(f"{p}.mlp.gate_proj.weight", (I, d))
        add(f"{p}.mlp.up_proj.weight", (I, d), 3.0)
        add(f"{p}.mlp.down_proj.weight", (d, I), 0.002)
    add("model.norm.weight", (d,), 0.1, 1.0)
    if not c["tied"]:
        add("lm_head.weight", (c["vocab"], d))
    # an all-zero scale group, and a group whose values all round to the clipping bound
    out[2][1][0, :128] = 0.0
    out[2][1][1, :128] = 0.04
    return out


def _encode(arr: np.ndarray, dtype: str) -> bytes:
    a = np.ascontiguousarray(arr, dtype=np.float32)
    if dtype == "F32":
        return a.tobytes()
    if dtype == "F16":
        return a.astype(np.float16).tobytes()
    return (a.view(np.uint32) >> 16).astype(np.uint16).tobytes()      # BF16 by truncation


def _write_safetensors(path: Path, items) -> None:
    header, blobs, off = {"__metadata__": {"format": "pt"}}, [], 0
    for name, arr, dtype in items:
        raw = _encode(arr, dtype)
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def byte_symbols():
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    out, n = {}, 0
    for b in range(256):
        if b in keep:
            out[b] = chr(b)
        else:
            out[b] = chr(256 + n)
            n += 1
    return out


def write_case(name: str, root: Path) -> Path:
    c = CASES[name]
    d = Path(root) / name
    d.mkdir(parents=True, exist_ok=True)
    cfg = {"vocab_size": c["vocab"], "hidden_size": c["dim"], "intermediate_size": c["inter"], "num_hidden_layers": c["layers"],
           "num_attention_heads": c["heads"], "num_key_value_heads": c["kv"], "max_position_embeddings": 32768,
           "tie_word_embeddings": c["tied"], "rms_norm_eps": 1e-6, "rope_theta": 1000000.0}
    (d / "config.json").write_text(json.dumps(cfg, indent=2))
    table = tensor_table(c)
    items = [(n, a, c["dtypes"][i % len(c["dtypes"])]) for i, (n, a) in enumerate(table)]
    per = (len(items) + c["shards"] - 1) // c["shards"]
    for s in range(c["shards"]):
        fname = "model.safetensors" if c["shards"] == 1 else f"model-{s + 1:05d}-of-{c['shards']:05d}.safetensors"
        _write_safetensors(d / fname, items[s * per:(s + 1) * per])
    # tokenizer resources: byte symbols, a few merges (some non-ASCII, one with characters JSON must escape)
    sym = byte_symbols()
    vocab = {sym[b]: i for i, b in enumerate(sorted(sym))}
    for extra in ("he", "ll", "hell", "hello", sym[32] + "w", "é".encode().decode("latin-1"), "q\"\\", sym[10] + sym[10]):
        vocab.setdefault(extra, len(vocab))
    vocab["<|endoftext|>"] = len(vocab)
    (d / "vocab.json").write_text(json.dumps(vocab, ensure_ascii=False), encoding="utf-8")
    n = len(vocab)
    tok = {"version": "1.0", "added_tokens": [{"id": n - 1, "content": "<|endoftext|>", "special": True},
                                              {"id": n, "content": "<|im_start|>", "special": True},
                                              {"id": n + 1, "content": "<|im_end|>", "special": True}]}
    (d / "tokenizer.json").write_text(json.dumps(tok, ensure_ascii=False), encoding="utf-8")
    tc = {"eos_token": "<|endoftext|>", "pad_token": "<|endoftext|>", "bos_token": None, "model_max_length": 131072,
          "additional_special_tokens": ["<|im_start|>", "<|endoftext|>", "hello"], "unk_token": "not-in-vocab"}
    (d / "tokenizer_config.json").write_text(json.dumps(tc, ensure_ascii=False), encoding="utf-8")
    return d
