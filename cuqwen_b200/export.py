"""Streaming exporter: a Hugging Face Qwen2.5 checkpoint directory (config.json + *.safetensors, optionally
vocab.json / tokenizer.json / tokenizer_config.json) -> CuQwen's ``.bin`` model file and tokenizer ranks JSON.

The output is byte-for-byte what the reference's ``export_weights.py`` writes (``export_weights`` :209-325,
``export_tokenizer`` :328-363) - same header, tensor order, quantiser and lm_head rule - but the checkpoint is never
held in memory: shards are memory-mapped, only their JSON headers are parsed up front, and every tensor is converted
and written in blocks of rows (the reference reads every shard completely, :60-65).  Peak memory is a few hundred MB
for any model size.  Nothing is downloaded: the directory must already be on disk.

    python -m cuqwen_b200.export --model-dir /path/to/Qwen2.5-7B-Instruct --model 7b --quantization int4
"""
from __future__ import annotations

import argparse
import json
import mmap
import os
import struct
from pathlib import Path

import numpy as np

from . import binfmt

ROW_BLOCK_BYTES = 64 << 20      # source bytes converted per step


class SafetensorsDir:
    """Index of every tensor of a directory of ``.safetensors`` shards (reference: MultiShardSafetensors,
    export_weights.py:68-114).  A later shard (in sorted file-name order) wins when a name repeats."""

    def __init__(self, model_dir):
        self.model_dir = Path(model_dir)
        files = sorted(f for f in os.listdir(self.model_dir) if f.endswith(".safetensors"))
        if not files:
            raise FileNotFoundError(f"No .safetensors files found in {self.model_dir}")
        self._maps: list[mmap.mmap] = []
        self._files = []
        self.entries: dict[str, tuple[int, str, list[int], int, int]] = {}
        for idx, name in enumerate(files):
            f = open(self.model_dir / name, "rb")
            self._files.append(f)
            (hlen,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(hlen))
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps.append(mm)
            base = 8 + hlen
            for key, meta in header.items():
                if key == "__metadata__":
                    continue
                a, b = meta["data_offsets"]
                self.entries[key] = (idx, meta["dtype"], list(meta["shape"]), base + a, base + b)

    def close(self) -> None:
        for mm in self._maps:
            mm.close()
        for f in self._files:
            f.close()
        self._maps, self._files = [], []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def contains(self, substring: str) -> bool:
        return any(substring in k for k in self.entries)

    def shape(self, key: str) -> list[int]:
        return self._entry(key)[2]

    def _entry(self, key: str):
        if key not in self.entries:
            raise KeyError(f"Tensor '{key}' not found across safetensor shards.")
        return self.entries[key]

    def rows(self, key: str, r0: int = 0, r1: int | None = None) -> np.ndarray:
        """Rows [r0, r1) of a tensor as fp16, converted like the reference (:96-106): BF16 widens to fp32 and
        rounds to fp16, F32 rounds to fp16, F16 is taken as is.  A 1-D tensor is one 'row' per element."""
        idx, dtype, shape, a, b = self._entry(key)
        n_rows = shape[0] if shape else 1
        inner = int(np.prod(shape[1:], dtype=np.int64)) if len(shape) > 1 else 1
        r1 = n_rows if r1 is None else r1
        size = {"BF16": 2, "F16": 2, "F32": 4}.get(dtype)
        if size is None:
            raise ValueError(f"Unsupported safetensors dtype '{dtype}' for key '{key}'")
        lo, hi = a + r0 * inner * size, a + r1 * inner * size
        if hi > b:
            raise ValueError(f"tensor '{key}': rows {r0}:{r1} reach past its data")
        raw = np.frombuffer(self._maps[idx], dtype=np.uint8, count=hi - lo, offset=lo)
        with np.errstate(over="ignore"):
            if dtype == "BF16":
                arr = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float16)
            elif dtype == "F16":
                arr = raw.view(np.float16).copy()
            else:
                arr = raw.view(np.float32).astype(np.float16)
        return arr.reshape([r1 - r0] + shape[1:])


def _row_block(shape, itemsize: int = 4) -> int:
    inner = int(np.prod(shape[1:], dtype=np.int64)) if len(shape) > 1 else 1
    return max(1, ROW_BLOCK_BYTES // max(1, inner * itemsize))


def write_fp16(f, st: SafetensorsDir, key: str) -> int:
    shape = st.shape(key)
    n_rows = shape[0] if shape else 1
    step, total = _row_block(shape), 0
    for r in range(0, n_rows, step):
        data = st.rows(key, r, min(n_rows, r + step)).tobytes()
        f.write(data)
        total += len(data)
    return total


def write_proj(f, st: SafetensorsDir, key: str, quant: int) -> int:
    """One projection matrix: fp16 as is; int8 / int4 as all weight rows, then all fp16 group scales
    (export_weights.py:150-206).  Rows are independent, so converting them block by block changes nothing."""
    if quant == binfmt.FP16:
        return write_fp16(f, st, key)
    shape = st.shape(key)
    if len(shape) != 2:
        raise ValueError(f"quantised export expects a 2D weight matrix, got shape {shape} for '{key}'")
    qmax = 127 if quant == binfmt.INT8 else 7
    step, total, scales = _row_block(shape), 0, []
    for r in range(0, shape[0], step):
        q, s = binfmt.quantize_groupwise(st.rows(key, r, min(shape[0], r + step)), qmax)
        data = (q if quant == binfmt.INT8 else binfmt.pack_int4(q)).tobytes()
        f.write(data)
        total += len(data)
        scales.append(s)
    data = np.concatenate(scales, axis=0).astype(np.float16).tobytes()
    f.write(data)
    return total + len(data)


def default_bin_name(model_size: str, quant: str) -> str:
    """weights/model_<quant>_<size with '.' as '_'>.bin, the path CuQwen's config table expects (export_weights.py:213)."""
    return os.path.join("weights", f"model_{quant}_{model_size.replace('.', '_')}.bin")


def export_weights(model_dir, out_bin_path, quant: str, log=lambda msg: None) -> int:
    """Writes the model file; returns its size in bytes."""
    q = binfmt.QUANT_ID[quant]
    with open(Path(model_dir) / "config.json") as f:
        cfg = json.load(f)
    dim, heads = cfg["hidden_size"], cfg["num_attention_heads"]
    tied = int(cfg.get("tie_word_embeddings", True))
    with SafetensorsDir(model_dir) as st:
        separate_head = st.contains("lm_head") and not tied
        head_int8 = q != binfmt.FP16 and separate_head
        hdr = binfmt.Header(cfg["vocab_size"], dim, cfg["intermediate_size"], cfg["num_hidden_layers"], heads,
                            cfg["num_key_value_heads"], cfg.get("head_dim", dim // heads),
                            cfg.get("max_position_embeddings", 32768), q, 1 if head_int8 else 0)
        out_dir = os.path.dirname(os.fspath(out_bin_path))
        if out_dir:
            os.makedirs(out_dir, exist_ok=True)
        total = 0
        with open(out_bin_path, "wb") as f:
            f.write(hdr.pack())
            total += 256
            total += write_fp16(f, st, "model.embed_tokens.weight")
            for l in range(hdr.layers):
                p = f"model.layers.{l}"
                log(f"layer {l}/{hdr.layers - 1}")
                total += write_fp16(f, st, f"{p}.input_layernorm.weight")
                for n in ("q", "k", "v"):
                    total += write_proj(f, st, f"{p}.self_attn.{n}_proj.weight", q)
                    total += write_fp16(f, st, f"{p}.self_attn.{n}_proj.bias")
                total += write_proj(f, st, f"{p}.self_attn.o_proj.weight", q)
                total += write_fp16(f, st, f"{p}.post_attention_layernorm.weight")
                for n in ("gate", "up", "down"):
                    total += write_proj(f, st, f"{p}.mlp.{n}_proj.weight", q)
            total += write_fp16(f, st, "model.norm.weight")
            if head_int8:
                total += write_proj(f, st, "lm_head.weight", binfmt.INT8)
            elif separate_head:
                total += write_fp16(f, st, "lm_head.weight")
    return total


def export_tokenizer(model_dir, out_json_path) -> None:
    """Writes the ranks file the tokenizer reads: {"vocab", "special_tokens", "added_tokens"} with the reference's
    key order and JSON formatting (export_weights.py:328-363)."""
    model_dir = Path(model_dir)
    with open(model_dir / "vocab.json", "r", encoding="utf-8") as f:
        vocab = json.load(f)
    added = {}
    if (model_dir / "tokenizer.json").exists():
        with open(model_dir / "tokenizer.json", "r", encoding="utf-8") as f:
            for entry in json.load(f).get("added_tokens", []):
                added[int(entry["id"])] = entry["content"]
    special = {}
    if (model_dir / "tokenizer_config.json").exists():
        with open(model_dir / "tokenizer_config.json", "r", encoding="utf-8") as f:
            tc = json.load(f)
        for k, v in tc.items():
            if isinstance(v, str) and v in vocab:
                special[k] = v
            elif isinstance(v, list):
                for item in v:
                    if isinstance(item, str) and item in vocab:
                        special[item] = item
    out_dir = os.path.dirname(os.fspath(out_json_path))
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
    with open(out_json_path, "w", encoding="utf-8") as f:
        json.dump({"vocab": vocab, "special_tokens": special, "added_tokens": added}, f, ensure_ascii=False, indent=2)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Export a local Qwen2.5 checkpoint directory to CuQwen's .bin format and tokenizer JSON.")
    ap.add_argument("--model-dir", required=True, help="directory with config.json and *.safetensors (no download is attempted)")
    ap.add_argument("--quantization", required=True, choices=["fp16", "int8", "int4"])
    ap.add_argument("--model", choices=sorted(binfmt.MODELS), help="size tag used for the default output name")
    ap.add_argument("--out", help="output .bin (default: weights/model_<quant>_<model>.bin)")
    ap.add_argument("--tokenizer-out", default=os.path.join("weights", "qwen25_bpe_ranks.json"))
    ap.add_argument("--no-tokenizer", action="store_true")
    a = ap.parse_args(argv)
    if not a.out and not a.model:
        ap.error("give --out or --model")
    out = a.out or default_bin_name(a.model, a.quantization)
    n = export_weights(a.model_dir, out, a.quantization, log=lambda m: print("  " + m, end="\r", flush=True))
    print(f"\nwrote {out} ({n / 2**20:.2f} MB)")
    if not a.no_tokenizer and (Path(a.model_dir) / "vocab.json").exists():
        export_tokenizer(a.model_dir, a.tokenizer_out)
        print(f"wrote {a.tokenizer_out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
