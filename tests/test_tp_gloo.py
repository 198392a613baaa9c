"""World-size-2 check of the tensor-parallel partition on CPU: each gloo rank computes its share of one decoder layer
and of the lm_head from the slices `cuqwen_b200.tp` hands it, partial sums meet in an all-reduce and sampler keys in
an all-gather, and the result must equal the unsharded computation."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest

from cuqwen_b200 import binfmt, tp

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

CFGS = {
    "kv_heads_split": dict(dim=256, inter=512, vocab=320, layers=1, heads=4, kv=2, hd=64, tied=False),
    "kv_head_shared": dict(dim=256, inter=768, vocab=336, layers=1, heads=4, kv=1, hd=128, tied=False),
}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rms(x, w):
    return x / np.sqrt(np.mean(x * x) + 1e-6) * w


def _attend(q, Kc, Vc, heads, kv_of_head, hd):
    out = np.zeros((heads, hd))
    for h in range(heads):
        s = Kc[kv_of_head[h]] @ q[h] / np.sqrt(hd)
        p = np.exp(s - s.max()); p /= p.sum()
        out[h] = p @ Vc[kv_of_head[h]]
    return out


def _layer(t, cfg, x, Kc, Vc, q_heads, kv_heads, mlp_cols, reduce):
    """One decoder layer on the given slices; `reduce` sums row-parallel partials across ranks.  K/V of the new token
    are appended to the (shared, seeded) cache rows of the KV heads this rank stores."""
    hd, grp, pfx = cfg["hd"], cfg["heads"] // cfg["kv"], "model.layers.0"
    xn = _rms(x, t[f"{pfx}.input_layernorm.weight"])
    q = (t[f"{pfx}.self_attn.q_proj.weight"] @ xn + t[f"{pfx}.self_attn.q_proj.bias"]).reshape(len(q_heads), hd)
    k = (t[f"{pfx}.self_attn.k_proj.weight"] @ xn + t[f"{pfx}.self_attn.k_proj.bias"]).reshape(len(kv_heads), hd)
    v = (t[f"{pfx}.self_attn.v_proj.weight"] @ xn + t[f"{pfx}.self_attn.v_proj.bias"]).reshape(len(kv_heads), hd)
    Kl = [np.vstack([Kc[g], k[i]]) for i, g in enumerate(kv_heads)]
    Vl = [np.vstack([Vc[g], v[i]]) for i, g in enumerate(kv_heads)]
    local_kv = [list(kv_heads).index(h // grp) for h in q_heads]
    att = _attend(q, Kl, Vl, len(q_heads), local_kv, hd).reshape(-1)
    x = x + reduce(t[f"{pfx}.self_attn.o_proj.weight"] @ att)
    xn = _rms(x, t[f"{pfx}.post_attention_layernorm.weight"])
    g, u = t[f"{pfx}.mlp.gate_proj.weight"] @ xn, t[f"{pfx}.mlp.up_proj.weight"] @ xn
    x = x + reduce(t[f"{pfx}.mlp.down_proj.weight"] @ (g / (1 + np.exp(-g)) * u))
    return x


def _inputs(cfg):
    rng = np.random.default_rng(7)
    t = {k: v.astype(np.float64) * (8 if v.ndim == 2 else 1) for k, v in binfmt.random_tensors(cfg, seed=3).items()}
    x = rng.standard_normal(cfg["dim"])
    Kc = rng.standard_normal((cfg["kv"], 9, cfg["hd"]))
    Vc = rng.standard_normal((cfg["kv"], 9, cfg["hd"]))
    return t, x, Kc, Vc


def _worker(rank, world, port, name, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = CFGS[name]
        t, x, Kc, Vc = _inputs(cfg)
        p = tp.plan(cfg, rank, world)
        mine = tp.shard_tensors(t, cfg, p)

        def allreduce(a):
            b = torch.from_numpy(np.ascontiguousarray(a))
            dist.all_reduce(b)
            return b.numpy()

        y = _layer(mine, cfg, x, Kc, Vc, range(p.q0, p.q1), range(p.kv0, p.kv1), (p.i0, p.i1), allreduce)
        logits = mine["lm_head.weight"] @ _rms(y, t["model.norm.weight"])
        best = int(np.argmax(logits))
        key = torch.tensor([tp.pack_argmax_key(float(np.float32(logits[best])), p.v0 + best) - (1 << 63)], dtype=torch.int64)
        keys = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(keys, key)
        token = tp.unpack_argmax_index(max(int(k.item()) for k in keys) + (1 << 63))
        if rank == 0:
            full = _layer(t, cfg, x, Kc, Vc, range(cfg["heads"]), range(cfg["kv"]), (0, cfg["inter"]), lambda a: a)
            want = int(np.argmax((t["lm_head.weight"] @ _rms(full, t["model.norm.weight"])).astype(np.float32)))
            ret["err"] = float(np.abs(full - y).max())
            ret["token"], ret["want"] = token, want
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", sorted(CFGS))
def test_two_rank_partition_reproduces_the_unsharded_layer(built, name):
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), name, ret), nprocs=2, join=True)
    assert ret["err"] < 1e-9, ret["err"]
    assert ret["token"] == ret["want"]


def test_argmax_key_orders_like_the_sampler():
    vals = [-3.5, -0.0, 0.0, 1e-8, 2.0, 65504.0]
    keys = [tp.pack_argmax_key(v, 5) for v in vals]
    assert keys == sorted(keys) and len({k >> 32 for k in keys[2:]}) == 4
    assert tp.pack_argmax_key(1.0, 3) > tp.pack_argmax_key(1.0, 4)           # ties go to the smaller index
    assert tp.unpack_argmax_index(tp.pack_argmax_key(1.0, 151935)) == 151935


@pytest.mark.parametrize("size", [2, 4, 8])
def test_shards_of_all_ranks_tile_the_model(built, size):
    """More ranks than KV heads: ranks that share a KV head split its query heads and each keeps that head's K and V.
    Whatever the split, the column slices of o_proj and down tile their matrices exactly once, the row slices of
    q / gate / up / lm_head do too, and every query head sits on a rank that also holds its KV head."""
    cfg = dict(dim=512, inter=2048, vocab=640, layers=1, heads=8, kv=2, hd=128, tied=False)
    t = {k: v for k, v in binfmt.random_tensors(cfg, seed=11).items()}
    pfx, hd, grp = "model.layers.0", cfg["hd"], cfg["heads"] // cfg["kv"]
    plans = [tp.plan(cfg, r, size) for r in range(size)]
    shards = [tp.shard_tensors(t, cfg, p) for p in plans]
    cat = lambda name, axis: np.concatenate([s[name] for s in shards], axis=axis)
    for name, axis in ((f"{pfx}.self_attn.q_proj.weight", 0), (f"{pfx}.self_attn.q_proj.bias", 0), (f"{pfx}.self_attn.o_proj.weight", 1),
                       (f"{pfx}.mlp.gate_proj.weight", 0), (f"{pfx}.mlp.up_proj.weight", 0), (f"{pfx}.mlp.down_proj.weight", 1), ("lm_head.weight", 0)):
        assert np.array_equal(cat(name, axis), t[name]), name
    for p, s in zip(plans, shards):
        assert p.q0 // grp >= p.kv0 and (p.q1 - 1) // grp < p.kv1                      # its query heads find their KV head locally
        assert np.array_equal(s[f"{pfx}.self_attn.k_proj.weight"], t[f"{pfx}.self_attn.k_proj.weight"][p.kv0 * hd:p.kv1 * hd])
        assert np.array_equal(s["model.norm.weight"], t["model.norm.weight"])          # replicated
    kv_copies = sum(p.kv1 - p.kv0 for p in plans)
    assert kv_copies == max(cfg["kv"], size)                                           # KV heads are replicated only when ranks outnumber them
