"""The C-ABI library loads without a GPU and exports every symbol include/cuqwen_b200.h declares; the host-only
entry points (model table, tensor-parallel plan, error strings) behave."""
import ctypes as C
import re
from pathlib import Path

import pytest

from cuqwen_b200 import _abi, binfmt

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "cuqwen_b200.h").read_text()


def declared_symbols():
    return sorted(set(re.findall(r"\b(cuqwen_[a-z0-9_]+)\s*\(", HEADER)))


def test_header_and_binding_tables_agree(built):
    assert declared_symbols() == sorted(_abi.SIGNATURES)


def test_every_declared_symbol_is_exported(built):
    raw = C.CDLL(str(_abi.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(raw, name), f"{name} is declared in the header but missing from the library"


def test_every_entry_point_cites_the_interface_it_replaces():
    # each comment block in front of an API function names a reference file (or says there is no counterpart)
    for name in ("cuqwen_create", "cuqwen_load", "cuqwen_step", "cuqwen_k_qkv", "cuqwen_k_attention", "cuqwen_k_mlp1", "cuqwen_k_gemv_add"):
        idx = HEADER.index(name + "(")
        block = HEADER[max(0, idx - 600):idx]
        assert re.search(r"(src/|include/|kernels\.cuh|benchmark/)[\w./]*:\d+", block), name


def test_model_table_matches_reference_config(built):
    for name, mid in (("0.5b", 0), ("1.5b", 1), ("3b", 2), ("7b", 3), ("14b", 4)):
        p = _abi.Params()
        _abi.check(_abi.lib().cuqwen_model_params(mid, 2, C.byref(p)))
        m = binfmt.MODELS[name]
        assert (p.vocab_size, p.dim, p.intermediate_size, p.n_layers, p.n_heads, p.n_kv_heads, p.head_dim) == (
            m["vocab"], m["dim"], m["inter"], m["layers"], m["heads"], m["kv"], m["hd"])
        assert p.max_seq_len == 32768 and p.quant == 2 and abs(p.norm_eps - 1e-6) < 1e-12 and p.rope_theta == 1e6
        assert abs(p.repetition_penalty - 1.1) < 1e-6
    p = _abi.Params()
    assert _abi.lib().cuqwen_model_params(7, 0, C.byref(p)) == 1
    assert b"out of range" in _abi.lib().cuqwen_last_error()


def test_error_strings(built):
    l = _abi.lib()
    assert l.cuqwen_strerror(0) == b"ok"
    seen = {l.cuqwen_strerror(i) for i in range(10)}
    assert len(seen) == 10 and l.cuqwen_strerror(99) == b"unknown error"


def plan(heads, kv, hd, inter, vocab, rank, size):
    out = (C.c_int * 9)()
    rc = _abi.lib().cuqwen_tp_plan(heads, kv, hd, inter, vocab, rank, size, out)
    return rc, list(out)


@pytest.mark.parametrize("model", ["7b", "14b", "1.5b", "3b"])
@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_tp_plan_covers_everything_once(built, model, size):
    m = binfmt.MODELS[model]
    if size > m["kv"] and size % m["kv"]:
        pytest.skip("not divisible")
    grp = m["heads"] // m["kv"]
    q_cover, i_cover, v_cover = [], [], []
    for r in range(size):
        rc, (q0, q1, k0, k1, g, i0, i1, v0, v1) = plan(m["heads"], m["kv"], m["hd"], m["inter"], m["vocab"], r, size)
        if rc:
            pytest.skip(f"plan refuses {model} at {size}: {_abi.lib().cuqwen_last_error()!r}")
        assert q1 > q0 and (q1 - q0) == (k1 - k0) * g                    # uniform heads per KV head on a rank
        assert q0 // grp >= k0 and (q1 - 1) // grp < k1                   # its query heads attend KV heads it stores
        assert (q0 * m["hd"]) % 128 == 0 and (q1 * m["hd"]) % 128 == 0    # o_proj slice holds whole scale groups
        assert i0 % 128 == 0 and i1 % 128 == 0 and v0 % 16 == 0 and v1 % 16 == 0
        q_cover += list(range(q0, q1)); i_cover.append((i0, i1)); v_cover.append((v0, v1))
    assert q_cover == list(range(m["heads"]))
    assert i_cover[0][0] == 0 and i_cover[-1][1] == m["inter"] and all(a[1] == b[0] for a, b in zip(i_cover, i_cover[1:]))
    assert v_cover[0][0] == 0 and v_cover[-1][1] == m["vocab"] and all(a[1] == b[0] for a, b in zip(v_cover, v_cover[1:]))
    sizes = [b - a for a, b in i_cover]
    assert max(sizes) - min(sizes) <= 128                                 # shares differ by at most one group


def test_tp_plan_7b_at_8_ranks_splits_heads_inside_kv_groups(built):
    got = [plan(28, 4, 128, 18944, 152064, r, 8)[1] for r in range(8)]
    assert [(g[0], g[1]) for g in got] == [(0, 3), (3, 7), (7, 10), (10, 14), (14, 17), (17, 21), (21, 24), (24, 28)]
    assert [(g[2], g[3]) for g in got] == [(0, 1), (0, 1), (1, 2), (1, 2), (2, 3), (2, 3), (3, 4), (3, 4)]
    assert sorted({g[6] - g[5] for g in got}) == [2304, 2432]            # 18 or 19 scale groups of the MLP per rank


def test_tp_plan_rejects_impossible_splits(built):
    assert plan(14, 2, 64, 4864, 151936, 0, 3)[0] == 1      # 3 ranks, 2 KV heads
    assert plan(14, 2, 64, 4864, 151936, 1, 2)[0] == 1      # 7 heads x 64 = 448 columns: not whole scale groups
    assert plan(28, 4, 128, 18944, 152064, 9, 8)[0] == 1    # rank out of range


def test_tensor_parallel_layer_bound(built):
    """Exchange sequence numbers are step * 512 + index + 1 with two exchanges per layer: a tensor-parallel engine with
    more layers than that window holds is refused at creation (single-GPU engines have no exchange and no bound)."""
    from cuqwen_b200 import engine as E
    from cuqwen_b200._abi import CuQwenError
    prm = E.custom_params(1024, 256, 512, 300, 4, 2, 64, "int4", max_seq_len=64)
    prm.tp_size, prm.tp_rank = 2, 0
    with pytest.raises(CuQwenError) as err:
        E.Engine(prm)
    assert err.value.code == 1 and "layers" in str(err.value)


def test_int8_kv_cache_needs_an_aligned_max_seq_len(built):
    """The 8-bit cache's row scales are fetched in 16-byte units: a max_seq_len that is not a multiple of 4 is refused
    at creation instead of faulting on the device."""
    from cuqwen_b200 import engine as E
    from cuqwen_b200._abi import CuQwenError
    prm = E.custom_params(1024, 256, 512, 2, 4, 2, 64, "int4", max_seq_len=66)
    prm.flags = E.FLAG_KV_INT8
    with pytest.raises(CuQwenError) as err:
        E.Engine(prm)
    assert err.value.code == 1 and "multiple of 4" in str(err.value)


def test_register_budget_of_the_gemv_kernels():
    """Two CTAs of the one-matrix GEMV kernels share an SM (the o_proj and down launches count on it): that needs at
    most 96 registers per thread.  The two-matrix kernels run one CTA per SM and may use up to 112.  Read from the
    ptxas log the in-tree build leaves behind; skipped when the library was built elsewhere."""
    from pathlib import Path
    log = Path(__file__).resolve().parent.parent / "build" / "obj" / "gemv_i4.ptxas.txt"
    if not log.exists():
        pytest.skip("no ptxas log (library not built in this tree)")
    text = log.read_text()
    found = re.findall(r"Compiling entry function '_ZN2cq11gemv_kernelILi(\d)ELi(\d)EEEvNS_8GemvArgsE'.*?Used (\d+) registers", text, re.S)
    assert found, "ptxas log has no gemv_kernel entries"
    for quant, epi, regs in found:
        limit = 112 if epi in ("3", "4") else 96          # SWIGLU / QKV : the others
        assert int(regs) <= limit, f"gemv_kernel<{quant},{epi}> uses {regs} registers (limit {limit})"
