"""The shared library loads without a GPU, exports every symbol the header declares, and
rejects bad arguments on the host before anything is launched."""
import ctypes as C
import os
import re

import pytest

from open_ommx_serve_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = open(os.path.join(ROOT, "include", "ommx_b200.h")).read()


def test_every_declared_symbol_is_exported():
    declared = set(re.findall(r"\b(ommx_b200_\w+)\s*\(", HEADER))
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    lib = _lib.load()
    for name in declared:
        assert getattr(lib, name) is not None


def test_abi_version_matches_header():
    want = int(re.search(r"#define OMMX_B200_ABI_VERSION (\d+)", HEADER).group(1))
    assert _lib.load().ommx_b200_abi_version() == want


def test_struct_layouts_match_header_field_order():
    for struct, cls in (("ommx_kv_planes", _lib.KVPlanes), ("ommx_pack_args", _lib.PackArgs),
                        ("ommx_decode_args", _lib.DecodeArgs), ("ommx_kv_pool", _lib.KVPool),
                        ("ommx_kv_append_args", _lib.KVAppendArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), HEADER, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names += [n.strip().lstrip("*") for n in re.sub(r"^(const\s+)?\w+\s+", "", decl).split(",")]
        assert names == [f[0] for f in cls._fields_], struct


def test_host_side_rejections():
    lib = _lib.load()
    assert lib.ommx_b200_pack_kv(None, None) == -1
    assert "null" in _lib.last_error()
    a = _lib.PackArgs()
    a.k = a.v = 16
    a.num_tokens = 48
    assert lib.ommx_b200_pack_kv(C.byref(a), None) == -1 and "multiple of 32" in _lib.last_error()
    d = _lib.DecodeArgs()
    assert lib.ommx_b200_decode(C.byref(d), None) == -1
    d.q = d.o = d.lse = d.attn_logits = d.b_seq_len = 256
    d.q_dtype = _lib.OMMX_DT_BF16
    d.planes.head_dim = 64
    assert lib.ommx_b200_decode(C.byref(d), None) == -2 and "head_dim" in _lib.last_error()
    ap = _lib.KVAppendArgs()
    assert lib.ommx_b200_kv_append_decode(C.byref(ap), None) == -1 and "batch" in _lib.last_error()
    ap.batch = 2
    ap.pool.k_hist = ap.pool.v_hist = ap.pool.seq_len = ap.pool.req_to_token = ap.pool.req_to_group = 256
    ap.pool.num_seqs, ap.pool.sink_tokens, ap.pool.recent_window, ap.pool.ring_cap = 2, 8, 32, 60
    assert lib.ommx_b200_kv_append_decode(C.byref(ap), None) == -1 and "ring_cap" in _lib.last_error()
    with pytest.raises(NotImplementedError):
        _lib.check(-2, "x")
    with pytest.raises(ValueError):
        _lib.check(-1, "x")


def test_min_splits_rule():
    lib = _lib.load()
    assert lib.ommx_b200_min_num_kv_splits(0, 16) == 1
    assert lib.ommx_b200_min_num_kv_splits(16384, 16) == 1
    assert lib.ommx_b200_min_num_kv_splits(16384 + 32, 16) == 2
    assert lib.ommx_b200_min_num_kv_splits(131008, 16) == 8


def test_package_fails_loudly_without_cuda_tensors():
    import torch
    from open_ommx_serve_b200 import ommx_pack_kv_canonical_block
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError):
        ommx_pack_kv_canonical_block(torch.zeros(32, 1, 128), torch.zeros(32, 1, 128),
                                     outliers_per_vector=6, outlier_repr="bitmap", use_pow2=True)


def test_auto_split_count_fills_whole_waves():
    """The split count minimises (waves of CTAs over the SMs) x (groups per CTA + fixed cost): with 148 SMs (the
    value used when no device is present) batch 8 takes 18 splits - 144 CTAs, one wave - not ceil(148 / 8) = 19."""
    lib = _lib.load()
    f = lib.ommx_b200_auto_num_kv_splits
    assert f(65472, 1, 8) in (147, 148)
    assert f(131008, 1, 8) in (147, 148)
    assert f(32704, 8, 8) == 18
    assert f(960, 1, 8) == 30                     # one group per CTA, no more splits than groups
    assert f(0, 1, 8) == 1
    for seq, b in ((65472, 2), (8000, 4), (32704, 32), (65472, 148)):
        s = f(seq, b, 8)
        assert 1 <= s <= max(1, (seq + 31) // 32)
        assert s >= lib.ommx_b200_min_num_kv_splits(seq, 16)
