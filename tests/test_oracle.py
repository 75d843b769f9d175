"""The CPU oracle against the fixtures produced by the reference's own code (bit for bit)."""
import glob
import os

import numpy as np
import pytest

from oracle import ommx_oracle as O
from helpers import GOLDEN, PLANES, load_golden

PACK_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "pack_*.npz"))
                    if "relidx7" not in os.path.basename(p))        # those have tests of their own


def _pack_from_golden(g):
    k, signed, pow2, omap, ps = (int(x) for x in g["cfg"])
    return O.pack_kv(g["K"], g["V"], outliers_per_vector=k, outlier_select="signed" if signed else "abs",
                     use_pow2=bool(pow2), kv_outlier_map=bool(omap), page_size=ps)


def test_fixture_list_complete():
    assert len(PACK_CASES) >= 12, PACK_CASES


@pytest.mark.parametrize("name", PACK_CASES)
def test_pack_bit_exact(name):
    g = load_golden(name)
    mine = _pack_from_golden(g)
    for p in PLANES:
        if p in g:
            assert p in mine, p
            assert mine[p].shape == g[p].shape and mine[p].dtype.itemsize == g[p].dtype.itemsize, p
            assert (mine[p].view(g[p].dtype) == g[p]).all(), f"{name}:{p}"
        else:
            assert p not in mine, p


@pytest.mark.parametrize("name", PACK_CASES)
def test_dequant_bit_exact(name):
    g = load_golden(name)
    Kd, Vd = O.dequant_kv(_pack_from_golden(g))
    assert (Kd == g["K_dq"]).all() and (Vd == g["V_dq"]).all()


def test_bitmap_layout_properties():
    """popcount == k, nibble ordinal == prefix popcount (the reference pins these in its
    bitmap tests: ommx_gpu_serve/tests/test_bitmap_outlier.py:176-246)."""
    g = load_golden("pack_default")
    word = g["k_obmp"].copy().view(np.uint32)[..., 0]
    pop = sum(((word >> np.uint32(b)) & 1) for b in range(32))
    assert (pop == 6).all()
    assert g["k_oval"].shape[-1] == 3


def test_fakequant_bit_exact():
    g = load_golden("fakequant_t200")
    K = np.ascontiguousarray(g["K"].transpose(1, 0, 2))
    V = np.ascontiguousarray(g["V"].transpose(1, 0, 2))
    assert (O.fakequant_group(K, is_key=True) == g["K_fq"]).all()
    assert (O.fakequant_group(V, is_key=False, top=0, bottom=0) == g["V_fq"]).all()
    import torch
    assert (O.fakequant_group_torch(torch.from_numpy(K), is_key=True).numpy() == g["K_fq"]).all()
    assert (O.fakequant_group_torch(torch.from_numpy(V), is_key=False, top=0, bottom=0).numpy() == g["V_fq"]).all()


def _attn_case(name):
    g = load_golden(name)
    seq, H, Hq, D, sink, recent = (int(x) for x in g["cfg"])
    K, V, q = (O.bf16_from_bits(g[n]) for n in ("K", "V", "q"))
    edge = O.packed_boundary(seq, sink, recent)
    planes = O.pack_kv(K[sink:edge], V[sink:edge])
    tail = list(range(sink)) + list(range(edge, seq))
    return g, q, planes, K[tail], V[tail], D


@pytest.mark.parametrize("name", ["attn_seq168", "attn_seq300_gqa8"])
def test_attention_oracle_matches_reference_oracle(name):
    g, q, planes, Kt, Vt, D = _attn_case(name)
    Kd, Vd = O.dequant_kv(planes)
    o, _ = O.attention_fp32(q, np.concatenate([Kd, Kt]), np.concatenate([Vd, Vt]), D ** -0.5)
    np.testing.assert_allclose(o, g["o"], rtol=0, atol=2e-6)


@pytest.mark.parametrize("name", ["attn_seq168", "attn_seq300_gqa8"])
@pytest.mark.parametrize("splits", [1, 3])
def test_split_kv_arithmetic_within_gate(name, splits):
    """The kernel-faithful restatement (bf16 rounding points, split + merge) stays inside the
    path's tolerance of the fp32 oracle: max-abs 2e-2, cosine 0.9999."""
    g, q, planes, Kt, Vt, D = _attn_case(name)
    o, lse, mid = O.decode_split_kv(q, planes, Kt, Vt, D ** -0.5, splits)
    cos, mabs, _ = O.compare(o, g["o"])
    assert cos >= 0.9999 and mabs <= 2e-2, (cos, mabs)
    o2, _, _ = O.decode_split_kv(q, planes, Kt, Vt, D ** -0.5, splits, split_pv=True)
    cos, mabs, _ = O.compare(o2, g["o"])
    assert cos >= 0.9999 and mabs <= 2e-2, (cos, mabs)


def test_split_ranges_rounding():
    # per = ceil(ceil(seq/S)/32)*32 ; trailing splits may be empty
    assert O.split_ranges(4032, 16) == [(i * 256, min((i + 1) * 256, 4032)) for i in range(16)]
    r = O.split_ranges(96, 4)
    assert r == [(0, 32), (32, 64), (64, 96), (96, 96)]


def test_merge_states_matches_full_softmax():
    rng = np.random.default_rng(0)
    K, V = rng.standard_normal((96, 1, 32)).astype(np.float32), rng.standard_normal((96, 1, 32)).astype(np.float32)
    q = rng.standard_normal((2, 32)).astype(np.float32)
    full, lse_full = O.attention_fp32(q, K, V, 0.2)
    parts = [O.attention_fp32(q, K[a:b], V[a:b], 0.2) for a, b in ((0, 40), (40, 41), (41, 96))]
    o, lse = O.merge_states(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]))
    np.testing.assert_allclose(o, full, atol=1e-6)
    np.testing.assert_allclose(lse, lse_full, atol=1e-6)


def test_packed_boundary_values():
    # 1K->960, 4K->4032, 64K->65472 packed tokens with sink 8 / recent 32
    for seq, packed in ((1024, 960), (4096, 4032), (16384, 16320), (65536, 65472), (131072, 131008), (71, 0), (72, 32)):
        assert O.packed_boundary(seq) - 8 == packed or (packed == 0 and O.packed_boundary(seq) <= 8)


@pytest.mark.parametrize("name", ["config1_ctx4096", "prefill_chunk_8192"])
def test_oracle_packer_hashes_to_the_reference_at_benchmark_size(name):
    """Config 1's 4 032 x 8 x 128 block and an 8 192-token chunk: every plane of the oracle's packer hashes
    (SHA-256) to what the reference packer made for the same seeded input (tests/golden/plane_sha256.json)."""
    import hashlib
    import json
    from helpers import GOLDEN, gaussian_kv
    rec = json.load(open(os.path.join(GOLDEN, "plane_sha256.json")))[name]
    T = 4096 if name.startswith("config1") else rec["tokens"] + 8
    K, V = gaussian_kv(rec["seed"], T, 8, 128)
    a, b = rec["first_token"], rec["first_token"] + rec["tokens"]
    pl = O.pack_kv(K[a:b].numpy(), V[a:b].numpy(), outliers_per_vector=6, kv_outlier_map=True, page_size=16)
    for plane, want in rec["sha256"].items():
        assert hashlib.sha256(np.ascontiguousarray(pl[plane]).tobytes()).hexdigest() == want, plane


@pytest.mark.parametrize("k", [6, 10])
def test_oracle_relidx7_planes_match_reference_fixture(k):
    """The reference packer run with outlier_repr='relidx7': same planes as the bitmask encoding except the index
    plane, which is its 7-bit position stream; the oracle's codec reproduces it and inverts it."""
    g = load_golden(f"pack_relidx7_k{k}")
    pl = O.pack_kv(g["K"], g["V"], outliers_per_vector=k, kv_outlier_map=True, page_size=16)
    for name in PLANES:
        if name in g and name != "k_obmp":
            assert (np.asarray(pl[name]).view(g[name].dtype) == g[name]).all(), name
    idx = O.relidx7_from_bitmask(pl["k_obmp"], k)
    assert idx.shape == g["k_oidx"].shape and (idx == g["k_oidx"]).all()
    assert (O.bitmask_from_relidx7(g["k_oidx"], k) == pl["k_obmp"]).all()
    planes = dict(pl, k_obmp=None, k_oidx=g["k_oidx"], outliers_per_vector=k)
    Kd, Vd = O.dequant_kv(O.with_bitmask(planes))
    assert (Kd == g["K_dq"]).all() and (Vd == g["V_dq"]).all()
