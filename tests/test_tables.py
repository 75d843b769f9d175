"""The frozen decision tables against live torch, and the library's host twins against them."""
import json
import os

import numpy as np
import torch

from oracle import gen_tables as G
from oracle import ommx_oracle as O
from open_ommx_serve_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _f32(bits):
    return np.asarray(bits, dtype=np.uint32).view(np.float32)


def test_tables_match_live_torch():
    """Re-derive both tables from torch's CPU log2/log and compare with the committed copy."""
    t = json.load(open(os.path.join(ROOT, "oracle", "tables.json")))
    assert G.derive_pow2_cuts(window=512, full_sweep=(127,)) == t["pow2_cut_mantissa"]
    assert G.derive_fp4_thresholds(window=4096) == t["fp4_first_upper_bits"]


def test_inc_file_matches_json():
    t = json.load(open(os.path.join(ROOT, "oracle", "tables.json")))
    inc = open(os.path.join(ROOT, "open_ommx_serve_b200", "csrc", "ommx_tables.inc")).read()
    for c in set(t["pow2_cut_mantissa"]):
        assert f"{c}u" in inc
    for th in t["fp4_first_upper_bits"]:
        assert f"0x{th:08x}u" in inc


def test_pow2_exponent_vs_torch_random():
    rng = np.random.default_rng(1)
    x = np.exp(rng.uniform(np.log(1e-12), np.log(1e30), 200000)).astype(np.float32)
    want = torch.round(torch.log2(torch.from_numpy(x))).numpy().astype(np.int32)
    assert (O.pow2_exponent(x) == want).all()


def test_host_twins_match_oracle():
    lib = _lib.load()
    t = json.load(open(os.path.join(ROOT, "oracle", "tables.json")))
    # around every cut of a spread of exponents, and around every FP4 threshold, both signs
    for E in (87, 99, 100, 120, 126, 127, 128, 129, 140, 200):
        cut = t["pow2_cut_mantissa"][E]
        bits = (np.uint32(E) << np.uint32(23)) | np.arange(cut - 40, cut + 40, dtype=np.uint32)
        x = _f32(bits)
        got = np.array([lib.ommx_b200_host_pow2_exponent(float(v)) for v in x])
        assert (got == O.pow2_exponent(x)).all(), E
    for th in t["fp4_first_upper_bits"]:
        bits = np.arange(th - 20, th + 20, dtype=np.uint32)
        for sign in (0, 0x80000000):
            m = _f32(bits | np.uint32(sign))
            got = np.array([lib.ommx_b200_host_fp4_encode(float(v)) for v in m])
            assert (got == O.fp4_encode(m)).all(), hex(th)
    # known answers: the FP4 levels are fixed points, -0.0 -> 0, tiny negative -> sign with magnitude 0
    for code, lvl in enumerate((0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)):
        assert lib.ommx_b200_host_fp4_encode(lvl) == code
        if lvl:
            assert lib.ommx_b200_host_fp4_encode(-lvl) == code | 8
    assert lib.ommx_b200_host_fp4_encode(-0.0) == 0
    assert lib.ommx_b200_host_fp4_encode(-1e-6) == 8
    assert lib.ommx_b200_host_fp4_encode(100.0) == 7


def test_fp4_encode_vs_reference_rule_random():
    rng = np.random.default_rng(2)
    m = (rng.standard_normal(200000) * 3).astype(np.float32)
    want = G.fp4_index(torch.from_numpy(m)).numpy()
    got = O.fp4_encode(m)
    assert ((got & 7) == (((want >= 2).astype(int) + (want >= 4) + (want >= 6)) * 2 + (want & 1))).all()
    assert ((got >> 3) == (m < 0)).all()
