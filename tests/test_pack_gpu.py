"""CUDA store kernel vs the reference-made fixtures and the CPU oracle: bit-exact planes."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import ommx_oracle as O
from helpers import GOLDEN, PLANES, assert_planes_equal, gaussian_kv, load_golden, plane_to_numpy

pytestmark = pytest.mark.gpu
PACK_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "pack_*.npz"))
                    if "relidx7" not in os.path.basename(p))        # those have tests of their own


def _gpu_pack(K, V, k=6, select="signed", pow2=True, omap=True, ps=16, scale_dtype=torch.bfloat16, **kw):
    from open_ommx_serve_b200 import ommx_pack_kv_canonical_block
    return ommx_pack_kv_canonical_block(
        K, V, outliers_per_vector=k, outlier_repr="bitmap", outlier_select=select, use_pow2=pow2,
        kv_outlier_map=omap, page_size=ps, scale_dtype=scale_dtype, device="cuda", **kw)


@pytest.mark.parametrize("name", PACK_CASES)
def test_pack_matches_reference_fixture(name):
    g = load_golden(name)
    k, signed, pow2, omap, ps = (int(x) for x in g["cfg"])
    out = _gpu_pack(torch.from_numpy(g["K"]), torch.from_numpy(g["V"]), k=k,
                    select="signed" if signed else "abs", pow2=bool(pow2), omap=bool(omap), ps=ps)
    assert_planes_equal(out, {p: g[p] for p in PLANES if p in g}, ctx=name + ":")
    assert out["kv_int8_scale"] == bool(pow2) and out["outlier_repr"] == "bitmap"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H", [(4032, 8), (256, 2), (32, 1)])
def test_pack_matches_oracle_seeded(T, H, dtype):
    K, V = gaussian_kv(42 + T, T, H, 128)
    want = O.pack_kv(K.numpy(), V.numpy())
    out = _gpu_pack(K.to(dtype), V.to(dtype))
    assert_planes_equal(out, want, ctx=f"T={T},H={H}:")


@pytest.mark.parametrize("k", [0, 1, 2, 3, 4, 5, 6, 7, 8, 12])
@pytest.mark.parametrize("mag", [4.0, 30.0])
def test_pack_outlier_count_and_magnitude_sweep(k, mag):
    K, V = gaussian_kv(5 + k, 128, 4, 128, mag=mag)
    want = O.pack_kv(K.numpy(), V.numpy(), outliers_per_vector=k)
    assert_planes_equal(_gpu_pack(K, V, k=k), want, ctx=f"k={k}:")


def test_pack_fp32_scale_planes_and_head_dim_64():
    K, V = gaussian_kv(77, 64, 2, 64, bf16=False)
    want = O.pack_kv(K.numpy(), V.numpy(), use_pow2=False, scale_bf16=False, kv_int8_scale=False)
    out = _gpu_pack(K, V, pow2=False, scale_dtype=torch.float32)
    assert_planes_equal(out, want)


def test_pack_full_size_64k_properties():
    """At the 64K benchmark size: popcount of every bitmask frame is k, code planes agree with
    the oracle on a sampled slice, and quantize->dequantize error is bounded by half a step."""
    T, H, D = 65472, 8, 128
    K, V = gaussian_kv(42, T, H, D)
    out = _gpu_pack(K.bfloat16(), V.bfloat16())
    word = plane_to_numpy(out["k_obmp"]).view(np.uint32)[..., 0]
    pop = np.zeros(word.shape, dtype=np.uint8)
    for b in range(32):
        pop += ((word >> np.uint32(b)) & 1).astype(np.uint8)
    assert (pop == 6).all()
    sl = slice(32 * 1000, 32 * 1004)
    want = O.pack_kv(K[sl].numpy(), V[sl].numpy())
    got = {p: plane_to_numpy(out[p]) for p in PLANES}
    for p in PLANES:
        lead = slice(1000 * 2, 1004 * 2) if p in ("k_base", "v_main", "v_scale", "v_zp") else slice(1000, 1004)
        assert (got[p][lead].view(want[p].dtype) == want[p]).all(), p
    planes = dict(got, head_dim=D, n_kv_heads=H, num_tokens=T, n_groups=T // 32, page_size=16,
                  outliers_per_vector=6, kv_outlier_map=True)
    sub = {p: (got[p][:64] if p in ("k_base", "v_main", "v_scale", "v_zp") else got[p][:32]) for p in PLANES}
    sub.update(head_dim=D, n_kv_heads=H, num_tokens=1024, n_groups=32, page_size=16,
               outliers_per_vector=6, kv_outlier_map=True)
    Kd, Vd = O.dequant_kv(sub)
    vstep = np.ldexp(1.0, sub["v_scale"].astype(np.int32)).reshape(1024, H, 4, 1)
    v = V[:1024].numpy().reshape(1024, H, 4, 32)
    rng = v.max(-1, keepdims=True) - v.min(-1, keepdims=True)
    bound = np.maximum(0.5 * vstep, rng - 3 * vstep) + np.abs(v).max(-1, keepdims=True) * 2.0 ** -8
    assert (np.abs(Vd.reshape(v.shape) - v) <= bound).all()


def test_pack_into_pool_slots_scattered():
    """Direct-to-slot store: same bytes as a contiguous pack, landed at permuted pages/slots,
    other slots untouched (slot isolation, reference: tests/test_kv_pool_parity.py)."""
    from open_ommx_serve_b200.attention.pack import alloc_planes, ommx_pack_kv_into
    K, V = gaussian_kv(9, 96, 8, 128)
    want = O.pack_kv(K.numpy(), V.numpy())
    pool = alloc_planes(20, 10, 8, 128, device="cuda")
    for t in pool.values():
        if t is not None:
            t.fill_(0x55 if t.dtype == torch.uint8 else 1)
    before = {n: t.clone() for n, t in pool.items() if t is not None}
    pages = torch.tensor([7, 3, 19, 0, 12, 5], dtype=torch.int32, device="cuda")
    slots = torch.tensor([9, 2, 4], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ommx_pack_kv_into(K.cuda(), V.cuda(), pool, dst_pages=pages, dst_groups=slots,
                      outliers_per_vector=6, status=status)
    assert int(status.item()) == 0
    for n in PLANES:
        got = plane_to_numpy(pool[n])
        idx = pages.cpu().numpy() if n in ("k_base", "v_main", "v_scale", "v_zp") else slots.cpu().numpy()
        assert (got[idx].view(want[n].dtype) == want[n]).all(), n
        mask = np.ones(got.shape[0], dtype=bool)
        mask[idx] = False
        assert (got[mask] == plane_to_numpy(before[n])[mask]).all(), n + " (untouched slots changed)"


def test_pack_status_word_instead_of_trap():
    from open_ommx_serve_b200.attention.pack import alloc_planes, ommx_pack_kv_into
    from open_ommx_serve_b200 import _lib
    K, V = gaussian_kv(3, 32, 2, 128)
    pool = alloc_planes(2, 1, 2, 128, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bad_pages = torch.tensor([0, 99], dtype=torch.int32, device="cuda")
    bad_slot = torch.tensor([-4], dtype=torch.int32, device="cuda")
    ommx_pack_kv_into(K.cuda(), V.cuda(), pool, dst_pages=bad_pages, dst_groups=bad_slot,
                      outliers_per_vector=6, status=status)
    bits = int(status.item())
    assert bits & _lib.ST_BAD_PAGE and bits & _lib.ST_BAD_GROUP
    Kn = K.clone()
    Kn[5, 1, 17] = float("nan")
    with pytest.raises(ValueError):
        _gpu_pack(Kn, V)
    Vn = V.clone()
    Vn[0, 0, 0] = float("inf")
    with pytest.raises(ValueError):
        _gpu_pack(K, Vn)


def test_pack_refusals():
    K, V = gaussian_kv(3, 32, 2, 128)
    from open_ommx_serve_b200 import ommx_pack_kv_canonical_block as pack
    with pytest.raises(ValueError):
        pack(K[:31], V[:31], outliers_per_vector=6, outlier_repr="bitmap", use_pow2=True, device="cuda")
    with pytest.raises(ValueError):
        pack(K, V, outliers_per_vector=6, outlier_repr="nope", device="cuda")
    with pytest.raises(NotImplementedError):
        pack(K, V, outliers_per_vector=6, outlier_repr="combinadic", device="cuda")
    with pytest.raises(NotImplementedError):
        pack(K, V, outliers_per_vector=18, outlier_repr="relidx7", device="cuda")
    with pytest.raises(NotImplementedError):
        pack(torch.cat([K, K]), torch.cat([V, V]), outliers_per_vector=6, outlier_repr="bitmap",
             group_tokens=64, device="cuda")
