"""The relidx7 outlier-index encoding (the reference's other serving preset): pack, re-encode, and decode.

Both encodings list the same outlier positions of a frame, so (a) the packer's relidx7 planes equal the
reference packer's, (b) the two re-encodings invert each other, and (c) decode over relidx7 planes gives the
very same bits as decode over the bitmask planes of the same cache, which the other tests hold to the oracle."""
import numpy as np
import pytest
import torch

from oracle import ommx_oracle as O
from helpers import PLANES, Case, assert_planes_equal, load_golden, plane_to_numpy

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k", [6, 10])
def test_pack_relidx7_equals_reference_fixture(k):
    from open_ommx_serve_b200 import ommx_pack_kv_canonical_block
    g = load_golden(f"pack_relidx7_k{k}")
    got = ommx_pack_kv_canonical_block(torch.from_numpy(g["K"]).cuda(), torch.from_numpy(g["V"]).cuda(), outliers_per_vector=k,
                                       outlier_repr="relidx7", outlier_select="signed", use_pow2=True,
                                       kv_outlier_map=True, page_size=16)
    assert got["k_obmp"] is None and got["outlier_repr"] == "relidx7" and got["k_field_bytes"] == (7 * k + 7) // 8
    want = {n: g[n] for n in PLANES if n in g}
    assert_planes_equal({n: got[n] for n in want}, want, ctx=f"relidx7 k={k}: ")
    assert (plane_to_numpy(got["k_oidx"]) == g["k_oidx"]).all()


@pytest.mark.parametrize("k", [1, 3, 6, 9, 10, 16])
def test_outlier_index_convert_round_trip(k):
    from open_ommx_serve_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(k)
    n = 4096
    masks = np.zeros(n, dtype=np.uint32)
    for i in range(n):
        masks[i] = np.bitwise_or.reduce(np.uint32(1) << rng.choice(32, size=k, replace=False).astype(np.uint32))
    obmp = torch.from_numpy(masks.view(np.uint8).reshape(n, 4).copy()).cuda()
    nbi = (7 * k + 7) // 8
    oidx = torch.zeros(n, nbi, dtype=torch.uint8, device="cuda")
    back = torch.zeros(n, 4, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.ommx_b200_outlier_index_convert(obmp.data_ptr(), oidx.data_ptr(), n, k, 1, status.data_ptr(), stream), "to relidx7")
    _lib.check(lib.ommx_b200_outlier_index_convert(oidx.data_ptr(), back.data_ptr(), n, k, 0, status.data_ptr(), stream), "to bitmask")
    assert int(status.item()) == 0
    assert torch.equal(back, obmp)
    assert (oidx.cpu().numpy() == O.relidx7_from_bitmask(obmp.cpu().numpy(), k)).all()
    bad = oidx.clone()
    bad[0, 0] = 0x7F                                              # position 127: beyond the group
    _lib.check(lib.ommx_b200_outlier_index_convert(bad.data_ptr(), back.data_ptr(), n, k, 0, status.data_ptr(), stream), "bad")
    assert int(status.item()) & _lib.ST_BAD_GROUP


@pytest.mark.parametrize("k,H,Hq", [(6, 8, 32), (10, 8, 32), (4, 2, 8), (10, 1, 8)])
def test_decode_relidx7_planes_equal_bitmask_planes(k, H, Hq):
    case = Case([3000, 500], H=H, Hq=Hq, seed=k + H, k=k)
    o_bm, lse_bm = case.run(num_kv_splits=9)
    obmp = case.pooled_np["k_obmp"]                                # pooled plane: slots no sequence owns are all zero
    words = obmp.reshape(-1, 4).copy().view(np.uint32)[:, 0]
    used = np.array([bin(int(w)).count("1") == k for w in words])
    flat = np.zeros((words.shape[0], (7 * k + 7) // 8), dtype=np.uint8)
    flat[used] = O.relidx7_from_bitmask(obmp.reshape(-1, 4)[used], k)
    oidx = torch.from_numpy(flat.reshape(obmp.shape[:-1] + (flat.shape[1],))).cuda()
    from open_ommx_serve_b200.attention.paged_decode import ommx_paged_decode_attention_canonical
    p = case.planes
    o = torch.zeros_like(o_bm)
    lse = torch.zeros_like(lse_bm)
    ommx_paged_decode_attention_canonical(
        case.q_dev, p["k_base"], p["k_scale"], p["k_zp"], oidx, p["k_oval"], p["v_main"], p["v_scale"], p["v_zp"],
        case.k_tail, case.v_tail, case.b_tail_len, o, lse, case.req_to_token, case.req_to_group, case.b_seq_len,
        sm_scale=case.sm_scale, page_size=16, k_outliers_per_vector=k, bitmap_read=False, k_obmp=None,
        k_fp4_mapscale=p["k_fp4_mapscale"], k_fp4_mapcenter=p["k_fp4_mapcenter"], kv_outlier_map=True,
        kv_int8_scale=True, num_kv_splits=9, max_seq_len=max(case.packed), max_tail_len=max(case.tails))
    torch.cuda.synchronize()
    assert torch.equal(o, o_bm) and torch.equal(lse, lse_bm)
