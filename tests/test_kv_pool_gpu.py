"""Device-resident KV pool (store side of the decode path) against the oracle.

Follows the reference's own store tests (test_kv_pool_parity.py: planes built incrementally equal
planes packed in bulk, byte for byte) with the CPU oracle as the bulk packer: sequences are
prefilled, decoded for a number of steps through ``append_decode_device`` only, and then every
plane, residual row and length is compared with a from-scratch pack of the full history."""
import numpy as np
import pytest
import torch

from oracle import ommx_oracle as O

from helpers import assert_planes_equal, check_fp32, gaussian_kv

pytestmark = pytest.mark.gpu

SINK, RECENT = 8, 32


def _pool(num_seqs, max_len, H, k=6, page_size=16):
    from open_ommx_serve_b200.attention.kv_pool import MultiSeqKVPool
    from open_ommx_serve_b200.attention.kv_window import WindowSpec
    return MultiSeqKVPool(128, H, num_seqs, max_len, outliers_per_vector=k,
                          window=WindowSpec(SINK, RECENT, 32, page_size), device="cuda")


def _seq_planes(pool, r, groups):
    """The plane rows request ``r`` owns, as a dict shaped like the oracle's output for ``groups`` groups."""
    ppg = pool.pages_per_group
    p0, g0 = r * pool.P_per_seq, r * pool.G_per_seq
    out = {}
    for name, t in pool.planes.items():
        if t is None:
            continue
        if name in ("k_base", "v_main", "v_scale", "v_zp"):
            out[name] = t[p0:p0 + groups * ppg]
        else:
            out[name] = t[g0:g0 + groups]
    return out


def _check_against_history(pool, hist_k, hist_v, k=6, page_size=16):
    B = len(hist_k)
    seqs = pool.seq_lens()
    for r in range(B):
        T = hist_k[r].shape[0]
        assert seqs[r] == T
        boundary = O.packed_boundary(T, SINK, RECENT)
        packed = max(0, boundary - SINK)
        assert int(pool.b_seq[r].item()) == packed
        tail_idx = list(range(min(SINK, T))) + list(range(boundary, T))
        assert int(pool.b_tail[r].item()) == len(tail_idx)
        want_k = hist_k[r][tail_idx].bfloat16()
        want_v = hist_v[r][tail_idx].bfloat16()
        assert torch.equal(pool.k_tail[r, :len(tail_idx)].cpu(), want_k), f"req {r}: residual K rows"
        assert torch.equal(pool.v_tail[r, :len(tail_idx)].cpu(), want_v), f"req {r}: residual V rows"
        if packed:
            want = O.pack_kv(hist_k[r][SINK:boundary].numpy(), hist_v[r][SINK:boundary].numpy(),
                             outliers_per_vector=k, page_size=page_size)
            assert_planes_equal(_seq_planes(pool, r, packed // 32), want, ctx=f"req {r}: ")
    assert int(pool.status.item()) == 0


@pytest.mark.parametrize("k,page_size", [(6, 16), (0, 16), (4, 8), (8, 32)])
def test_incremental_store_equals_bulk_pack(k, page_size):
    H, lens, steps = 2, [100, 40, 333, 7], 75
    pool = _pool(len(lens), 512, H, k=k, page_size=page_size)
    hist_k, hist_v = [], []
    for r, T in enumerate(lens):
        K, V = gaussian_kv(100 + r, T, H, 128)
        pool.append_block(r, K.cuda().bfloat16(), V.cuda().bfloat16())
        hist_k.append(K)
        hist_v.append(V)
    pool.decode_inputs_device(len(lens), refresh=True)
    _check_against_history(pool, hist_k, hist_v, k=k, page_size=page_size)
    g = torch.Generator().manual_seed(5)
    for step in range(steps):
        Kn = torch.randn(len(lens), H, 128, generator=g).bfloat16()
        Vn = torch.randn(len(lens), H, 128, generator=g).bfloat16()
        Kn[:, :, 3] *= 12.0
        pool.append_decode_device(Kn.cuda(), Vn.cuda(), len(lens))
        for r in range(len(lens)):
            hist_k[r] = torch.cat([hist_k[r], Kn[r:r + 1].float()])
            hist_v[r] = torch.cat([hist_v[r], Vn[r:r + 1].float()])
        if step in (0, 23, 24, 31, 32, 55, steps - 1):
            _check_against_history(pool, hist_k, hist_v, k=k, page_size=page_size)


def test_store_feeds_decode_without_host_state():
    """append_decode_device -> decode_inputs_device -> the decode kernels, with nothing in between."""
    from open_ommx_serve_b200 import ommx_paged_decode_attention_canonical
    H, Hq, lens = 2, 8, [300, 90]
    pool = _pool(len(lens), 1024, H)
    hist_k, hist_v = [], []
    for r, T in enumerate(lens):
        K, V = gaussian_kv(200 + r, T, H, 128)
        pool.append_block(r, K.cuda().bfloat16(), V.cuda().bfloat16())
        hist_k.append(K)
        hist_v.append(V)
    g = torch.Generator().manual_seed(9)
    B = len(lens)
    o = torch.zeros(B, Hq, 128, device="cuda")
    lse = torch.zeros(B, Hq, device="cuda")
    for step in range(40):
        Kn = torch.randn(B, H, 128, generator=g).bfloat16()
        Vn = torch.randn(B, H, 128, generator=g).bfloat16()
        pool.append_decode_device(Kn.cuda(), Vn.cuda(), B)
        for r in range(B):
            hist_k[r] = torch.cat([hist_k[r], Kn[r:r + 1].float()])
            hist_v[r] = torch.cat([hist_v[r], Vn[r:r + 1].float()])
    q = torch.randn(B, Hq, 128, generator=g).bfloat16()
    d = pool.decode_inputs_device(B)
    ommx_paged_decode_attention_canonical(
        q.cuda(), d["k_base"], d["k_scale"], d["k_zp"], None, d["k_oval"], d["v_main"], d["v_scale"], d["v_zp"],
        d["k_tail"], d["v_tail"], d["b_tail_len"], o, lse, d["req_to_token"], d["req_to_group"], d["b_seq_len"],
        sm_scale=128 ** -0.5, page_size=d["page_size"], k_outliers_per_vector=d["k_outliers_per_vector"],
        bitmap_read=True, k_obmp=d["k_obmp"], k_fp4_mapscale=d["k_fp4_mapscale"],
        k_fp4_mapcenter=d["k_fp4_mapcenter"], kv_outlier_map=True, kv_int8_scale=True,
        max_seq_len=d["max_seq_len"], max_tail_len=d["max_tail_len"])
    for r in range(B):
        T = hist_k[r].shape[0]
        boundary = O.packed_boundary(T, SINK, RECENT)
        pl = O.pack_kv(hist_k[r][SINK:boundary].numpy(), hist_v[r][SINK:boundary].numpy(), outliers_per_vector=6)
        Kd, Vd = O.dequant_kv(pl)
        Kf = np.concatenate([hist_k[r][:SINK].numpy(), Kd, hist_k[r][boundary:].numpy()])
        Vf = np.concatenate([hist_v[r][:SINK].numpy(), Vd, hist_v[r][boundary:].numpy()])
        want, _ = O.attention_fp32(q[r].float().numpy(), Kf, Vf, 128 ** -0.5)
        check_fp32(o[r], want, ctx=f"req {r}")


def test_refusals():
    from open_ommx_serve_b200.attention.kv_pool import MultiSeqKVPool
    with pytest.raises(NotImplementedError):
        MultiSeqKVPool(128, 2, 1, 256, outlier_repr="relidx7")
    with pytest.raises(NotImplementedError):
        MultiSeqKVPool(128, 2, 1, 256, outliers_per_vector=3)
    pool = _pool(1, 256, 2)
    with pytest.raises(ValueError):
        pool.append_decode_device(torch.zeros(1, 2, 128, device="cuda"), torch.zeros(1, 2, 128, device="cuda"), 1)
