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


def test_decode_step_is_graph_capturable():
    """One CUDA graph holds store + decode of a step; replaying it walks the sequences forward,
    including the steps on which a group completes, with no host work between replays."""
    from open_ommx_serve_b200 import ommx_paged_decode_attention_canonical
    from open_ommx_serve_b200.attention.paged_decode import _auto_num_kv_splits
    H, Hq, lens, B = 2, 8, [70, 200], 2
    pool = _pool(B, 512, H)
    eager = _pool(B, 512, H)
    for r, T in enumerate(lens):
        K, V = gaussian_kv(300 + r, T, H, 128)
        for pl in (pool, eager):
            pl.append_block(r, K.cuda().bfloat16(), V.cuda().bfloat16())
    k_in = torch.zeros(B, H, 128, dtype=torch.bfloat16, device="cuda")
    v_in = torch.zeros_like(k_in)
    q_in = torch.zeros(B, Hq, 128, dtype=torch.bfloat16, device="cuda")
    o = torch.zeros(B, Hq, 128, device="cuda")
    lse = torch.zeros(B, Hq, device="cuda")
    max_packed = pool.window.packed_len(512)
    splits = _auto_num_kv_splits(max_packed, B, device=torch.device("cuda"), kv_heads=H)
    ws = torch.empty(B, Hq, splits + 1, 129, device="cuda")

    def step(pl, out_o, out_lse):
        pl.append_decode_device(k_in, v_in, B)
        d = pl.decode_inputs_device(B, max_packed)
        ommx_paged_decode_attention_canonical(
            q_in, d["k_base"], d["k_scale"], d["k_zp"], None, d["k_oval"], d["v_main"], d["v_scale"], d["v_zp"],
            d["k_tail"], d["v_tail"], d["b_tail_len"], out_o, out_lse, d["req_to_token"], d["req_to_group"],
            d["b_seq_len"], sm_scale=128 ** -0.5, page_size=d["page_size"], k_outliers_per_vector=6,
            bitmap_read=True, k_obmp=d["k_obmp"], k_fp4_mapscale=d["k_fp4_mapscale"],
            k_fp4_mapcenter=d["k_fp4_mapcenter"], kv_outlier_map=True, kv_int8_scale=True, num_kv_splits=splits,
            max_seq_len=d["max_seq_len"], max_tail_len=d["max_tail_len"], attn_logits=ws)

    g = torch.Generator().manual_seed(3)
    rows = [(torch.randn(B, H, 128, generator=g).bfloat16(), torch.randn(B, H, 128, generator=g).bfloat16(),
             torch.randn(B, Hq, 128, generator=g).bfloat16()) for _ in range(41)]
    k_in.copy_(rows[0][0]); v_in.copy_(rows[0][1]); q_in.copy_(rows[0][2])
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        step(pool, o, lse)                                    # warm-up outside capture (step 0)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    k_in.copy_(rows[1][0]); v_in.copy_(rows[1][1]); q_in.copy_(rows[1][2])
    with torch.cuda.graph(graph):
        step(pool, o, lse)                                    # capture launches nothing: step 1 runs at first replay
    o_e = torch.zeros_like(o)
    lse_e = torch.zeros_like(lse)
    k_keep, v_keep, q_keep = k_in.clone(), v_in.clone(), q_in.clone()
    k_in.copy_(rows[0][0]); v_in.copy_(rows[0][1]); q_in.copy_(rows[0][2])
    step(eager, o_e, lse_e)
    for i in range(1, 41):
        k_in.copy_(rows[i][0]); v_in.copy_(rows[i][1]); q_in.copy_(rows[i][2])
        graph.replay()
        step(eager, o_e, lse_e)
        assert torch.equal(o, o_e) and torch.equal(lse, lse_e), f"step {i}"
    assert pool.seq_lens() == eager.seq_lens() == [lens[0] + 41, lens[1] + 41]
    for name, t in pool.planes.items():
        if t is not None:
            assert torch.equal(t, eager.planes[name]), name
    del k_keep, v_keep, q_keep


def test_selected_slots_remap_batch_rows():
    """Batch rows can stand for any distinct request slots; the others are left untouched."""
    H = 2
    pool = _pool(4, 512, H)
    hist = {}
    for r, T in enumerate([50, 120, 75, 200]):
        K, V = gaussian_kv(400 + r, T, H, 128)
        pool.append_block(r, K.cuda().bfloat16(), V.cuda().bfloat16())
        hist[r] = [K, V]
    pool.select_slots([3, 1])
    g = torch.Generator().manual_seed(2)
    for _ in range(40):
        Kn, Vn = torch.randn(2, H, 128, generator=g).bfloat16(), torch.randn(2, H, 128, generator=g).bfloat16()
        pool.append_decode_device(Kn.cuda(), Vn.cuda(), 2)
        for row, r in enumerate((3, 1)):
            hist[r][0] = torch.cat([hist[r][0], Kn[row:row + 1].float()])
            hist[r][1] = torch.cat([hist[r][1], Vn[row:row + 1].float()])
    assert pool.seq_lens() == [50, 160, 75, 240]
    d = pool.decode_inputs_device(2)
    assert d["req_to_group"][0, 0].item() == 3 * pool.G_per_seq and d["req_to_group"][1, 0].item() == pool.G_per_seq
    for row, r in enumerate((3, 1)):
        T = hist[r][0].shape[0]
        boundary = O.packed_boundary(T, SINK, RECENT)
        assert int(pool.b_seq[row].item()) == boundary - SINK
        want = O.pack_kv(hist[r][0][SINK:boundary].numpy(), hist[r][1][SINK:boundary].numpy(), outliers_per_vector=6)
        assert_planes_equal(_seq_planes(pool, r, (boundary - SINK) // 32), want, ctx=f"slot {r}: ")
        tail_idx = list(range(SINK)) + list(range(boundary, T))
        assert torch.equal(pool.k_tail[row, :len(tail_idx)].cpu(), hist[r][0][tail_idx].bfloat16())
    with pytest.raises(ValueError):
        pool.select_slots([1, 1])
    with pytest.raises(ValueError):
        pool.append_decode_device(torch.zeros(3, H, 128, dtype=torch.bfloat16, device="cuda"),
                                  torch.zeros(3, H, 128, dtype=torch.bfloat16, device="cuda"), 3)


def test_single_request_store_mirrors_the_pool():
    from open_ommx_serve_b200.attention.kv_store import CanonicalKVStore
    from open_ommx_serve_b200.attention.kv_window import WindowSpec
    H = 2
    st = CanonicalKVStore(128, H, 512, window=WindowSpec(SINK, RECENT, 32, 16))
    K, V = gaussian_kv(77, 90, H, 128)
    st.append_block(K.cuda().bfloat16(), V.cuda().bfloat16())
    g = torch.Generator().manual_seed(1)
    for _ in range(50):
        kn, vn = torch.randn(H, 128, generator=g).bfloat16(), torch.randn(H, 128, generator=g).bfloat16()
        st.append(kn.cuda(), vn.cuda())
        K, V = torch.cat([K, kn[None].float()]), torch.cat([V, vn[None].float()])
    assert st.seq_len == 140
    _check_against_history(st.pool, [K], [V])
    d = st.decode_inputs()
    assert int(d["b_seq_len"].item()) == 96 and d["planes"]["req_to_group"].shape[0] == 1
    with pytest.raises(RuntimeError):
        st.append_block(K.cuda().bfloat16(), V.cuda().bfloat16())
    st.reset_inplace()
    assert st.seq_len == 0


def test_refusals():
    from open_ommx_serve_b200.attention.kv_pool import MultiSeqKVPool
    with pytest.raises(NotImplementedError):
        MultiSeqKVPool(128, 2, 1, 256, outlier_repr="relidx7")
    with pytest.raises(NotImplementedError):
        MultiSeqKVPool(128, 2, 1, 256, outliers_per_vector=3)
    pool = _pool(1, 256, 2)
    with pytest.raises(ValueError):
        pool.append_decode_device(torch.zeros(1, 2, 128, device="cuda"), torch.zeros(1, 2, 128, device="cuda"), 1)
