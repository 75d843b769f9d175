"""Every store / pool entry point the reference's serving loops call, held to the reference's own
store criterion (its tests/test_kv_pool_parity.py): planes, residual rows and lengths built step by
step through an entry point equal a from-scratch bulk pack of the full history, byte for byte."""
import pytest
import torch

from oracle import ommx_oracle as O

from helpers import assert_planes_equal, gaussian_kv
from test_kv_pool_gpu import SINK, RECENT, _pool, _seq_planes

pytestmark = pytest.mark.gpu
H, D = 2, 128


def _history(lens, seed=300):
    ks, vs = [], []
    for r, T in enumerate(lens):
        K, V = gaussian_kv(seed + r, T, H, D)
        ks.append(K)
        vs.append(V)
    return ks, vs


def _new_rows(g, B):
    Kn = torch.randn(B, H, D, generator=g).bfloat16()
    Vn = torch.randn(B, H, D, generator=g).bfloat16()
    Kn[:, :, 5] *= 12.0
    return Kn, Vn


def _check_planes(pool, r, hist_k, hist_v):
    T = hist_k.shape[0]
    boundary = O.packed_boundary(T, SINK, RECENT)
    packed = max(0, boundary - SINK)
    if packed:
        want = O.pack_kv(hist_k[SINK:boundary].numpy(), hist_v[SINK:boundary].numpy(), outliers_per_vector=6, page_size=16)
        assert_planes_equal(_seq_planes(pool, r, packed // 32), want, ctx=f"req {r}: ")
    return boundary, packed


def test_append_and_append_decode_batched_with_ragged_slots():
    lens = [100, 40, 333, 7]
    pool = _pool(len(lens), 512, H)
    hk, hv = _history(lens)
    for r in range(len(lens)):
        assert pool.append_block(r, hk[r].cuda().bfloat16(), hv[r].cuda().bfloat16()) == O.packed_boundary(lens[r], SINK, RECENT) // 32
    g = torch.Generator().manual_seed(1)
    total = 0
    for step in range(70):
        slots = [3, 0, 2] if step % 2 == 0 else [1]          # ragged, remapped batches
        Kn, Vn = _new_rows(g, len(slots))
        if len(slots) == 1:
            total += pool.append(slots[0], Kn[0].cuda(), Vn[0].cuda())
        else:
            total += pool.append_decode_batched(slots, Kn.cuda(), Vn.cuda())
        for i, r in enumerate(slots):
            hk[r] = torch.cat([hk[r], Kn[i:i + 1].float()])
            hv[r] = torch.cat([hv[r], Vn[i:i + 1].float()])
    assert pool.seq_lens() == [h.shape[0] for h in hk] == pool.seq_len
    want_groups = [O.packed_boundary(h.shape[0], SINK, RECENT) // 32 - O.packed_boundary(l, SINK, RECENT) // 32
                   for h, l in zip(hk, lens)]
    assert total == sum(want_groups)
    for r in range(len(lens)):
        _check_planes(pool, r, hk[r], hv[r])
        assert pool.regroup(r) == 0
    # read side: decode_inputs_batched over a remapped selection, tail_bf16_batched, request_planes
    sel = [2, 0]
    d = pool.decode_inputs_batched(sel)
    kt, vt, n = pool.tail_bf16_batched(sel)
    for b, r in enumerate(sel):
        T = hk[r].shape[0]
        boundary = O.packed_boundary(T, SINK, RECENT)
        idx = list(range(min(SINK, T))) + list(range(boundary, T))
        assert int(d["b_seq_len"][b]) == boundary - SINK and int(d["b_tail_len"][b]) == len(idx) == int(n[b])
        assert torch.equal(d["k_tail"][b, :len(idx)].cpu(), hk[r][idx].bfloat16())
        assert torch.equal(vt[b, :len(idx)].cpu(), hv[r][idx].bfloat16()) and torch.equal(kt[b, :len(idx)].cpu(), hk[r][idx].bfloat16())
        assert torch.equal(d["req_to_group"][b].cpu(), pool._req_to_group[r].cpu())
        rp = pool.request_planes(r)
        want = O.pack_kv(hk[r][SINK:boundary].numpy(), hv[r][SINK:boundary].numpy(), outliers_per_vector=6, page_size=16)
        assert_planes_equal(rp, want, ctx=f"request_planes {r}: ")
        assert rp["n_groups"] == (boundary - SINK) // 32
    assert d["max_seq_len"] == max(O.packed_boundary(hk[r].shape[0], SINK, RECENT) - SINK for r in sel)
    assert d["planes"]["k_base"] is pool.k_base and d["packed_start_offset"] == 0
    assert int(pool.status.item()) == 0


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_append_decode_captured_and_decode_inputs_captured(idx_dtype):
    """The graph form: device-side (slot, position) indices, caller-owned control tensors, one CUDA graph
    replayed across group boundaries with only the index buffers refreshed in between."""
    lens = [70, 101, 9]
    B = len(lens)
    pool = _pool(4, 512, H)
    slots = [2, 0, 3]                                          # batch row -> pool slot
    hk, hv = _history(lens, seed=40)
    for b, r in enumerate(slots):
        pool.append_block(r, hk[b].cuda().bfloat16(), hv[b].cuda().bfloat16())
    T = pool.max_tail_len
    rows = torch.tensor(slots, dtype=idx_dtype, device="cuda")
    cols = torch.zeros(B, dtype=idx_dtype, device="cuda")
    tidx = torch.zeros(B, T, dtype=idx_dtype, device="cuda")
    kt = torch.zeros(B, T, H, D, dtype=torch.bfloat16, device="cuda")
    vt = torch.zeros_like(kt)
    b_seq = torch.zeros(B, dtype=torch.int32, device="cuda")
    b_tail = torch.zeros(B, dtype=torch.int32, device="cuda")
    Kn_dev = torch.zeros(B, H, D, dtype=torch.bfloat16, device="cuda")
    Vn_dev = torch.zeros_like(Kn_dev)

    def step():
        pool.append_decode_captured(rows, cols, Kn_dev, Vn_dev)
        return pool.decode_inputs_captured(rows, b_seq, b_tail, tidx, kt, vt, 512)

    def refresh(n_new):
        """the host seam: positions of the row about to be written and the residual indices after it"""
        cols.copy_(torch.tensor([h.shape[0] for h in hk], dtype=idx_dtype))
        ti = torch.zeros(B, T, dtype=idx_dtype)
        for b in range(B):
            seq = hk[b].shape[0] + n_new
            bd = O.packed_boundary(seq, SINK, RECENT)
            idx = list(range(min(SINK, seq))) + list(range(bd, seq))
            ti[b, :len(idx)] = torch.tensor(idx, dtype=idx_dtype)
            b_seq[b], b_tail[b] = bd - SINK, len(idx)
        tidx.copy_(ti)

    g = torch.Generator().manual_seed(3)
    graph = None
    for it in range(72):
        Kn, Vn = _new_rows(g, B)
        Kn_dev.copy_(Kn)
        Vn_dev.copy_(Vn)
        refresh(1)
        if it == 0:
            step()                                             # eager once (index check on)
        else:
            if graph is None:
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    d = step()
            graph.replay()
        for b in range(B):
            hk[b] = torch.cat([hk[b], Kn[b:b + 1].float()])
            hv[b] = torch.cat([hv[b], Vn[b:b + 1].float()])
        if it in (0, 1, 30, 31, 32, 71):
            torch.cuda.synchronize()
            for b, r in enumerate(slots):
                boundary, _ = _check_planes(pool, r, hk[b], hv[b])
                idx = list(range(min(SINK, hk[b].shape[0]))) + list(range(boundary, hk[b].shape[0]))
                assert torch.equal(kt[b, :len(idx)].cpu(), hk[b][idx].bfloat16())
                assert torch.equal(vt[b, :len(idx)].cpu(), hv[b][idx].bfloat16())
    assert torch.equal(d["req_to_token"].cpu(), pool._req_to_token[slots].cpu())
    assert int(pool.status.item()) == 0
    bad = rows.clone()
    bad[1] = 99
    with pytest.raises(IndexError):
        pool.append_decode_captured(bad, cols, Kn_dev, Vn_dev)


def test_seed_and_advance_seq_device():
    lens = [50, 120]
    pool = _pool(2, 512, H)
    hk, hv = _history(lens, seed=77)
    for r in range(2):
        pool.append_block(r, hk[r].cuda().bfloat16(), hv[r].cuda().bfloat16())
    seq = pool.decode_seed_seq_device([0, 1])
    assert seq.tolist() == lens
    pool.advance_seq_device(2)
    assert pool.seq_lens() == [51, 121]


def test_step_past_capacity_is_refused_and_leaves_the_neighbour_alone():
    """A request stepped beyond max_seq_len plus its spare group must not write into the next
    request's pages: the row is refused, a status bit is raised, lengths stop advancing."""
    pool = _pool(2, 96, H)                       # 4 group slots per request
    hk, hv = _history([96, 96], seed=9)
    for r in range(2):
        pool.append_block(r, hk[r].cuda().bfloat16(), hv[r].cuda().bfloat16())
    before = {n: t.clone() for n, t in pool.planes.items() if t is not None}
    cap_groups = pool.G_per_seq
    g = torch.Generator().manual_seed(2)
    pool.select_slots([0])
    steps = cap_groups * 32 + SINK + RECENT + 40 - 96       # far enough to complete a group beyond the table row
    for _ in range(steps):
        Kn, Vn = _new_rows(g, 1)
        pool._call(pool._append_args(1, 1, Kn.cuda(), Vn.cuda()))
    assert int(pool.status.item()) & 16                      # OMMX_ST_BAD_LENGTH
    last_ok = SINK + RECENT + cap_groups * 32 + 31           # longest length whose groups fit the table row
    assert pool.seq_lens()[0] == last_ok and pool.seq_lens()[1] == 96
    r1 = _seq_planes(pool, 1, cap_groups)
    p0, g0 = pool.P_per_seq, pool.G_per_seq
    for name, t in r1.items():
        ref = before[name][p0:p0 + cap_groups * pool.pages_per_group] if name in ("k_base", "v_main", "v_scale", "v_zp") \
            else before[name][g0:g0 + cap_groups]
        assert torch.equal(t, ref), f"{name} of the neighbouring request changed"


def test_store_graph_entry_points():
    """CanonicalKVStore: append / maybe_regroup (eager loop) and write_token / advance_to /
    gather_tail_into (graph loop) build the same planes as a bulk pack."""
    from open_ommx_serve_b200.attention.kv_store import CanonicalKVStore
    from open_ommx_serve_b200.attention.kv_window import WindowSpec
    for mode in ("eager", "graph"):
        st = CanonicalKVStore(D, H, 512, outliers_per_vector=6, window=WindowSpec(SINK, RECENT, 32, 16), device="cuda")
        K, V = gaussian_kv(5, 90, H, D)
        st.append_block(K.cuda().bfloat16(), V.cuda().bfloat16())
        assert st.seq_len == 90 and st.packed_groups == 1
        g = torch.Generator().manual_seed(8)
        pos = torch.zeros(1, dtype=torch.int64, device="cuda")
        T = st.pool.max_tail_len
        tail_idx = torch.zeros(T, dtype=torch.int64, device="cuda")
        kt = torch.zeros(1, T, H, D, dtype=torch.bfloat16, device="cuda")
        vt = torch.zeros_like(kt)
        packed_total = 0
        for _ in range(70):
            Kn, Vn = _new_rows(g, 1)
            K, V = torch.cat([K, Kn.float()]), torch.cat([V, Vn.float()])
            if mode == "eager":
                st.append(Kn[0].cuda(), Vn[0].cuda())
                packed_total += st.maybe_regroup()
            else:
                pos.fill_(K.shape[0] - 1)
                st.write_token(pos, Kn[0].cuda(), Vn[0].cuda())
                packed_total += st.advance_to(K.shape[0])
                idx = st.window.tail_indices(K.shape[0])
                tail_idx.zero_()
                tail_idx[:len(idx)] = torch.tensor(idx, device="cuda")
                st.gather_tail_into(tail_idx, kt, vt, len(idx))
                assert torch.equal(kt[0, :len(idx)].cpu(), K[idx].bfloat16())
        assert st.seq_len == 160 and st.packed_groups == (160 - 40) // 32 and packed_total == st.packed_groups - 1
        boundary = O.packed_boundary(160, SINK, RECENT)
        want = O.pack_kv(K[SINK:boundary].numpy(), V[SINK:boundary].numpy(), outliers_per_vector=6, page_size=16)
        assert_planes_equal(st.decode_planes(), want, ctx=mode + ": ")
        kt2, vt2, n = st.tail_bf16()
        idx = st.window.tail_indices(160)
        assert n == len(idx) and torch.equal(kt2[0].cpu(), K[idx].bfloat16()) and torch.equal(vt2[0].cpu(), V[idx].bfloat16())
        assert int(st.pool.status.item()) == 0
