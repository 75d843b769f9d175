"""The head-output exchange fused into stage 2 (ommx_head_gather), two ranks on two GPUs.

Each rank decodes its half of the kv heads of the same cache; stage 2 stores the rows into both ranks'
buffers.  Held against an NCCL all-gather of the same outputs (equal bit for bit: the same floats travel) and
against the unsharded decode on one GPU.  Runs as two child processes (CUDA IPC maps another PROCESS's memory);
skipped with fewer than two GPUs.  Ranks leave only between steps, with nothing in flight."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from helpers import Case
    from open_ommx_serve_b200 import sharding
    from open_ommx_serve_b200.attention.paged_decode import ommx_paged_decode_attention_canonical as decode
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        case = Case([3000, 700], H=8, Hq=32, seed=5, device=dev)
        o_full, _ = case.run(num_kv_splits=7)
        planes = sharding.shard_planes({**case.planes, "n_kv_heads": 8}, rank, world)
        q = sharding.shard_heads(case.q_dev, rank, world, 1)
        k_tail = sharding.shard_heads(case.k_tail, rank, world, 2)
        v_tail = sharding.shard_heads(case.v_tail, rank, world, 2)
        B, hq = q.shape[0], q.shape[1]
        pg = sharding.PeerHeadGather(world, rank, 2, B, hq, 128, dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ok = True
        for step in range(5):                                        # alternating buffers, as layers of a stack do
            o = torch.zeros(B, hq, 128, dtype=torch.float32, device=dev)
            lse = torch.zeros(B, hq, dtype=torch.float32, device=dev)
            decode(q, planes["k_base"], planes["k_scale"], planes["k_zp"], None, planes["k_oval"], planes["v_main"],
                   planes["v_scale"], planes["v_zp"], k_tail, v_tail, case.b_tail_len, o, lse, case.req_to_token,
                   case.req_to_group, case.b_seq_len, sm_scale=case.sm_scale, page_size=16, k_outliers_per_vector=6,
                   bitmap_read=True, k_obmp=planes["k_obmp"], k_fp4_mapscale=planes["k_fp4_mapscale"],
                   k_fp4_mapcenter=planes["k_fp4_mapcenter"], kv_outlier_map=True, kv_int8_scale=True,
                   num_kv_splits=7, max_seq_len=max(case.packed), max_tail_len=max(case.tails), status=status,
                   head_gather=pg.plan(step))
            torch.cuda.synchronize()
            want = torch.empty(world, B, hq, 128, dtype=torch.float32, device=dev)
            dist.all_gather_into_tensor(want, o)
            ok &= torch.equal(pg.gathered(step), want)
            ok &= bool((pg.full_heads(step) - o_full).abs().max().item() < 2e-3)
        ok &= int(status.item()) == 0
        pg.close()
        out_q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_stage2_peer_gather_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29533, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    for p in procs:
        if p.is_alive():                                             # a child that hangs is ended by its exact handle
            p.terminate()
        assert p.exitcode == 0
    got = dict(q.get(timeout=5) for _ in range(2))
    assert got == {0: True, 1: True}


def test_stage2_exchange_indexing_eight_ranks_on_one_gpu():
    """Send and receive indexing of the exchange for 8 ranks, on one GPU: the seven "peers" are plain local buffers.
    Their words are written into this rank's receive buffer beforehand with the call count the kernel will expect, so
    nothing waits for another kernel; afterwards `out` must hold those values in the peers' slots and this rank's rows
    in its own, and every peer buffer must hold this rank's rows as (value, call count) words in slot `rank`."""
    import ctypes as C
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import Case
    from open_ommx_serve_b200 import _lib
    world, rank = 8, 3
    case = Case([700, 300], H=1, Hq=4, seed=9)
    B, hq, D = 2, 4, 128
    dev = torch.device("cuda")
    recv = [torch.zeros(world, B, hq, D, dtype=torch.int64, device=dev) for _ in range(world)]
    gen = torch.Generator().manual_seed(3)
    want = torch.randn(world, B, hq, D, generator=gen).to(dev)
    words = (want.view(torch.int32).to(torch.int64) & 0xFFFFFFFF) | (1 << 32)          # call count 1
    for r in range(world):
        if r != rank:
            recv[rank][r] = words[r]
    recv_ptrs = torch.tensor([t.data_ptr() for t in recv], dtype=torch.int64, device=dev)
    out = torch.zeros(world, B, hq, D, dtype=torch.float32, device=dev)
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    g = _lib.HeadGather()
    g.world, g.rank, g.recv, g.out, g.state = world, rank, recv_ptrs.data_ptr(), out.data_ptr(), state.data_ptr()

    class Plan:
        def check(self, batch, heads, head_dim, device):
            assert (batch, heads, head_dim) == (B, hq, D)
            return C.addressof(g)

    status = torch.zeros(1, dtype=torch.int32, device=dev)
    o, _ = case.run(num_kv_splits=3, status=status, head_gather=Plan())
    assert int(status.item()) == 0 and state.tolist() == [1, 0]
    assert torch.equal(out[rank], o)
    for r in range(world):
        if r == rank:
            continue
        assert torch.equal(out[r], want[r]), f"slot {r} received"
        sent = recv[r][rank]
        assert torch.equal((sent >> 32), torch.ones_like(sent)), f"call count in peer {r}"
        low = sent & 0xFFFFFFFF
        bits = torch.where(low >= 2 ** 31, low - 2 ** 32, low).to(torch.int32)          # the low word as a signed pattern
        assert torch.equal(bits.view(torch.float32), o), f"rows sent to peer {r}"
