"""Head sharding + all-gather of the N>1 path, run as two gloo ranks on CPU.

Each rank attends with its own kv heads only (the CPU oracle stands in for the kernel), the
outputs are all-gathered, and the result must equal the unsharded answer exactly.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ommx_oracle as O
from open_ommx_serve_b200 import sharding
from helpers import gaussian_kv, plane_to_torch, plane_to_numpy, PLANES


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, seq, H, Hq, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D, sink = 128, 8
        K, V = gaussian_kv(5, seq, H, D)
        q = torch.randn(1, Hq, D, generator=torch.Generator().manual_seed(9)).bfloat16().float()
        edge = O.packed_boundary(seq)
        full = O.pack_kv(K[sink:edge].numpy(), V[sink:edge].numpy())
        tail = list(range(sink)) + list(range(edge, seq))
        planes_t = {n: plane_to_torch(n, full[n], "cpu") for n in PLANES}
        mine = sharding.shard_planes(planes_t, rank, world)
        local = dict(full)
        local.update({n: plane_to_numpy(mine[n]) for n in PLANES})
        local["n_kv_heads"] = H // world
        q_l = sharding.shard_heads(q, rank, world, axis=1)[0].numpy()
        kt = sharding.shard_heads(K[tail][None], rank, world, axis=2)[0].numpy()
        vt = sharding.shard_heads(V[tail][None], rank, world, axis=2)[0].numpy()
        o_l, _, _ = O.decode_split_kv(q_l, local, kt, vt, D ** -0.5, 2)
        o = sharding.gather_head_outputs(torch.from_numpy(o_l)[None], world)
        if rank == 0:
            want, _, _ = O.decode_split_kv(q[0].numpy(), full, K[tail].numpy(), V[tail].numpy(), D ** -0.5, 2)
            ret["max_abs"] = float(np.abs(o[0].numpy() - want).max())
            ret["shape"] = tuple(o.shape)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_ranks_equal_unsharded(world):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_rank_main, args=(world, port, 200, 4, 8, ret), nprocs=world, join=True)
        assert ret["shape"] == (1, 8, 128)
        assert ret["max_abs"] == 0.0


def test_shard_range_and_refusals():
    assert sharding.shard_range(8, 3, 4) == (6, 8)
    assert [sharding.shard_range(8, r, 8) for r in (0, 7)] == [(0, 1), (7, 8)]
    with pytest.raises(ValueError):
        sharding.shard_range(8, 0, 3)
    with pytest.raises(ValueError):
        sharding.shard_range(8, 4, 4)
    planes = {"k_base": torch.zeros(2, 16, 8, 32, dtype=torch.uint8), "k_scale": torch.zeros(1, 8, 128, dtype=torch.int8),
              "k_oval": None, "n_kv_heads": 8}
    out = sharding.shard_planes(planes, 1, 4)
    assert out["k_base"].shape == (2, 16, 2, 32) and out["k_scale"].shape == (1, 2, 128)
    assert out["n_kv_heads"] == 2 and out["k_base"].is_contiguous()
