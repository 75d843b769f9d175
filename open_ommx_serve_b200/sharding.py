"""KV-head sharding of the decode path across the GPUs of one node.

Attention is independent per kv head, so rank ``r`` of ``n`` keeps kv heads
``[r*Hkv/n, (r+1)*Hkv/n)`` of every plane and the query heads that read them; page and group
tables, sequence lengths and residual-row counts are replicated.  Nothing is exchanged during
attention; one all-gather of the ``[B, Hq/n, D]`` head outputs per layer reassembles ``[B, Hq, D]``.
This is the split vLLM tensor parallelism applies to the reference backend
(ommx_gpu_serve/integration/vllm/backend.py:859-873 of the reference).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

#: planes indexed [pages, page_size, H, ...] (head axis 2) and [group_slots, H, D, ...] (head axis 1)
PAGE_PLANES = ("k_base", "v_main", "v_scale", "v_zp")
GROUP_PLANES = ("k_scale", "k_zp", "k_obmp", "k_oval", "k_fp4_mapscale", "k_fp4_mapcenter")


def shard_range(n_heads: int, rank: int, world: int):
    """Half-open head range owned by ``rank``; ``n_heads`` must divide evenly."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank={rank} world={world}")
    if n_heads % world != 0:
        raise ValueError(f"{n_heads} heads do not split over {world} ranks")
    per = n_heads // world
    return rank * per, (rank + 1) * per


def shard_planes(planes: dict, rank: int, world: int) -> dict:
    """This rank's kv heads of every plane, as contiguous tensors (other entries pass through)."""
    out = dict(planes)
    for name in PAGE_PLANES + GROUP_PLANES:
        t = planes.get(name)
        if t is None:
            continue
        axis = 2 if name in PAGE_PLANES else 1
        lo, hi = shard_range(int(t.shape[axis]), rank, world)
        out[name] = t.narrow(axis, lo, hi - lo).contiguous()
    if "n_kv_heads" in out:
        out["n_kv_heads"] = int(out["k_base"].shape[2])
    return out


def shard_heads(x: torch.Tensor, rank: int, world: int, axis: int) -> torch.Tensor:
    """Slice the head axis of q ``[B,Hq,D]`` (axis 1) or of residual rows ``[B,T,Hkv,D]`` (axis 2)."""
    lo, hi = shard_range(int(x.shape[axis]), rank, world)
    return x.narrow(axis, lo, hi - lo).contiguous()


def gather_head_outputs(o_local: torch.Tensor, world: int, group=None,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather ``[B, Hq/n, D]`` head outputs into ``[B, Hq, D]`` (rank order = head order)."""
    import torch.distributed as dist
    if world == 1:
        return o_local
    B, hq, D = o_local.shape
    stacked = torch.empty(world, B, hq, D, dtype=o_local.dtype, device=o_local.device) if out is None else out
    try:
        dist.all_gather_into_tensor(stacked, o_local.contiguous(), group=group)
    except (RuntimeError, NotImplementedError):          # backends without the tensor form
        parts = [torch.empty_like(o_local) for _ in range(world)]
        dist.all_gather(parts, o_local.contiguous(), group=group)
        stacked = torch.stack(parts)
    return stacked.permute(1, 0, 2, 3).reshape(B, world * hq, D)


class _GatherPlan:
    """One call's ``ommx_head_gather`` descriptor plus the geometry it was built for."""

    def __init__(self, owner, index):
        self.owner, self.index = owner, index

    def check(self, batch, n_q_heads, head_dim, device):
        o = self.owner
        if (batch, n_q_heads, head_dim) != (o.batch, o.hq_local, o.head_dim) or device != o.device:
            raise ValueError(f"head_gather was built for batch {o.batch} x {o.hq_local} heads x {o.head_dim} on {o.device}")
        return C.addressof(o._structs[self.index])


class PeerHeadGather:
    """The head-output exchange of a kv-head sharded decode, fused into stage 2 (``ommx_head_gather``).

    Stands where the reference's serving stack runs a collective on the attention output of its tensor-parallel
    ranks (ommx_gpu_serve/integration/vllm/backend.py:859-873 shards the heads; the gather itself is vLLM's).
    Every rank allocates ``buffers`` receive buffers ``[world, batch, Hq/n, D]`` of 8-byte (value, call count)
    words in memory the other processes of the node map over NVLink (CUDA IPC); handles travel once through
    ``torch.distributed``.  A decode call given ``head_gather=gather.plan(i)`` leaves all ranks' rows in
    ``gather.gathered(i)`` (a plain local f32 tensor) when its kernels are done.  Every rank must make the same
    sequence of such calls, and consecutive calls must use different buffers (layers of a stack do).  NCCL
    (``gather_head_outputs``) remains the plain alternative.
    """

    def __init__(self, world: int, rank: int, buffers: int, batch: int, hq_local: int, head_dim: int,
                 device: torch.device, group=None):
        import torch.distributed as dist
        from . import _lib
        if not 2 <= world <= 32:
            raise ValueError("PeerHeadGather serves 2..32 ranks")
        if buffers < 2:
            raise ValueError("at least two buffers: a peer may be one call ahead")
        self.world, self.rank, self.buffers = world, rank, buffers
        self.batch, self.hq_local, self.head_dim, self.device = batch, hq_local, head_dim, torch.device(device)
        self._lib = lib = _lib.load()
        self.buf_words = world * batch * hq_local * head_dim
        self.bytes = buffers * self.buf_words * 8
        self._own = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        # Every step that can fail on one rank alone is followed by a vote, so that all ranks raise together instead
        # of one leaving the others inside a collective.
        with torch.cuda.device(self.device):
            rc = lib.ommx_b200_peer_alloc(self.bytes, C.byref(self._own), handle)
        why = "" if rc == 0 else _lib.last_error()
        self._vote(rc == 0, "ommx_b200_peer_alloc: " + why, group)
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._bases, self._opened = [], []
        ok, why = True, ""
        for r in range(world):
            if r == rank:
                self._bases.append(int(self._own.value))
                continue
            ptr = C.c_void_p()
            h = (C.c_uint8 * 64).from_buffer_copy(handles[r])
            with torch.cuda.device(self.device):
                rc = lib.ommx_b200_peer_open(h, C.byref(ptr))
            if rc != 0:
                ok, why = False, _lib.last_error()
                break
            self._bases.append(int(ptr.value))
            self._opened.append(int(ptr.value))
        self._vote(ok, "ommx_b200_peer_open: " + why, group)
        # device-side pointer table recv[buffer][r]; results and the two state words are plain local tensors
        self._recv = torch.tensor([[b + i * self.buf_words * 8 for b in self._bases] for i in range(buffers)],
                                  dtype=torch.int64).to(self.device)
        self._out = torch.zeros(buffers, world, batch, hq_local, head_dim, dtype=torch.float32, device=self.device)
        self._state = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._structs = (_lib.HeadGather * buffers)()
        for i in range(buffers):
            g = self._structs[i]
            g.world, g.rank = world, rank
            g.recv = self._recv[i].data_ptr()
            g.out = self._out[i].data_ptr()
            g.state = self._state.data_ptr()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)                                 # every rank has mapped every buffer

    def _vote(self, ok: bool, what: str, group):
        """All ranks learn whether any of them failed; on failure each releases what it holds and raises."""
        import torch.distributed as dist
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 1:
            return
        with torch.cuda.device(self.device):
            for p in getattr(self, "_opened", []):
                self._lib.ommx_b200_peer_close(p)
            self._opened = []
            if self._own.value:
                self._lib.ommx_b200_peer_free(self._own)
                self._own = C.c_void_p()
        raise RuntimeError("PeerHeadGather: peer memory could not be set up on every rank"
                           + ("" if ok else f" (this rank: {what})"))

    def plan(self, i: int) -> _GatherPlan:
        return _GatherPlan(self, i % self.buffers)

    def gathered(self, i: int) -> torch.Tensor:
        """``[world, batch, Hq/n, D]`` f32 result of buffer ``i``: rank r's heads in slot r."""
        return self._out[i % self.buffers]

    def all_buffers(self) -> torch.Tensor:
        """``[buffers, world, batch, Hq/n, D]`` f32: every buffer's result."""
        return self._out

    def full_heads(self, i: int) -> torch.Tensor:
        """``[batch, Hq, D]`` (rank order = head order), a copy."""
        v = self.gathered(i)
        return v.permute(1, 0, 2, 3).reshape(self.batch, self.world * self.hq_local, self.head_dim)

    def close(self, group=None):
        """Unmap the peers' memory and free the own allocation; call on every rank, with no kernel in flight."""
        import torch.distributed as dist
        from . import _lib
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)                                 # nobody stores into a buffer that is going away
        with torch.cuda.device(self.device):
            for p in self._opened:
                _lib.check(self._lib.ommx_b200_peer_close(p), "ommx_b200_peer_close")
            self._opened = []
            dist.barrier(group=group)
            if self._own.value:
                _lib.check(self._lib.ommx_b200_peer_free(self._own), "ommx_b200_peer_free")
                self._own = C.c_void_p()
