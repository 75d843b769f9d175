"""KV-head sharding of the decode path across the GPUs of one node.

Attention is independent per kv head, so rank ``r`` of ``n`` keeps kv heads
``[r*Hkv/n, (r+1)*Hkv/n)`` of every plane and the query heads that read them; page and group
tables, sequence lengths and residual-row counts are replicated.  Nothing is exchanged during
attention; one all-gather of the ``[B, Hq/n, D]`` head outputs per layer reassembles ``[B, Hq, D]``.
This is the split vLLM tensor parallelism applies to the reference backend
(ommx_gpu_serve/integration/vllm/backend.py:859-873 of the reference).
"""
from __future__ import annotations

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
