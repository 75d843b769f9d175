"""Single-request KV store for the decode hot path.

Mirror of ``CanonicalKVStore`` in the reference (``ommx_gpu_serve/attention/kv_store.py:93``) for
the ring-sized, bitmap / power-of-two serving recipe, with the methods its two callers use:

* the eager decode loop (``hf_eager/_ommx_llama_modeling.py``): ``append_block`` :429, ``append``
  :349, ``maybe_regroup`` :492, ``decode_inputs`` :696, ``decode_planes`` :614, ``tail_bf16`` :678;
* the CUDA-graph decode path (``integration/vllm/metadata.py``): ``write_token`` :361 and
  ``gather_tail_into`` :397 inside the captured region with device-side indices, ``advance_to``
  :387 on the host between replays, ``decode_planes_full`` :651, ``reset_inplace`` :331.

It is the one-request case of :class:`MultiSeqKVPool`.  A row write - ``append`` or
``write_token`` - is one library call that also quantizes and packs the 32-token group the row
completed, on the device, so ``maybe_regroup`` / ``advance_to`` only keep the host-side counters
(``seq_len``, ``packed_groups``) in step and report how many groups that covered.  Residual history
is ring sized (the reference's ``OMMX_KV_RING=1`` layout); the full-history layout is not built.
"""
from __future__ import annotations

from typing import Optional

import torch

from .kv_pool import MultiSeqKVPool
from .kv_window import WindowSpec


class CanonicalKVStore:
    def __init__(self, head_dim: int, n_kv_heads: int, max_seq_len: int, *, k_format: str = "i2f4",
                 v_format: str = "i2", outliers_per_vector: int = 6, outlier_select: str = "signed", outlier_repr: str = "bitmap",
                 use_pow2: bool = True, kv_outlier_map: Optional[bool] = True, kv_int8_scale: Optional[bool] = True,
                 window: Optional[WindowSpec] = None, group_channels: int = 32,
                 scale_dtype: torch.dtype = torch.bfloat16, device="cuda") -> None:
        if str(v_format).lower() not in ("i2", "bf16"):
            raise ValueError(f"v_format must be i2|bf16; got {v_format!r}")
        if str(v_format).lower() != "i2":
            raise NotImplementedError("v_format 'bf16' is not served (INT2 V)")
        self.pool = MultiSeqKVPool(head_dim, n_kv_heads, 1, max_seq_len, k_format=k_format,
                                   outliers_per_vector=outliers_per_vector, outlier_select=outlier_select,
                                   outlier_repr=outlier_repr, use_pow2=use_pow2, kv_outlier_map=kv_outlier_map,
                                   kv_int8_scale=kv_int8_scale, window=window, group_channels=group_channels,
                                   scale_dtype=scale_dtype, device=device)
        p = self.pool
        self.D, self.H, self.k, self.ps, self.gt, self.gc = p.D, p.H, p.k, p.ps, p.gt, p.gc
        self.window, self.device, self.max_seq_len = p.window, p.device, p.max_seq_len
        self.kv_cap = self.max_seq_len
        self.k_format, self.v_format = "i2f4", "int2"
        self.outlier_repr, self.outlier_select = p.outlier_repr, p.outlier_select
        self.kv_outlier_map, self.kv_int8_scale, self.kv_ring = p.kv_outlier_map, True, True
        self.pages_per_group, self.G_cap, self.P_cap = p.pages_per_group, p.G_cap, p.P_cap
        self.k_hist, self.v_hist = p.k_hist[0], p.v_hist[0]          # [ring_cap, H, D] views
        self._req_to_token_full, self._req_to_group_full = p._req_to_token, p._req_to_group
        self._row = torch.zeros(1, dtype=torch.int64, device=self.device)

    # host-side counters, shared with the pool's lists
    seq_len = property(lambda self: self.pool.seq_len[0], lambda self, v: self._set_seq(v))
    packed_groups = property(lambda self: self.pool.packed_groups[0],
                             lambda self, v: self.pool.packed_groups.__setitem__(0, int(v)))

    def _set_seq(self, v) -> None:
        self.pool.seq_len[0] = int(v)
        self.pool.seq_dev.fill_(int(v))

    # plane tensors under the reference's attribute names
    k_base = property(lambda self: self.pool.k_base)
    k_scale = property(lambda self: self.pool.k_scale)
    k_zp = property(lambda self: self.pool.k_zp)
    k_obmp = property(lambda self: self.pool.k_obmp)
    k_oval = property(lambda self: self.pool.k_oval)
    k_fp4_mapscale = property(lambda self: self.pool.k_fp4_mapscale)
    k_fp4_mapcenter = property(lambda self: self.pool.k_fp4_mapcenter)
    v_main = property(lambda self: self.pool.v_main)
    v_scale = property(lambda self: self.pool.v_scale)
    v_zp = property(lambda self: self.pool.v_zp)
    k_oidx = k_crank = None

    def _ring_slot_host(self, pos: int) -> int:
        return self.pool._ring_slot_host(pos)

    def _ring_slot_dev(self, pos: torch.Tensor) -> torch.Tensor:
        return self.pool._ring_slot_dev(pos)

    # ── write path ───────────────────────────────────────────────────────────
    def reset_inplace(self) -> None:
        """New sequence in the same tensors (addresses a captured graph holds stay valid)."""
        self.seq_len = 0
        self.packed_groups = 0

    def append_block(self, K: torch.Tensor, V: torch.Tensor) -> None:
        """Prefill block ``[T, H, D]`` into a fresh store."""
        if self.seq_len != 0:
            raise RuntimeError("ring append_block expects a fresh store (seq_len==0); chunked prefill under the "
                               "ring layout is unsupported (the ring cannot retain an unpacked prefix). "
                               "Call reset_inplace() before each prefill block.")
        self.pool.append_block(0, K, V)
        self.pool.decode_inputs_device(1, refresh=True)

    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """One decode step's K/V row ``[H, D]``: ring write, pack of a completed group, lengths."""
        counted = self.packed_groups
        self.pool.append_decode_batched([0], k.reshape(1, self.H, self.D), v.reshape(1, self.H, self.D))
        self.packed_groups = counted            # the reference counts completed groups in maybe_regroup(), not here

    def write_token(self, pos: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        """Capture-safe row write at the device-side absolute position ``pos`` (``[1]`` int64 or int32): ring
        write plus quantize + pack of the group that position completes.  Leaves the lengths to
        ``advance_to`` on the host, as in the reference."""
        if pos.dim() != 1 or int(pos.numel()) != 1 or not pos.is_cuda:
            raise ValueError("pos must be a CUDA tensor of one element")
        row = self._row if pos.dtype == torch.int64 else self._row.to(torch.int32)
        self.pool.append_decode_captured(row, pos, k.reshape(1, self.H, self.D), v.reshape(1, self.H, self.D))

    def advance_to(self, seq_len: int) -> int:
        """Host seam between replays: set the current length; returns the groups completed since the last
        count (the row writes have packed them already)."""
        self.seq_len = int(seq_len)
        return self.maybe_regroup()

    def maybe_regroup(self) -> int:
        return self.pool.regroup(0)

    def gather_tail_into(self, tail_idx: torch.Tensor, k_tail: torch.Tensor, v_tail: torch.Tensor,
                         n_valid: int = 0) -> None:
        """Capture-safe gather of the residual rows at absolute positions ``tail_idx`` (``[T]`` device int) into
        the fixed ``[1, T, H, D]`` buffers; entries past ``n_valid`` are the caller's padding (position 0)."""
        T = int(tail_idx.numel())
        self.pool._gather_tail(None, tail_idx.reshape(1, T), k_tail.reshape(1, T, self.H, self.D),
                               v_tail.reshape(1, T, self.H, self.D))

    # ── read path ────────────────────────────────────────────────────────────
    def decode_planes(self) -> dict:
        """Plane dict sliced to the packed prefix (shapes grow with the sequence; for eager use)."""
        G = self.packed_groups
        P = G * self.pages_per_group
        pl = self.pool.planes

        def cut(name, n):
            t = pl.get(name)
            return None if t is None else t[:n]

        return {"k_base": cut("k_base", P), "k_scale": cut("k_scale", G), "k_zp": cut("k_zp", G), "k_oidx": None,
                "k_oval": cut("k_oval", G), "k_crank": None, "k_obmp": cut("k_obmp", G),
                "k_fp4_mapscale": cut("k_fp4_mapscale", G), "k_fp4_mapcenter": cut("k_fp4_mapcenter", G),
                "v_main": cut("v_main", P), "v_scale": cut("v_scale", P), "v_zp": cut("v_zp", P),
                "req_to_token": torch.arange(P, dtype=torch.int32, device=self.device).reshape(1, P),
                "req_to_group": torch.arange(G, dtype=torch.int32, device=self.device).reshape(1, G),
                "head_dim": self.D, "n_kv_heads": self.H, "num_tokens": G * self.gt, "n_groups": G,
                "page_size": self.ps, "outliers_per_vector": self.k, "outlier_repr": self.outlier_repr,
                "outlier_select": self.outlier_select, "group_tokens": self.gt, "group_channels": self.gc,
                "k_format": self.k_format, "v_format": self.v_format, "k_base_bits": 2, "oval_bits": 4,
                "kv_outlier_map": bool(self.kv_outlier_map), "kv_int8_scale": True}

    def decode_planes_full(self) -> dict:
        """Full-capacity, fixed-address planes and identity tables (what a captured graph binds)."""
        pl, p = self.pool.planes, self.pool
        return {"k_base": pl["k_base"], "k_scale": pl["k_scale"], "k_zp": pl["k_zp"], "k_oidx": None,
                "k_oval": pl.get("k_oval"), "k_crank": None, "k_obmp": pl.get("k_obmp"), "outlier_repr": "bitmap",
                "k_fp4_mapscale": pl.get("k_fp4_mapscale"), "k_fp4_mapcenter": pl.get("k_fp4_mapcenter"),
                "v_main": pl["v_main"], "v_scale": pl["v_scale"], "v_zp": pl["v_zp"],
                "req_to_token": p._req_to_token, "req_to_group": p._req_to_group,
                "page_size": self.ps, "outliers_per_vector": self.k, "k_format": "i2f4", "v_format": "int2",
                "head_dim": self.D, "n_kv_heads": self.H, "kv_outlier_map": bool(p.kv_outlier_map),
                "kv_int8_scale": True}

    def tail_bf16(self):
        """bf16 residual rows (sink, then everything from the boundary on): ``(k_tail, v_tail, n_rows)`` with
        ``[1, n_rows, H, D]`` tensors."""
        idx = self.window.tail_indices(self.seq_len)
        if not idx:
            kt = torch.zeros(1, 0, self.H, self.D, dtype=torch.bfloat16, device=self.device)
            return kt, kt.clone(), 0
        ti = torch.tensor([self._ring_slot_host(p) for p in idx], dtype=torch.long, device=self.device)
        return (self.k_hist.index_select(0, ti).unsqueeze(0).contiguous(),
                self.v_hist.index_select(0, ti).unsqueeze(0).contiguous(), len(idx))

    def decode_inputs(self) -> dict:
        """Argument bundle of the decode call at the current state; lengths stay on the device."""
        p = self.pool
        return {"planes": self.decode_planes_full(), "k_tail": p.k_tail[:1], "v_tail": p.v_tail[:1],
                "b_tail_len": p.b_tail[:1], "b_seq_len": p.b_seq[:1], "packed_start_offset": 0,
                "max_seq_len": max(1, self.window.packed_len(self.max_seq_len)),
                "max_tail_len": p.max_tail_len}


__all__ = ["CanonicalKVStore"]
