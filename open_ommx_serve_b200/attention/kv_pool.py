"""Device-resident KV pool for batched paged decode: the store side of the decode hot path.

Mirror of ``MultiSeqKVPool`` in the reference (``ommx_gpu_serve/attention/kv_pool.py:93``): one
shared set of quantized planes, a small bf16 residual ring per request (attention sink rows
pinned, recent rows sliding), per-request page and group-slot tables, and every call the
reference's serving loops make on the class:

=============================================  ===============================================
reference method (kv_pool.py)                  here
=============================================  ===============================================
``append_block(req, K, V)`` :310               prefill: quantize the completed prefix straight
                                               from the input into the request's pages / slots
                                               (``ommx_pack_kv_into``), keep the live rows
``append(req, k, v)`` :370                     one row of one request
``append_decode_batched(slots, K, V)`` :383    one row per listed request slot
``append_decode_device(K, V, B)`` :440         one row per batch row, lengths on the device
``append_decode_captured(rows, cols, K, V)``   one row per batch row at caller-given device
:490                                           (slot, position) indices
``regroup(req)`` :637                          bookkeeping only (see below)
``pool_planes()`` :738, ``request_planes`` :776
``tail_bf16_batched(slots)`` :818
``decode_inputs_batched(slots)`` :938
``decode_inputs_captured(sel, ...)`` :886
``decode_seed_seq_device`` :1015, ``advance_seq_device`` :1037, ``decode_inputs_device`` :1048
=============================================  ===============================================

Every write call is ONE library call (``ommx_b200_kv_append_decode``): ring write of the new
row, quantize + pack of the 32-token group that the row completed (if any) straight from the
ring into the request's next pages and group slot, and the length bookkeeping, on the device,
with a fixed launch shape - where the reference writes the row, loops over requests on the
host to find completed groups and packs them in a second pass (:552-635,
``kv_store_ops.py:22-57``).  Because a completed group is packed by the write call itself,
``regroup`` has nothing left to pack: it only brings the host-side ``packed_groups`` count up to
date and returns how many groups that covered.

The device array ``seq_dev`` is the authoritative length per request; ``seq_len`` /
``packed_groups`` are the reference's host-side lists, kept in step by the host-driven calls
(the device-indexed calls leave them alone, as in the reference).  Residual history is ring
sized (the reference's ``OMMX_KV_RING=1`` layout); the full-history layout is not built.
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import torch

from .. import _lib
from .kv_window import WindowSpec
from .pack import alloc_planes, ommx_pack_kv_into, planes_struct

_CAPTURED_WRITE_CHECK = os.environ.get("OMMX_KV_CAPTURED_WRITE_CHECK", "1").strip().lower() not in {"0", "false", "off", "no"}


class MultiSeqKVPool:
    """Per-layer plane pool + residual rings + tables for ``num_seqs`` requests (ring sizing)."""

    def __init__(self, head_dim: int, n_kv_heads: int, num_seqs: int, max_seq_len: int, *,
                 k_format: str = "i2f4", outliers_per_vector: int = 6, outlier_select: str = "signed",
                 outlier_repr: str = "bitmap", use_pow2: bool = True, kv_outlier_map: Optional[bool] = True,
                 kv_int8_scale: Optional[bool] = True, window: Optional[WindowSpec] = None,
                 group_channels: int = 32, scale_dtype: torch.dtype = torch.bfloat16, device="cuda") -> None:
        if head_dim % 32 != 0:
            raise ValueError(f"head_dim must be a multiple of 32; got {head_dim}")
        if str(k_format).lower() not in ("i2f4", "itf4"):
            raise ValueError(f"k_format must be i2f4|itf4; got {k_format!r}")
        if str(k_format).lower() != "i2f4":
            raise NotImplementedError(f"k_format {k_format!r} is not served (i2f4)")
        if str(outlier_repr).lower() != "bitmap":
            raise NotImplementedError(f"outlier_repr {outlier_repr!r} is not served (bitmap)")
        if str(outlier_select).lower() != "signed":
            raise NotImplementedError("the device store serves outlier_select='signed'")
        kv_outlier_map = True if kv_outlier_map is None else bool(kv_outlier_map)
        kv_int8_scale = bool(use_pow2) if kv_int8_scale is None else bool(kv_int8_scale)
        if not (use_pow2 and kv_int8_scale):
            raise NotImplementedError("the device store serves power-of-two int8 scales")
        if scale_dtype != torch.bfloat16:
            raise NotImplementedError("zero-point / map planes are bfloat16")
        if int(group_channels) != 32:
            raise NotImplementedError("group_channels must be 32")
        if int(outliers_per_vector) not in (0, 2, 4, 6, 8):
            raise NotImplementedError("outliers_per_vector must be one of 0, 2, 4, 6, 8")
        self.window = window or WindowSpec()
        if int(self.window.group_tokens) != 32:
            raise NotImplementedError("group_tokens must be 32")
        self.D, self.H = int(head_dim), int(n_kv_heads)
        self.num_seqs, self.max_seq_len = int(num_seqs), int(max_seq_len)
        self.k = int(outliers_per_vector)
        self.k_format, self.outlier_select, self.outlier_repr = "i2f4", "signed", "bitmap"
        self.use_pow2, self.kv_int8_scale, self.scale_dtype = True, True, scale_dtype
        self.kv_outlier_map = bool(kv_outlier_map) and self.k > 0
        self.gt, self.gc, self.ps = 32, 32, int(self.window.page_size)
        self.k_base_bits, self.oval_bits = 2, 4
        if self.gt % self.ps != 0:
            raise ValueError(f"group_tokens (32) must be a multiple of page_size ({self.ps})")
        self.pages_per_group = self.gt // self.ps
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("MultiSeqKVPool needs a CUDA device (there is no CPU path)")
        # one spare group per request, as in the reference (a just-completed group never overruns)
        self.G_per_seq = max(1, (self.max_seq_len + self.gt - 1) // self.gt + 1)
        self.P_per_seq = self.G_per_seq * self.pages_per_group
        self.G_cap, self.P_cap = self.num_seqs * self.G_per_seq, self.num_seqs * self.P_per_seq
        self.planes = alloc_planes(self.P_cap, self.G_cap, self.H, self.D, page_size=self.ps,
                                   outliers_per_vector=self.k, kv_outlier_map=self.kv_outlier_map,
                                   device=self.device)
        self.sink, self.recent = int(self.window.sink_tokens), int(self.window.recent_window)
        self.kv_ring = True
        self._ring_sink, self._ring_rec = self.sink, self.recent + 2 * self.gt
        self.ring_cap = self.sink + self.recent + 2 * self.gt
        self.S_ring = self.ring_cap
        dev = self.device
        self.k_hist = torch.zeros(self.num_seqs, self.ring_cap, self.H, self.D, dtype=torch.bfloat16, device=dev)
        self.v_hist = torch.zeros_like(self.k_hist)
        self.seq_dev = torch.zeros(self.num_seqs, dtype=torch.int32, device=dev)
        self.seq_len = [0] * self.num_seqs          # host-side lengths (host-driven calls keep them in step)
        self.packed_groups = [0] * self.num_seqs
        self._req_to_group = torch.arange(self.G_cap, dtype=torch.int32, device=dev).reshape(self.num_seqs, self.G_per_seq)
        self._req_to_token = torch.arange(self.P_cap, dtype=torch.int32, device=dev).reshape(self.num_seqs, self.P_per_seq)
        self.max_tail_len = int(self.window.max_tail_len(self.max_seq_len))
        self.k_tail = torch.zeros(self.num_seqs, self.max_tail_len, self.H, self.D, dtype=torch.bfloat16, device=dev)
        self.v_tail = torch.zeros_like(self.k_tail)
        self.b_seq = torch.zeros(self.num_seqs, dtype=torch.int32, device=dev)
        self.b_tail = torch.zeros(self.num_seqs, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._sel = None                     # batch row -> request slot (None: row i is slot i)
        self._sel_key = None
        self._r2t_sel = self._r2g_sel = None
        self._planes_cache = None
        self._dbuf = None

    # plane tensors under the reference's attribute names
    k_base = property(lambda self: self.planes["k_base"])
    k_scale = property(lambda self: self.planes["k_scale"])
    k_zp = property(lambda self: self.planes["k_zp"])
    k_obmp = property(lambda self: self.planes.get("k_obmp"))
    k_oval = property(lambda self: self.planes.get("k_oval"))
    k_fp4_mapscale = property(lambda self: self.planes.get("k_fp4_mapscale"))
    k_fp4_mapcenter = property(lambda self: self.planes.get("k_fp4_mapcenter"))
    v_main = property(lambda self: self.planes["v_main"])
    v_scale = property(lambda self: self.planes["v_scale"])
    v_zp = property(lambda self: self.planes["v_zp"])
    k_oidx = k_crank = None

    def select_slots(self, slots=None) -> None:
        """Choose which request slots the batch rows of the following calls stand for (``None``: row i =
        slot i).  A host-side event (the batch changed), done outside the decode loop: the tables of the
        chosen slots are gathered once here so that the per-step calls allocate nothing."""
        if slots is None:
            self._sel = self._sel_key = self._r2t_sel = self._r2g_sel = None
            return
        idx = tuple(int(x) for x in slots)
        if idx == self._sel_key:
            return
        if len(set(idx)) != len(idx) or any(not 0 <= x < self.num_seqs for x in idx):
            raise ValueError(f"slots must be distinct and inside [0, {self.num_seqs}); got {list(idx)}")
        self._sel = torch.tensor(idx, dtype=torch.int32, device=self.device)
        self._sel_key = idx
        sel = self._sel.long()
        self._r2t_sel = self._req_to_token.index_select(0, sel).contiguous()
        self._r2g_sel = self._req_to_group.index_select(0, sel).contiguous()

    # ── helpers ──────────────────────────────────────────────────────────────
    def _ring_slot_host(self, pos: int) -> int:
        """Absolute token position -> ring row (reference :285-292)."""
        p = int(pos)
        return p if p < self._ring_sink else self._ring_sink + (p - self._ring_sink) % self._ring_rec

    def _ring_slot_dev(self, pos: torch.Tensor) -> torch.Tensor:
        """The same map on a device tensor, without a host sync (reference :294-306)."""
        return torch.where(pos < self._ring_sink, pos, (pos - self._ring_sink) % self._ring_rec + self._ring_sink)

    _ring_row = _ring_slot_dev

    def _pool_struct(self, a_pool) -> None:
        a_pool.planes = planes_struct(self.planes, k=self.k, outlier_map=self.kv_outlier_map)
        a_pool.k_hist, a_pool.v_hist = self.k_hist.data_ptr(), self.v_hist.data_ptr()
        a_pool.num_seqs, a_pool.ring_cap = self.num_seqs, self.ring_cap
        a_pool.sink_tokens, a_pool.recent_window = self.sink, self.recent
        a_pool.seq_len = self.seq_dev.data_ptr()
        a_pool.req_to_token, a_pool.req_to_group = self._req_to_token.data_ptr(), self._req_to_group.data_ptr()
        a_pool.pages_per_seq, a_pool.groups_per_seq = self.P_per_seq, self.G_per_seq

    def _append_args(self, B: int, advance, K=None, V=None, *, slots=None, write_pos=None, outputs=True) -> "_lib.KVAppendArgs":
        a = _lib.KVAppendArgs()
        self._pool_struct(a.pool)
        if K is not None:
            a.k_new, a.v_new = K.data_ptr(), V.data_ptr()
            a.new_stride_b, a.new_stride_h = int(K.stride(0)), int(K.stride(1))
        if slots is None and write_pos is None:
            a.slots = None if self._sel is None else self._sel.data_ptr()
            if self._sel is not None and int(B) != int(self._sel.numel()):
                raise ValueError(f"batch {B} does not match the {int(self._sel.numel())} selected slots")
        else:
            is64 = {torch.int64: 1, torch.int32: 0}
            dt = (slots if slots is not None else write_pos).dtype
            if dt not in is64 or (slots is not None and write_pos is not None and slots.dtype != write_pos.dtype):
                raise ValueError("slot / position index tensors must both be int32 or both int64")
            for t in (slots, write_pos):
                if t is not None and (not t.is_cuda or not t.is_contiguous() or int(t.numel()) != int(B)):
                    raise ValueError(f"slot / position index tensors must be contiguous CUDA tensors of {B} entries")
            a.slots = None if slots is None else slots.data_ptr()
            a.write_pos = None if write_pos is None else write_pos.data_ptr()
            a.index_is_int64 = is64[dt]
        a.batch, a.advance = int(B), int(advance)
        a.outlier_select, a.use_pow2 = 1, 1
        if outputs:
            a.k_tail, a.v_tail, a.max_tail = self.k_tail.data_ptr(), self.v_tail.data_ptr(), self.max_tail_len
            a.b_seq_len, a.b_tail_len = self.b_seq.data_ptr(), self.b_tail.data_ptr()
        a.status = self.status.data_ptr()
        return a

    def _call(self, a) -> None:
        lib = _lib.load()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.ommx_b200_kv_append_decode(a, stream), "ommx_b200_kv_append_decode")

    def _rows(self, K: torch.Tensor, V: torch.Tensor, B: int):
        K, V = K.reshape(B, self.H, self.D), V.reshape(B, self.H, self.D)
        if K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16 or K.device != self.device:
            K, V = K.to(self.device, torch.bfloat16), V.to(self.device, torch.bfloat16)
        if K.stride(-1) != 1 or V.stride() != K.stride():
            K, V = K.contiguous(), V.contiguous()
        return K, V

    def _host_step(self, slots) -> int:
        """Advance the host-side lengths of ``slots`` by one row each; groups that completed."""
        total = 0
        for r in slots:
            self.seq_len[r] += 1
            target = self.window.num_groups(self.seq_len[r])
            total += max(0, target - self.packed_groups[r])
            self.packed_groups[r] = max(self.packed_groups[r], target)
        return total

    # ── write path ───────────────────────────────────────────────────────────
    def append_block(self, req: int, K: torch.Tensor, V: torch.Tensor) -> int:
        """Prefill of a fresh request slot with bf16 ``K``/``V`` ``[T, H, D]``; returns groups packed."""
        r, T = int(req), int(K.shape[0])
        if not 0 <= r < self.num_seqs:
            raise IndexError(f"request slot {r} outside [0, {self.num_seqs})")
        if T > self.max_seq_len:
            raise RuntimeError(f"MultiSeqKVPool req {r} capacity {self.max_seq_len} exceeded")
        Kb, Vb = K.to(self.device, torch.bfloat16), V.to(self.device, torch.bfloat16)
        target = self.window.num_groups(T)
        if target > 0:
            t0, t1 = self.sink, self.sink + target * self.gt
            ommx_pack_kv_into(Kb[t0:t1], Vb[t0:t1], self.planes,
                              dst_pages=self._req_to_token[r, :target * self.pages_per_group].contiguous(),
                              dst_groups=self._req_to_group[r, :target].contiguous(),
                              outliers_per_vector=self.k, kv_outlier_map=self.kv_outlier_map,
                              status=self.status)
        boundary = self.window.boundary(T)
        lo = max(self.sink, boundary - self.gt)
        parts = [torch.arange(0, min(self.sink, T), device=self.device)]
        if lo < T:
            parts.append(torch.arange(lo, T, device=self.device))
        live = torch.cat(parts).to(torch.long)
        rows = self._ring_slot_dev(live)
        self.k_hist[r].index_copy_(0, rows, Kb.index_select(0, live))
        self.v_hist[r].index_copy_(0, rows, Vb.index_select(0, live))
        self.seq_dev[r] = T
        self.seq_len[r], self.packed_groups[r] = T, target
        return target

    def append(self, req: int, k: torch.Tensor, v: torch.Tensor) -> int:
        """One decode step's K/V row ``[H, D]`` of request ``req``; returns groups packed (0 or 1)."""
        return self.append_decode_batched([int(req)], k.reshape(1, self.H, self.D), v.reshape(1, self.H, self.D))

    def append_decode_batched(self, slots: Sequence[int], K: torch.Tensor, V: torch.Tensor) -> int:
        """One new row ``[B, H, D]`` for each request of ``slots``; returns the groups packed this step."""
        slots = [int(s) for s in slots]
        B = len(slots)
        if B == 0:
            return 0
        if any(not 0 <= r < self.num_seqs for r in slots):
            raise IndexError(f"request slots {slots} outside [0, {self.num_seqs})")
        identity = slots == list(range(B))
        prev = (self._sel, self._sel_key, self._r2t_sel, self._r2g_sel)
        if identity:
            self._sel = None
        else:
            self.select_slots(slots)
        try:
            Kb, Vb = self._rows(K, V, B)
            total = self._host_step(slots)
            self._call(self._append_args(B, 1, Kb, Vb))
        finally:
            if identity:
                self._sel, self._sel_key, self._r2t_sel, self._r2g_sel = prev
        return total

    def append_decode_device(self, K: torch.Tensor, V: torch.Tensor, B: int) -> int:
        """One decode step for rows ``0..B-1`` (row i = request slot i, or the slots chosen with
        ``select_slots``): ``K``/``V`` are ``[B, H, D]`` bf16.

        Ring write, quantize + pack of completed groups, length advance and the decode inputs of the
        step, on the device, without a host loop over tensors or a synchronisation (CUDA-graph
        capturable; a replayed graph advances the device lengths, not the host-side lists)."""
        if K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16 or not K.is_cuda:
            raise ValueError("K/V must be bf16 CUDA tensors [B, H, D]")
        if tuple(K.shape) != (int(B), self.H, self.D) or tuple(V.shape) != tuple(K.shape):
            raise ValueError(f"K/V must be [{B}, {self.H}, {self.D}]")
        if K.stride(-1) != 1 or V.stride() != K.stride():
            K, V = K.contiguous(), V.contiguous()
        total = 0
        if not torch.cuda.is_current_stream_capturing():
            total = self._host_step(range(int(B)) if self._sel_key is None else self._sel_key)
        self._call(self._append_args(B, 1, K, V))
        return total

    def append_decode_captured(self, rows: torch.Tensor, cols: torch.Tensor, K: torch.Tensor, V: torch.Tensor) -> None:
        """One new row per batch row at device-side indices: request slot ``rows[i]``, absolute
        position ``cols[i]`` (``[B]`` int64 or int32 buffers the host refreshes between replays).

        As in the reference the host-side ``seq_len`` / ``packed_groups`` and the device lengths are left
        to the caller (``advance_seq_device``); unlike it, a 32-token group that ``cols[i]`` completes is
        quantized and packed by this call itself, so no host regroup pass has to follow."""
        B = int(rows.shape[0])
        Kb, Vb = self._rows(K, V, B)
        if _CAPTURED_WRITE_CHECK and not torch.cuda.is_current_stream_capturing():
            self._check_captured_indices(rows, cols)
        self._call(self._append_args(B, 2, Kb, Vb, slots=rows.contiguous(), write_pos=cols.contiguous(), outputs=False))

    def _check_captured_indices(self, rows: torch.Tensor, cols: torch.Tensor) -> None:
        """Refuse an out-of-range device-indexed write with the offending value named (reference :526-550)."""
        rmin, rmax, cmin, cmax = int(rows.min()), int(rows.max()), int(cols.min()), int(cols.max())
        if not (0 <= rmin and rmax < self.num_seqs):
            raise IndexError(f"OMMX captured KV write: pool slot index out of range - rows span [{rmin}, {rmax}] "
                             f"but the pool holds {self.num_seqs} slots.")
        if not (0 <= cmin and cmax < self.max_seq_len + self.gt):
            raise IndexError(f"OMMX captured KV write: write column out of range - cols span [{cmin}, {cmax}] but a "
                             f"request holds at most max_seq_len={self.max_seq_len} tokens (cols is the absolute position).")

    def regroup(self, req: int) -> int:
        """Groups of request ``req`` that completed since the last count.  The write calls have already
        packed them on the device; this only brings ``packed_groups`` up to date (reference :637-652)."""
        r = int(req)
        target = self.window.num_groups(self.seq_len[r])
        n = max(0, target - self.packed_groups[r])
        self.packed_groups[r] = max(self.packed_groups[r], target)
        return n

    # ── read path ────────────────────────────────────────────────────────────
    def pool_planes(self) -> dict:
        """Whole-pool plane dict + the batched tables (fixed addresses; built once; reference :738-774)."""
        if self._planes_cache is None:
            p = self.planes
            self._planes_cache = {
                "k_base": p["k_base"], "k_scale": p["k_scale"], "k_zp": p["k_zp"], "k_oidx": None,
                "k_oval": p.get("k_oval"), "k_crank": None, "k_obmp": p.get("k_obmp"),
                "k_fp4_mapscale": p.get("k_fp4_mapscale"), "k_fp4_mapcenter": p.get("k_fp4_mapcenter"),
                "v_main": p["v_main"], "v_scale": p["v_scale"], "v_zp": p["v_zp"],
                "req_to_token": self._req_to_token, "req_to_group": self._req_to_group,
                "page_size": self.ps, "outliers_per_vector": self.k, "outlier_repr": self.outlier_repr,
                "outlier_select": self.outlier_select, "k_format": self.k_format, "head_dim": self.D,
                "n_kv_heads": self.H, "group_tokens": self.gt, "group_channels": self.gc,
                "k_base_bits": self.k_base_bits, "oval_bits": self.oval_bits,
                "kv_outlier_map": bool(self.kv_outlier_map), "kv_int8_scale": True}
        return self._planes_cache

    def request_planes(self, req: int) -> dict:
        """Contiguous planes of one request (its live pages / group slots gathered through the tables), in the
        layout a single-sequence dequantizer reads (reference :776-816)."""
        r = int(req)
        G = self.packed_groups[r]
        P = G * self.pages_per_group
        gidx = self._req_to_group[r, :G].to(torch.long)
        pidx = self._req_to_token[r, :P].to(torch.long)
        p = self.planes

        def take(name, idx):
            t = p.get(name)
            return None if t is None else t.index_select(0, idx)

        return {"k_base": take("k_base", pidx), "k_scale": take("k_scale", gidx), "k_zp": take("k_zp", gidx),
                "k_oidx": None, "k_oval": take("k_oval", gidx), "k_crank": None, "k_obmp": take("k_obmp", gidx),
                "k_fp4_mapscale": take("k_fp4_mapscale", gidx), "k_fp4_mapcenter": take("k_fp4_mapcenter", gidx),
                "v_main": take("v_main", pidx), "v_scale": take("v_scale", pidx), "v_zp": take("v_zp", pidx),
                "head_dim": self.D, "n_kv_heads": self.H, "num_tokens": G * self.gt, "n_groups": G,
                "page_size": self.ps, "outliers_per_vector": self.k, "outlier_repr": self.outlier_repr,
                "outlier_select": self.outlier_select, "group_tokens": self.gt, "group_channels": self.gc,
                "k_format": self.k_format, "k_base_bits": self.k_base_bits, "oval_bits": self.oval_bits,
                "kv_outlier_map": bool(self.kv_outlier_map), "kv_int8_scale": True}

    def _gather_tail(self, sel, tidx, kt, vt) -> None:
        lib = _lib.load()
        pool = _lib.KVPool()
        self._pool_struct(pool)
        B, T = int(tidx.shape[0]), int(tidx.shape[1])
        if tidx.dtype not in (torch.int32, torch.int64) or (sel is not None and sel.dtype != tidx.dtype):
            raise ValueError("sel / tail index tensors must both be int32 or both int64")
        if tuple(kt.shape) != (B, T, self.H, self.D) or not kt.is_contiguous() or not vt.is_contiguous() or tuple(vt.shape) != tuple(kt.shape):
            raise ValueError(f"k_tail / v_tail must be contiguous [{B}, {T}, {self.H}, {self.D}]")
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.ommx_b200_kv_gather_tail(pool, None if sel is None else sel.contiguous().data_ptr(),
                                                    tidx.contiguous().data_ptr(), 1 if tidx.dtype == torch.int64 else 0,
                                                    B, T, kt.data_ptr(), vt.data_ptr(), self.status.data_ptr(), stream),
                       "ommx_b200_kv_gather_tail")

    def tail_bf16_batched(self, slots: Sequence[int]):
        """``(k_tail [B,T,H,D], v_tail, b_tail_len [B])`` of the listed requests: sink and recent rows, zero
        padded to ``max_tail_len`` (reference :818-842)."""
        slots = [int(s) for s in slots]
        B, T = len(slots), self.max_tail_len
        idx = torch.zeros(B, T, dtype=torch.int64)
        n = torch.zeros(B, dtype=torch.int32)
        for b, r in enumerate(slots):
            ti = self.window.tail_indices(self.seq_len[r])[:T]
            idx[b, :len(ti)] = torch.tensor(ti, dtype=torch.int64)
            n[b] = len(ti)
        kt = torch.zeros(B, T, self.H, self.D, dtype=torch.bfloat16, device=self.device)
        vt = torch.zeros_like(kt)
        self._gather_tail(torch.tensor(slots, dtype=torch.int64, device=self.device), idx.to(self.device), kt, vt)
        valid = (torch.arange(T).view(1, T) < n.view(B, 1)).to(self.device)
        kt.mul_(valid.view(B, T, 1, 1))
        vt.mul_(valid.view(B, T, 1, 1))
        return kt, vt, n.to(self.device)

    def _ensure_decode_buffers(self, B: int) -> None:
        """Fixed-address buffers of the batched decode calls, allocated once (reference :844-884)."""
        if self._dbuf is not None and self._dbuf["cap"] >= B:
            return
        cap, T, dev = max(B, self.num_seqs), self.max_tail_len, self.device
        self._dbuf = {"cap": cap,
                      "kt": torch.zeros(cap, T, self.H, self.D, dtype=torch.bfloat16, device=dev),
                      "vt": torch.zeros(cap, T, self.H, self.D, dtype=torch.bfloat16, device=dev),
                      "b_tail": torch.zeros(cap, dtype=torch.int32, device=dev),
                      "b_seq": torch.zeros(cap, dtype=torch.int32, device=dev),
                      "sel": torch.zeros(cap, dtype=torch.long, device=dev),
                      "tidx_dev": torch.zeros(cap, T, dtype=torch.long, device=dev),
                      "seq_dev": torch.zeros(cap, dtype=torch.long, device=dev),
                      "rows": torch.zeros(cap, dtype=torch.long, device=dev),
                      "cols": torch.zeros(cap, dtype=torch.long, device=dev)}

    def _bundle(self, r2t, r2g, kt, vt, b_tail, b_seq, max_seq_len) -> dict:
        """The reference's argument bundle (:925-936), with the plane entries repeated at the top level."""
        planes = dict(self.pool_planes())
        planes["req_to_token"], planes["req_to_group"] = r2t, r2g
        out = {"planes": planes, "k_tail": kt, "v_tail": vt, "b_tail_len": b_tail, "b_seq_len": b_seq,
               "req_to_token": r2t, "req_to_group": r2g, "packed_start_offset": 0,
               "max_seq_len": int(max_seq_len), "max_tail_len": self.max_tail_len}
        for name in ("k_base", "k_scale", "k_zp", "k_oidx", "k_oval", "k_obmp", "k_fp4_mapscale", "k_fp4_mapcenter",
                     "v_main", "v_scale", "v_zp", "page_size", "kv_outlier_map"):
            out[name] = planes[name]
        out["k_outliers_per_vector"] = self.k
        return out

    def decode_inputs_captured(self, sel: torch.Tensor, b_seq_len: torch.Tensor, b_tail_len: torch.Tensor,
                               tidx_dev: torch.Tensor, kt: torch.Tensor, vt: torch.Tensor, max_seq_len: int) -> dict:
        """Argument bundle from caller-owned fixed-address control tensors: ``sel`` ``[B]`` batch row -> pool
        slot, packed and residual lengths, ``tidx_dev`` ``[B, T]`` absolute residual token positions, and the
        residual output buffers ``kt`` / ``vt``, which one gather launch fills (reference :886-936)."""
        self._gather_tail(sel, tidx_dev, kt, vt)
        sel_l = sel.to(torch.long)
        return self._bundle(self._req_to_token.index_select(0, sel_l), self._req_to_group.index_select(0, sel_l),
                            kt, vt, b_tail_len, b_seq_len, max_seq_len)

    def decode_inputs_batched(self, slots: Sequence[int]) -> dict:
        """Argument bundle for the listed requests at their current lengths (reference :938-1011): lengths and
        residual rows are rebuilt on the device from the device lengths; ``max_seq_len`` comes from the
        host-side group counts, so nothing synchronises."""
        slots = [int(s) for s in slots]
        B = len(slots)
        identity = slots == list(range(B))
        if identity:
            self.select_slots(None)
        else:
            self.select_slots(slots)
        self._call(self._append_args(B, 0))
        max_seq = max(1, max([self.packed_groups[r] for r in slots] + [0]) * self.gt)
        return self._bundle(self._req_to_token[:B] if identity else self._r2t_sel,
                            self._req_to_group[:B] if identity else self._r2g_sel,
                            self.k_tail[:B], self.v_tail[:B], self.b_tail[:B], self.b_seq[:B], max_seq)

    def decode_seed_seq_device(self, slots: Sequence[int]) -> torch.Tensor:
        """Start of a device-driven decode loop over ``slots`` (reference :1015-1035): binds the batch rows to
        the slots, makes the device lengths equal the host-side ones and returns them (``[B]`` int64)."""
        slots = [int(s) for s in slots]
        B = len(slots)
        self._ensure_decode_buffers(B)
        self.select_slots(None if slots == list(range(B)) else slots)
        seed = torch.tensor([self.seq_len[r] for r in slots], dtype=torch.int32)
        idx = torch.tensor(slots, dtype=torch.long, device=self.device)
        self.seq_dev.index_copy_(0, idx, seed.to(self.device))
        d = self._dbuf
        d["rows"][:B].copy_(idx)
        d["sel"][:B].copy_(idx)
        d["seq_dev"][:B].copy_(seed.to(self.device, torch.long))
        return d["seq_dev"][:B]

    def advance_seq_device(self, B: int) -> None:
        """Advance the device lengths of the batch rows by one (reference :1037-1046); for callers that wrote
        with ``append_decode_captured``, which leaves the lengths alone."""
        if self._sel is None:
            self.seq_dev[:B].add_(1)
        else:
            self.seq_dev.index_add_(0, self._sel.long(), torch.ones(B, dtype=torch.int32, device=self.device))
        if self._dbuf is not None:
            self._dbuf["seq_dev"][:B].add_(1)
            self._dbuf["cols"][:B].copy_(self._dbuf["seq_dev"][:B] - 1)

    def decode_inputs_device(self, B: int, max_seq_len: Optional[int] = None, *, refresh: bool = False) -> dict:
        """Arguments of the decode call for rows ``0..B-1`` (reference :1048-1105); ``refresh`` recomputes
        lengths and residual rows from the current device state (needed once after prefill, before the first
        decode step - ``append_decode_device`` leaves them up to date)."""
        if refresh:
            self._call(self._append_args(B, 0))
        return self._bundle(self._req_to_token[:B] if self._sel is None else self._r2t_sel,
                            self._req_to_group[:B] if self._sel is None else self._r2g_sel,
                            self.k_tail[:B], self.v_tail[:B], self.b_tail[:B], self.b_seq[:B],
                            max_seq_len if max_seq_len is not None else self.window.packed_len(self.max_seq_len))

    def seq_lens(self):
        """Host copy of the device sequence lengths (synchronises; tests and logging only)."""
        return self.seq_dev.cpu().tolist()


__all__ = ["MultiSeqKVPool"]
