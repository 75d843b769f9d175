"""Device-resident KV pool for batched paged decode: the store side of the decode hot path.

Mirror of the decode-serving part of ``MultiSeqKVPool`` in the reference
(``ommx_gpu_serve/attention/kv_pool.py:93``): one shared set of quantized planes, a small bf16
residual ring per request (attention sink rows pinned, recent rows sliding), per-request page and
group-slot tables, and the three calls a serving loop makes:

``append_block(req, K, V)``
    prefill: quantize the completed prefix straight from the input into the request's pages and
    group slots (``ommx_pack_kv_into``) and keep only the live residual rows in the ring
    (reference ``append_block`` :310-372).
``append_decode_device(K, V, B)``
    one decode step for rows ``0..B-1``: ring write, quantize + pack of the 32-token group the step
    completed (if any), sequence length advance and the step's decode inputs, all on the device in
    one library call (``ommx_b200_kv_append_decode``) - the reference does the write with
    ``_kv_write_token``, loops over requests on the host to find completed groups and packs them
    in a second pass (:440-488, ``kv_store_ops.py:22-57``).
``decode_inputs_device(B, max_seq_len)``
    the argument bundle of ``ommx_paged_decode_attention_canonical`` for the current lengths
    (reference :1048-1105).  After ``append_decode_device`` it is already up to date.

There is no host mirror of the sequence lengths in the decode loop and no host synchronisation;
``seq_lens()`` copies the device lengths back for tests and logging only.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib
from .kv_window import WindowSpec
from .pack import alloc_planes, ommx_pack_kv_into, planes_struct


class MultiSeqKVPool:
    """Per-layer plane pool + residual rings + tables for ``num_seqs`` requests (ring sizing)."""

    def __init__(self, head_dim: int, n_kv_heads: int, num_seqs: int, max_seq_len: int, *,
                 k_format: str = "i2f4", outliers_per_vector: int = 6, outlier_select: str = "signed",
                 outlier_repr: str = "bitmap", use_pow2: bool = True, kv_outlier_map: bool = True,
                 kv_int8_scale: bool = True, window: Optional[WindowSpec] = None,
                 group_channels: int = 32, device="cuda") -> None:
        if head_dim % 32 != 0:
            raise ValueError(f"head_dim must be a multiple of 32; got {head_dim}")
        if str(k_format).lower() != "i2f4":
            raise NotImplementedError(f"k_format {k_format!r} is not served (i2f4)")
        if str(outlier_repr).lower() != "bitmap":
            raise NotImplementedError(f"outlier_repr {outlier_repr!r} is not served (bitmap)")
        if str(outlier_select).lower() != "signed":
            raise NotImplementedError("the device store serves outlier_select='signed'")
        if not (use_pow2 and kv_int8_scale):
            raise NotImplementedError("the device store serves power-of-two int8 scales")
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
        self.kv_outlier_map = bool(kv_outlier_map) and self.k > 0
        self.gt, self.ps = 32, int(self.window.page_size)
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
        self.ring_cap = self.sink + self.recent + 2 * self.gt
        dev = self.device
        self.k_hist = torch.zeros(self.num_seqs, self.ring_cap, self.H, self.D, dtype=torch.bfloat16, device=dev)
        self.v_hist = torch.zeros_like(self.k_hist)
        self.seq_dev = torch.zeros(self.num_seqs, dtype=torch.int32, device=dev)
        self._req_to_group = torch.arange(self.G_cap, dtype=torch.int32, device=dev).reshape(self.num_seqs, self.G_per_seq)
        self._req_to_token = torch.arange(self.P_cap, dtype=torch.int32, device=dev).reshape(self.num_seqs, self.P_per_seq)
        self.max_tail_len = int(self.window.max_tail_len(self.max_seq_len))
        self.k_tail = torch.zeros(self.num_seqs, self.max_tail_len, self.H, self.D, dtype=torch.bfloat16, device=dev)
        self.v_tail = torch.zeros_like(self.k_tail)
        self.b_seq = torch.zeros(self.num_seqs, dtype=torch.int32, device=dev)
        self.b_tail = torch.zeros(self.num_seqs, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._sel = None                     # batch row -> request slot (None: row i is slot i)
        self._r2t_sel = self._r2g_sel = None

    def select_slots(self, slots=None) -> None:
        """Choose which request slots the batch rows of the following calls stand for (``None``: row i =
        slot i).  A host-side event (the batch changed), done outside the decode loop: the tables of the
        chosen slots are gathered once here so that the per-step calls allocate nothing."""
        if slots is None:
            self._sel = self._r2t_sel = self._r2g_sel = None
            return
        idx = [int(x) for x in slots]
        if len(set(idx)) != len(idx) or any(not 0 <= x < self.num_seqs for x in idx):
            raise ValueError(f"slots must be distinct and inside [0, {self.num_seqs}); got {idx}")
        self._sel = torch.tensor(idx, dtype=torch.int32, device=self.device)
        sel = self._sel.long()
        self._r2t_sel = self._req_to_token.index_select(0, sel).contiguous()
        self._r2g_sel = self._req_to_group.index_select(0, sel).contiguous()

    # ── helpers ──────────────────────────────────────────────────────────────
    def _ring_row(self, pos: torch.Tensor) -> torch.Tensor:
        rec = self.ring_cap - self.sink
        return torch.where(pos < self.sink, pos, self.sink + (pos - self.sink) % rec)

    def _append_args(self, B: int, advance: bool, K=None, V=None) -> "_lib.KVAppendArgs":
        a = _lib.KVAppendArgs()
        a.pool.planes = planes_struct(self.planes, k=self.k, outlier_map=self.kv_outlier_map)
        a.pool.k_hist, a.pool.v_hist = self.k_hist.data_ptr(), self.v_hist.data_ptr()
        a.pool.num_seqs, a.pool.ring_cap = self.num_seqs, self.ring_cap
        a.pool.sink_tokens, a.pool.recent_window = self.sink, self.recent
        a.pool.seq_len = self.seq_dev.data_ptr()
        a.pool.req_to_token, a.pool.req_to_group = self._req_to_token.data_ptr(), self._req_to_group.data_ptr()
        a.pool.pages_per_seq, a.pool.groups_per_seq = self.P_per_seq, self.G_per_seq
        if K is not None:
            a.k_new, a.v_new = K.data_ptr(), V.data_ptr()
            a.new_stride_b, a.new_stride_h = int(K.stride(0)), int(K.stride(1))
        a.slots = None if self._sel is None else self._sel.data_ptr()
        if self._sel is not None and int(B) != int(self._sel.numel()):
            raise ValueError(f"batch {B} does not match the {int(self._sel.numel())} selected slots")
        a.batch, a.advance = int(B), 1 if advance else 0
        a.outlier_select, a.use_pow2 = 1, 1
        a.k_tail, a.v_tail, a.max_tail = self.k_tail.data_ptr(), self.v_tail.data_ptr(), self.max_tail_len
        a.b_seq_len, a.b_tail_len = self.b_seq.data_ptr(), self.b_tail.data_ptr()
        a.status = self.status.data_ptr()
        return a

    def _call(self, a) -> None:
        lib = _lib.load()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(lib.ommx_b200_kv_append_decode(a, stream), "ommx_b200_kv_append_decode")

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
        rows = self._ring_row(live)
        self.k_hist[r].index_copy_(0, rows, Kb.index_select(0, live))
        self.v_hist[r].index_copy_(0, rows, Vb.index_select(0, live))
        self.seq_dev[r] = T
        return target

    def append_decode_device(self, K: torch.Tensor, V: torch.Tensor, B: int) -> None:
        """One decode step for rows ``0..B-1`` (row i = request slot i, or the slots chosen with
        ``select_slots``): ``K``/``V`` are ``[B, H, D]`` bf16.

        Ring write, quantize + pack of completed groups, length advance and the decode inputs of the
        step, on the device, without a host loop or synchronisation (CUDA-graph capturable)."""
        if K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16 or not K.is_cuda:
            raise ValueError("K/V must be bf16 CUDA tensors [B, H, D]")
        if tuple(K.shape) != (int(B), self.H, self.D) or tuple(V.shape) != tuple(K.shape):
            raise ValueError(f"K/V must be [{B}, {self.H}, {self.D}]")
        if K.stride(-1) != 1 or V.stride() != K.stride():
            K, V = K.contiguous(), V.contiguous()
        self._call(self._append_args(B, True, K, V))

    # ── read path ────────────────────────────────────────────────────────────
    def decode_inputs_device(self, B: int, max_seq_len: Optional[int] = None, *, refresh: bool = False) -> dict:
        """Arguments of the decode call for rows ``0..B-1``; ``refresh`` recomputes lengths and residual
        rows from the current device state (needed once after prefill, before the first decode step)."""
        if refresh:
            self._call(self._append_args(B, False))
        p = self.planes
        return dict(k_base=p["k_base"], k_scale=p["k_scale"], k_zp=p["k_zp"], k_oidx=None, k_oval=p["k_oval"],
                    v_main=p["v_main"], v_scale=p["v_scale"], v_zp=p["v_zp"],
                    k_tail=self.k_tail[:B], v_tail=self.v_tail[:B], b_tail_len=self.b_tail[:B],
                    req_to_token=self._req_to_token[:B] if self._sel is None else self._r2t_sel,
                    req_to_group=self._req_to_group[:B] if self._sel is None else self._r2g_sel, b_seq_len=self.b_seq[:B],
                    k_obmp=p["k_obmp"], k_fp4_mapscale=p["k_fp4_mapscale"], k_fp4_mapcenter=p["k_fp4_mapcenter"],
                    max_seq_len=int(max_seq_len if max_seq_len is not None else self.window.packed_len(self.max_seq_len)),
                    max_tail_len=self.max_tail_len, page_size=self.ps, k_outliers_per_vector=self.k,
                    kv_outlier_map=self.kv_outlier_map)

    def seq_lens(self):
        """Host copy of the device sequence lengths (synchronises; tests and logging only)."""
        return self.seq_dev.cpu().tolist()


__all__ = ["MultiSeqKVPool"]
