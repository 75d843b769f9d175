"""Single-request KV store for the decode hot path.

Mirror of ``CanonicalKVStore`` in the reference (``ommx_gpu_serve/attention/kv_store.py:93``) for
the ring-sized, bitmap / power-of-two serving recipe: the same method names a decode loop calls
(``append_block`` :429, ``append`` :349, ``reset_inplace`` :331, ``decode_planes_full`` :651,
``decode_inputs`` :696).  It is the one-request case of :class:`MultiSeqKVPool`: every step's ring
write, group completion test, quantize + pack and length bookkeeping run on the device in one
library call, so nothing here keeps a host copy of the sequence length."""
from __future__ import annotations

from typing import Optional

import torch

from .kv_pool import MultiSeqKVPool
from .kv_window import WindowSpec


class CanonicalKVStore:
    def __init__(self, head_dim: int, n_kv_heads: int, max_seq_len: int, *, k_format: str = "i2f4",
                 outliers_per_vector: int = 6, outlier_select: str = "signed", outlier_repr: str = "bitmap",
                 use_pow2: bool = True, kv_outlier_map: bool = True, kv_int8_scale: bool = True,
                 window: Optional[WindowSpec] = None, group_channels: int = 32, device="cuda") -> None:
        self.pool = MultiSeqKVPool(head_dim, n_kv_heads, 1, max_seq_len, k_format=k_format,
                                   outliers_per_vector=outliers_per_vector, outlier_select=outlier_select,
                                   outlier_repr=outlier_repr, use_pow2=use_pow2, kv_outlier_map=kv_outlier_map,
                                   kv_int8_scale=kv_int8_scale, window=window, group_channels=group_channels,
                                   device=device)
        p = self.pool
        self.D, self.H, self.k, self.ps, self.gt = p.D, p.H, p.k, p.ps, p.gt
        self.window, self.device, self.max_seq_len = p.window, p.device, p.max_seq_len
        self._fresh = True

    # ── write path ───────────────────────────────────────────────────────────
    def reset_inplace(self) -> None:
        """New sequence in the same tensors (addresses a captured graph holds stay valid)."""
        self.pool.seq_dev.zero_()
        self._fresh = True

    def append_block(self, K: torch.Tensor, V: torch.Tensor) -> None:
        """Prefill block ``[T, H, D]`` into a fresh store."""
        if not self._fresh:
            raise RuntimeError("append_block expects a fresh store (ring sizing cannot retain an unpacked "
                               "prefix); call reset_inplace() first")
        self.pool.append_block(0, K, V)
        self.pool.decode_inputs_device(1, refresh=True)
        self._fresh = False

    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """One decode step's K/V row ``[H, D]``: ring write, pack of a completed group, lengths."""
        kb = k.reshape(1, self.H, self.D).to(self.device, torch.bfloat16)
        vb = v.reshape(1, self.H, self.D).to(self.device, torch.bfloat16)
        self.pool.append_decode_device(kb, vb, 1)
        self._fresh = False

    # ── read path ────────────────────────────────────────────────────────────
    @property
    def seq_len(self) -> int:
        """Tokens held (copies one int from the device: for tests and logging)."""
        return int(self.pool.seq_dev[0].item())

    def decode_planes_full(self) -> dict:
        """Full-capacity, fixed-address planes and identity tables (what a captured graph binds)."""
        pl, p = self.pool.planes, self.pool
        return {"k_base": pl["k_base"], "k_scale": pl["k_scale"], "k_zp": pl["k_zp"], "k_oidx": None,
                "k_oval": pl["k_oval"], "k_crank": None, "k_obmp": pl["k_obmp"], "outlier_repr": "bitmap",
                "k_fp4_mapscale": pl["k_fp4_mapscale"], "k_fp4_mapcenter": pl["k_fp4_mapcenter"],
                "v_main": pl["v_main"], "v_scale": pl["v_scale"], "v_zp": pl["v_zp"],
                "req_to_token": p._req_to_token, "req_to_group": p._req_to_group,
                "page_size": self.ps, "outliers_per_vector": self.k, "k_format": "i2f4", "v_format": "int2",
                "head_dim": self.D, "n_kv_heads": self.H, "kv_outlier_map": bool(p.kv_outlier_map),
                "kv_int8_scale": True}

    def decode_inputs(self) -> dict:
        """Argument bundle of the decode call at the current state; lengths stay on the device."""
        p = self.pool
        return {"planes": self.decode_planes_full(), "k_tail": p.k_tail[:1], "v_tail": p.v_tail[:1],
                "b_tail_len": p.b_tail[:1], "b_seq_len": p.b_seq[:1], "packed_start_offset": 0,
                "max_seq_len": max(1, self.window.packed_len(self.max_seq_len)),
                "max_tail_len": p.max_tail_len}


__all__ = ["CanonicalKVStore"]
