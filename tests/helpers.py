"""Shared builders for the parity tests: seeded inputs, pooled planes, oracle answers."""
from __future__ import annotations

import os

import numpy as np
import torch

from oracle import ommx_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
PLANES = ("k_base", "k_scale", "k_zp", "k_obmp", "k_oval", "k_fp4_mapscale", "k_fp4_mapcenter",
          "v_main", "v_scale", "v_zp")
#: oracle plane name -> key in the package's plane dict
BF16_PLANES = ("k_zp", "k_fp4_mapscale", "k_fp4_mapcenter", "v_zp")


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def gaussian_kv(seed, T, H, D, mag=12.0, bf16=True):
    """N(0,1) K/V, 4 K channels per head scaled by ``mag`` (same draw order as the fixtures)."""
    g = torch.Generator().manual_seed(seed)
    K = torch.randn(T, H, D, generator=g)
    V = torch.randn(T, H, D, generator=g)
    for h in range(H):
        idx = torch.randperm(D, generator=torch.Generator().manual_seed(seed + 1 + h))[:4]
        K[:, h, idx] *= mag
    if bf16:
        K, V = K.bfloat16().float(), V.bfloat16().float()
    return K, V


def plane_to_torch(name, arr, device):
    """numpy plane from the oracle (bf16 as uint16 bits) -> torch tensor in the package's dtype."""
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if arr.dtype == np.uint16:
        t = t.view(torch.bfloat16)
    return t.to(device)


def plane_to_numpy(t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def assert_planes_equal(got: dict, want: dict, ctx=""):
    """Bit-exact comparison of every plane present in ``want`` (numpy, bf16 as uint16)."""
    for name in PLANES:
        if name not in want or want[name] is None:
            assert got.get(name) is None, f"{ctx}{name}: unexpected plane"
            continue
        g = plane_to_numpy(got[name]) if isinstance(got[name], torch.Tensor) else got[name]
        w = want[name]
        assert g.shape == w.shape, f"{ctx}{name}: shape {g.shape} vs {w.shape}"
        if g.dtype != w.dtype:
            g = g.view(w.dtype) if g.dtype.itemsize == w.dtype.itemsize else g.astype(w.dtype)
        bad = int((g != w).sum())
        assert bad == 0, f"{ctx}{name}: {bad} of {w.size} elements differ"


class Case:
    """A batch of sequences with pooled, optionally permuted, quantized planes + bf16 residual rows."""

    def __init__(self, seq_lens, H=8, Hq=32, D=128, seed=42, k=6, page_size=16, permute=True,
                 sink=8, recent=32, outlier_map=True, mag=12.0, spare_pages=3, device="cuda",
                 tables_dtype=torch.int32):
        self.seq_lens, self.H, self.Hq, self.D, self.k, self.ps = list(seq_lens), H, Hq, D, k, page_size
        self.sm_scale = D ** -0.5
        B = len(seq_lens)
        self.q = torch.randn(B, Hq, D, generator=torch.Generator().manual_seed(seed + 7)).bfloat16()
        self.per_seq = []
        packed = [max(0, O.packed_boundary(s, sink, recent) - sink) for s in seq_lens]
        tails = [s - p for s, p in zip(seq_lens, packed)]
        n_pages = [p // page_size for p in packed]
        n_groups = [p // 32 for p in packed]
        # pooled planes keep pages*page_size == group_slots*32 (the launcher derives the group size from it)
        tot_groups = sum(n_groups) + spare_pages
        tot_pages = tot_groups * (32 // page_size)
        if permute:
            pperm = torch.randperm(tot_pages, generator=torch.Generator().manual_seed(4242)).numpy()
            gperm = torch.randperm(tot_groups, generator=torch.Generator().manual_seed(4243)).numpy()
        else:
            pperm, gperm = np.arange(tot_pages), np.arange(tot_groups)
        max_pages, max_groups = max(n_pages + [1]), max(n_groups + [1])
        r2t = np.zeros((B, max_pages + 2), dtype=np.int64)
        r2g = np.zeros((B, max_groups + 2), dtype=np.int64)
        max_tail = max(tails + [1])
        k_tail = torch.zeros(B, max_tail, H, D, dtype=torch.bfloat16)
        v_tail = torch.zeros(B, max_tail, H, D, dtype=torch.bfloat16)
        pooled = None
        po = go = 0
        for b, s in enumerate(seq_lens):
            K, V = gaussian_kv(seed + 1000 * b, s, H, D, mag=mag)
            edge = sink + packed[b] if packed[b] else min(sink, s)
            tail_idx = list(range(min(sink, s))) + list(range(edge, s)) if packed[b] else list(range(s))
            k_tail[b, :len(tail_idx)] = K[tail_idx].bfloat16()
            v_tail[b, :len(tail_idx)] = V[tail_idx].bfloat16()
            rec = {"K": K, "V": V, "tail_idx": tail_idx, "packed": packed[b], "planes": None}
            if packed[b]:
                pl = O.pack_kv(K[sink:edge].numpy(), V[sink:edge].numpy(), outliers_per_vector=k,
                               kv_outlier_map=outlier_map, page_size=page_size)
                rec["planes"] = pl
                if pooled is None:
                    pooled = {}
                    for name in PLANES:
                        if name in pl:
                            lead = tot_pages if name in ("k_base", "v_main", "v_scale", "v_zp") else tot_groups
                            pooled[name] = np.zeros((lead,) + pl[name].shape[1:], dtype=pl[name].dtype)
                pp = pperm[po:po + n_pages[b]]
                gp = gperm[go:go + n_groups[b]]
                for name in PLANES:
                    if name in pl:
                        pooled[name][pp if name in ("k_base", "v_main", "v_scale", "v_zp") else gp] = pl[name]
                r2t[b, :n_pages[b]] = pp
                r2g[b, :n_groups[b]] = gp
                po += n_pages[b]
                go += n_groups[b]
            self.per_seq.append(rec)
        self.packed, self.tails = packed, tails
        dev = torch.device(device)
        self.device = dev
        if pooled is None:   # nothing quantized anywhere: empty planes
            pooled = {"k_base": np.zeros((0, page_size, H, D // 4), np.uint8), "v_main": np.zeros((0, page_size, H, D // 4), np.uint8),
                      "v_scale": np.zeros((0, page_size, H, D // 32), np.int8), "v_zp": np.zeros((0, page_size, H, D // 32), np.uint16),
                      "k_scale": np.zeros((0, H, D), np.int8), "k_zp": np.zeros((0, H, D), np.uint16)}
            if k > 0:
                pooled.update(k_obmp=np.zeros((0, H, D, 4), np.uint8), k_oval=np.zeros((0, H, D, (k + 1) // 2), np.uint8),
                              k_fp4_mapscale=np.zeros((0, H, D), np.uint16), k_fp4_mapcenter=np.zeros((0, H, D), np.uint16))
        self.pooled_np = pooled
        self.planes = {n: plane_to_torch(n, a, dev) for n, a in pooled.items()}
        self.req_to_token = torch.from_numpy(r2t).to(tables_dtype).to(dev)
        self.req_to_group = torch.from_numpy(r2g).to(tables_dtype).to(dev)
        self.b_seq_len = torch.tensor(packed, dtype=torch.int32, device=dev)
        self.b_tail_len = torch.tensor(tails, dtype=torch.int32, device=dev)
        self.k_tail, self.v_tail = k_tail.to(dev), v_tail.to(dev)
        self.q_dev = self.q.to(dev)
        self.outlier_map = outlier_map and k > 0

    def run(self, num_kv_splits=None, o_dtype=torch.float32, status=None, attn_logits=None, **kw):
        from open_ommx_serve_b200.attention.paged_decode import ommx_paged_decode_attention_canonical
        B = len(self.seq_lens)
        o = torch.full((B, self.Hq, self.D), float("nan"), dtype=o_dtype, device=self.device)
        lse = torch.full((B, self.Hq), float("nan"), dtype=torch.float32, device=self.device)
        p = self.planes
        ommx_paged_decode_attention_canonical(
            self.q_dev, p["k_base"], p["k_scale"], p["k_zp"], None, p.get("k_oval"),
            p["v_main"], p["v_scale"], p["v_zp"], self.k_tail, self.v_tail, self.b_tail_len,
            o, lse, self.req_to_token, self.req_to_group, self.b_seq_len,
            sm_scale=self.sm_scale, page_size=self.ps, k_outliers_per_vector=self.k,
            bitmap_read=self.k > 0, k_obmp=p.get("k_obmp"),
            k_fp4_mapscale=p.get("k_fp4_mapscale"), k_fp4_mapcenter=p.get("k_fp4_mapcenter"),
            kv_outlier_map=self.outlier_map, kv_int8_scale=True, num_kv_splits=num_kv_splits,
            max_seq_len=kw.pop("max_seq_len", max(self.packed + [0]) if kw.pop("pass_max", True) else None),
            max_tail_len=kw.pop("max_tail_len", max(self.tails + [0]) if kw.pop("pass_max_tail", True) else None),
            attn_logits=attn_logits, status=status, **kw)
        torch.cuda.synchronize()
        return o, lse

    def oracle_kernel_arith(self, num_kv_splits=1, split_pv=False):
        """The reference kernel's arithmetic (bf16 rounding points, split + merge) restated on CPU."""
        B = len(self.seq_lens)
        o = np.zeros((B, self.Hq, self.D), dtype=np.float32)
        lse = np.zeros((B, self.Hq), dtype=np.float32)
        empty = np.zeros((0, self.H, self.D), dtype=np.float32)
        for b, rec in enumerate(self.per_seq):
            Kt = rec["K"][rec["tail_idx"]].numpy()
            Vt = rec["V"][rec["tail_idx"]].numpy()
            q = self.q[b].float().numpy()
            if rec["planes"] is not None:
                o[b], lse[b], _ = O.decode_split_kv(q, rec["planes"], Kt, Vt, self.sm_scale, num_kv_splits,
                                                    split_pv=split_pv)
            else:
                o[b], lse[b] = O.attention_fp32(q, Kt, Vt, self.sm_scale)
        return o, lse

    def oracle(self):
        """fp64 attention over (dequantized planes + bf16 residual rows), per sequence."""
        B = len(self.seq_lens)
        o = np.zeros((B, self.Hq, self.D), dtype=np.float32)
        lse = np.zeros((B, self.Hq), dtype=np.float32)
        for b, rec in enumerate(self.per_seq):
            Kt = rec["K"][rec["tail_idx"]].numpy()
            Vt = rec["V"][rec["tail_idx"]].numpy()
            if rec["planes"] is not None:
                Kd, Vd = O.dequant_kv(rec["planes"])
                Kt, Vt = np.concatenate([Kd, Kt]), np.concatenate([Vd, Vt])
            o[b], lse[b] = O.attention_fp32(self.q[b].float().numpy(), Kt, Vt, self.sm_scale)
        return o, lse


def check_close(got, want, *, cos_min=0.9999, max_abs=2e-2, rel_l2_max=None, ctx=""):
    """The attention gate of the path: max-abs <= 2e-2 and cosine >= 0.9999 against the
    reference kernel's arithmetic.  Against plain fp32 attention the reference's own gate
    applies instead (cos >= 0.999, rel-L2 <= 0.02): pass ``cos_min=0.999, max_abs=None,
    rel_l2_max=0.02``."""
    g = got.detach().float().cpu().numpy() if isinstance(got, torch.Tensor) else got
    assert np.isfinite(g).all(), f"{ctx}: non-finite output"
    cos, mabs, rel = O.compare(g, want)
    if os.environ.get("OMMX_TEST_LOG"):
        with open(os.environ["OMMX_TEST_LOG"], "a") as f:
            f.write(f"{ctx}: cos={cos:.7f} max_abs={mabs:.3e} rel_l2={rel:.3e}\n")
    ok = cos >= cos_min and (max_abs is None or mabs <= max_abs) and (rel_l2_max is None or rel <= rel_l2_max)
    assert ok, f"{ctx}: cos={cos:.6f} max_abs={mabs:.3e} rel_l2={rel:.3e}"
    return cos, mabs, rel


def check_fp32(got, want, ctx=""):
    """The reference's own kernel-vs-fp32-oracle gate (attention/oracle.py: COS_MIN, REL_L2_MAX)."""
    return check_close(got, want, cos_min=0.999, max_abs=None, rel_l2_max=0.02, ctx=ctx)
