"""CPU oracle for the OMMX paged-decode hot path.  TEST INFRASTRUCTURE - NOT A PRODUCT PATH.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import this
module; the shipped package never does (it fails loudly when the CUDA library is missing).

It restates, in plain numpy, the arithmetic of the reference project
(Youngmin17/open_ommx_serve) for the one path this repository accelerates:

  * ``pack_kv``            - KV quantize + pack  (ommx_gpu_serve/attention/pack.py:293-655,
                             ommx_gpu_serve/attention/codec.py:45-65, :330-372)
  * ``dequant_kv``         - packed planes -> fp32 K/V (pack.py:701-781, codec.py:68-80)
  * ``attention_fp32``     - textbook fp32 GQA attention (ommx_gpu_serve/attention/oracle.py:33-50)
  * ``decode_split_kv``    - the split-KV stage-1 / stage-2 arithmetic with the reference kernel's
                             bf16 rounding points (ommx_gpu_serve/attention/paged_decode.py
                             :1428-1449, :1738-1770, :1923-1951, :2043-2068, :2234-2284, :2400-2500)
  * ``packed_boundary``    - sink / packed-prefix / recent-tail arithmetic (attention/kv_window.py:35-58)
  * ``fakequant_group``    - the accuracy-side fake quantizer that is the timed CPU baseline
                             (ommx_fakequant/quant_function.py:152-429, :17-55)

Parity pin: tests/golden/*.npz were produced by running the reference's own packer, dequantizer
and fake quantizer in the build container (tests/golden/make_golden.py); tests/test_oracle.py
checks every function here against them bit for bit.  The two calls into a math library
(log2 / log) are replaced by the frozen threshold tables of oracle/tables.json (see
oracle/gen_tables.py), so results do not depend on the host CPU.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(_HERE, "tables.json")) as _f:
    _T = json.load(_f)
POW2_CUT = np.asarray(_T["pow2_cut_mantissa"], dtype=np.uint32)
FP4_THRESH = np.asarray(_T["fp4_first_upper_bits"], dtype=np.uint32)
FP4_LEVELS = np.asarray(_T["fp4_levels"], dtype=np.float32)

GROUP_TOKENS = 32
GROUP_CHANNELS = 32
F32 = np.float32


# ───────────────────────────── scalar helpers ─────────────────────────────

def bf16_round(x):
    """fp32 -> nearest bf16 (ties to even) -> fp32.  Finite inputs."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    b = a.view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000
    return b.astype(np.uint32).view(np.float32).reshape(a.shape)


def bf16_bits(x):
    """fp32 array (already bf16-representable or not) -> uint16 bf16 bit patterns (RNE)."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def pow2_exponent(x):
    """round_half_even(log2(x)) for positive normal fp32 ``x`` via the frozen cut table."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    E = (bits >> 23) & 0xFF
    mant = bits & 0x7FFFFF
    return (E.astype(np.int32) - 127 + (mant >= POW2_CUT[E]).astype(np.int32)).reshape(np.shape(x))


def fp4_encode(m):
    """fp32 -> FP4 E2M1 code (sign<<3 | exp<<1 | mant), nearest in log magnitude, ties low."""
    m = np.ascontiguousarray(m, dtype=np.float32)
    a = np.abs(m).view(np.uint32)
    idx = np.zeros(m.shape, dtype=np.uint8)
    for t in FP4_THRESH:
        idx += (a >= t).astype(np.uint8)
    sign = (m < 0).astype(np.uint8)
    exp = (idx >= 2).astype(np.uint8) + (idx >= 4) + (idx >= 6)
    return ((sign << 3) | (exp.astype(np.uint8) << 1) | (idx & 1)).astype(np.uint8)


def fp4_decode(code):
    c = np.asarray(code).astype(np.int32) & 0xF
    mag = FP4_LEVELS[((c >> 1) & 3) * 2 + (c & 1)]
    return np.where((c >> 3) & 1, -mag, mag).astype(np.float32)


def packed_boundary(seq_len, sink=8, recent=32, group_tokens=GROUP_TOKENS):
    extra = int(seq_len) - sink - recent
    if extra <= 0:
        return min(sink, int(seq_len))
    return sink + (extra // group_tokens) * group_tokens


def _pack2(codes):
    """codes [..., D] in 0..3 -> uint8 [..., D/4]; channel c -> byte c//4, bits 2*(c%4)."""
    c = codes.astype(np.uint8).reshape(*codes.shape[:-1], codes.shape[-1] // 4, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).astype(np.uint8)


def _unpack2(plane):
    p = plane.astype(np.uint8)
    out = np.stack([(p >> s) & 3 for s in (0, 2, 4, 6)], axis=-1)
    return out.reshape(*plane.shape[:-1], plane.shape[-1] * 4)


def _affine_scale(rng, use_pow2, scale_bf16):
    """scale = max(range,1e-8)/3, optionally snapped to a power of two; returns (scale, exponent)."""
    scale = np.maximum(rng.astype(F32), F32(1e-8)) / F32(3.0)
    e = None
    if use_pow2:
        e = pow2_exponent(np.maximum(scale, F32(1e-12)))
        scale = np.ldexp(F32(1.0), e).astype(F32)
    if scale_bf16:
        scale = bf16_round(scale)
    return scale.astype(F32), e


# ───────────────────────────── quantize + pack ─────────────────────────────

def pack_kv(K, V, *, outliers_per_vector=6, outlier_select="signed", use_pow2=True,
            kv_outlier_map=True, kv_int8_scale=True, scale_bf16=True, page_size=16):
    """Quantize + pack ``K``/``V`` ``[T, H, D]`` (T a multiple of 32 and of ``page_size``).

    Returns the plane dict of the reference ABI with the flat-bitmask outlier index
    (pack.py:628-655).  bf16 planes are returned as uint16 bit patterns.
    """
    K = np.ascontiguousarray(K, dtype=np.float32)
    V = np.ascontiguousarray(V, dtype=np.float32)
    T, H, D = K.shape
    gt, gc, k = GROUP_TOKENS, GROUP_CHANNELS, int(outliers_per_vector)
    assert V.shape == K.shape and T % gt == 0 and T % page_size == 0 and D % gc == 0
    if not np.isfinite(V).all():
        raise ValueError("V pack: non-finite input")
    if not np.isfinite(K).all():
        raise ValueError("K pack: non-finite input")
    G, pages = T // gt, T // page_size
    x = K.reshape(G, gt, H, D).transpose(0, 2, 3, 1)            # [G,H,D,32] vectors along tokens
    pos = np.arange(gt)

    omask = np.zeros(x.shape, dtype=bool)
    if k > 0:
        if outlier_select == "signed":
            kt = (k + 1) // 2
            kb = k - kt
            order = np.argsort(-x, axis=-1, kind="stable")      # descending, ties -> low index
            np.put_along_axis(omask, order[..., :kt], True, axis=-1)
            if kb > 0:
                rest = np.where(omask, F32(1e9), x)
                order = np.argsort(rest, axis=-1, kind="stable")
                np.put_along_axis(omask, order[..., :kb], True, axis=-1)
        elif outlier_select == "abs":
            order = np.argsort(-np.abs(x), axis=-1, kind="stable")
            np.put_along_axis(omask, order[..., :k], True, axis=-1)
        else:
            raise ValueError(outlier_select)
    keep = ~omask
    mn = np.where(keep, x, F32(1e9)).min(-1, keepdims=True)
    mx = np.where(keep, x, F32(-1e9)).max(-1, keepdims=True)
    mn = np.where(mn > 1e8, F32(0), mn).astype(F32)
    mx = np.where(mx < -1e8, F32(0), mx).astype(F32)
    scale, e = _affine_scale(mx - mn, use_pow2, scale_bf16)
    zp = bf16_round(mn) if scale_bf16 else mn
    code = np.clip(np.rint((x - zp) / scale), 0, 3).astype(np.uint8)     # [G,H,D,32]

    out = {}
    if k > 0:
        if kv_outlier_map:
            omn = np.where(omask, x, F32(1e9)).min(-1, keepdims=True)
            omx = np.where(omask, x, F32(-1e9)).max(-1, keepdims=True)
            center = ((omx + omn) / F32(2.0)).astype(F32)
            # torch evaluates ``12.0 / tensor`` as reciprocal(tensor) * 12 (two roundings)
            mscale = ((F32(1.0) / np.maximum(omx - omn, F32(1e-8))).astype(F32) * F32(12.0)).astype(F32)
            if scale_bf16:
                center, mscale = bf16_round(center), bf16_round(mscale)
            fpc = fp4_encode(((x - center) * mscale).astype(F32))
            out["k_fp4_mapscale"] = bf16_bits(mscale[..., 0]) if scale_bf16 else mscale[..., 0]
            out["k_fp4_mapcenter"] = bf16_bits(center[..., 0]) if scale_bf16 else center[..., 0]
        else:
            fpc = fp4_encode(((x - zp) / scale).astype(F32))
        # flat bitmask: bit p of the little-endian 32-bit frame = token p is an outlier
        word = (omask.astype(np.uint64) << pos.astype(np.uint64)).sum(-1).astype(np.uint32)
        out["k_obmp"] = np.ascontiguousarray(word)[..., None].view(np.uint8).reshape(G, H, D, 4)
        # value stream: nibble s = code of the s-th outlier in ascending token order
        rank = np.cumsum(omask, axis=-1) - 1
        nbytes = (k + 1) // 2
        stream = np.zeros((G, H, D), dtype=np.uint64)
        contrib = np.where(omask, fpc.astype(np.uint64) << (4 * np.maximum(rank, 0)).astype(np.uint64), 0)
        stream = contrib.sum(-1).astype(np.uint64)
        out["k_oval"] = np.stack([(stream >> np.uint64(8 * i)) & np.uint64(0xFF) for i in range(nbytes)],
                                 axis=-1).astype(np.uint8)
    codes_tok = code.transpose(0, 3, 1, 2).reshape(T, H, D)            # token-major
    out["k_base"] = _pack2(codes_tok).reshape(pages, page_size, H, D // 4)
    int8 = bool(kv_int8_scale and use_pow2)
    out["k_scale"] = (e[..., 0].astype(np.int8) if int8 else
                      (bf16_bits(scale[..., 0]) if scale_bf16 else scale[..., 0]))
    out["k_zp"] = bf16_bits(zp[..., 0]) if scale_bf16 else zp[..., 0]

    v = V.reshape(T, H, D // gc, gc)
    vmn = v.min(-1, keepdims=True)
    vmx = v.max(-1, keepdims=True)
    vscale, ve = _affine_scale(vmx - vmn, use_pow2, scale_bf16)
    vzp = bf16_round(vmn) if scale_bf16 else vmn
    vcode = np.clip(np.rint((v - vzp) / vscale), 0, 3).astype(np.uint8)
    out["v_main"] = _pack2(vcode.reshape(T, H, D)).reshape(pages, page_size, H, D // 4)
    out["v_scale"] = (ve[..., 0].astype(np.int8) if int8 else
                      (bf16_bits(vscale[..., 0]) if scale_bf16 else vscale[..., 0])
                      ).reshape(pages, page_size, H, D // gc)
    out["v_zp"] = (bf16_bits(vzp[..., 0]) if scale_bf16 else vzp[..., 0]).reshape(
        pages, page_size, H, D // gc)
    out.update(head_dim=D, n_kv_heads=H, num_tokens=T, n_groups=G, page_size=int(page_size),
               outliers_per_vector=k, kv_outlier_map=bool(kv_outlier_map and k > 0),
               kv_int8_scale=int8, scale_bf16=bool(scale_bf16))
    return out


def relidx7_from_bitmask(obmp, k):
    """Flat bitmask plane [..., 4] -> relidx7 plane [..., ceil(7k/8)]: the k token positions of a frame, ascending,
    7 bits each, LSB first (ommx_gpu_serve/attention/codec.py:91-113, pack.py:128-165 of the reference)."""
    obmp = np.ascontiguousarray(obmp, dtype=np.uint8)
    lead = obmp.shape[:-1]
    word = obmp.reshape(-1, 4).copy().view(np.uint32)[:, 0]
    n = word.shape[0]
    nbi = (7 * k + 7) // 8
    bits = ((word[:, None] >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(bool)
    if not (bits.sum(1) == k).all():
        raise ValueError("a frame does not hold exactly k outliers")
    pos = np.nonzero(bits)[1].reshape(n, k).astype(np.uint64)            # ascending within a frame
    stream_bits = np.zeros((n, nbi * 8), dtype=np.uint8)
    for r in range(k):
        for b in range(7):
            stream_bits[:, 7 * r + b] = (pos[:, r] >> np.uint64(b)) & np.uint64(1)
    out = np.packbits(stream_bits.reshape(n, nbi, 8), axis=-1, bitorder="little")[..., 0]
    return out.reshape(lead + (nbi,))


def bitmask_from_relidx7(oidx, k):
    """Inverse of :func:`relidx7_from_bitmask` (codec.py:116-130): relidx7 plane -> flat bitmask plane [..., 4]."""
    oidx = np.ascontiguousarray(oidx, dtype=np.uint8)
    lead = oidx.shape[:-1]
    nbi = oidx.shape[-1]
    sb = np.unpackbits(oidx.reshape(-1, nbi), axis=-1, bitorder="little")
    word = np.zeros(sb.shape[0], dtype=np.uint32)
    for r in range(k):
        pos = np.zeros(sb.shape[0], dtype=np.uint32)
        for b in range(7):
            pos |= sb[:, 7 * r + b].astype(np.uint32) << np.uint32(b)
        if (pos > 31).any():
            raise ValueError("a relidx7 position lies beyond the 32-token group")
        word |= np.uint32(1) << pos
    return np.ascontiguousarray(word)[:, None].view(np.uint8).reshape(lead + (4,))


def with_bitmask(planes):
    """Planes whose outlier index is the relidx7 stream (``k_oidx``) re-expressed with the flat bitmask the other
    oracle functions read; planes that already hold ``k_obmp`` pass through."""
    if planes.get("k_obmp") is not None or planes.get("k_oidx") is None:
        return planes
    out = dict(planes)
    out["k_obmp"] = bitmask_from_relidx7(planes["k_oidx"], int(planes["k_oval"].shape[-1]) * 2 if "outliers_per_vector" not in planes
                                         else int(planes["outliers_per_vector"]))
    return out


def _plane_f32(p, scale_bf16):
    return bf16_from_bits(p) if (scale_bf16 and p.dtype == np.uint16) else p.astype(F32)


def dequant_kv(planes):
    """Packed planes -> fp32 ``(K, V)`` ``[T, H, D]`` (identity page / group tables)."""
    T, H, D = planes["num_tokens"], planes["n_kv_heads"], planes["head_dim"]
    G, k = planes["n_groups"], planes["outliers_per_vector"]
    sb = planes.get("scale_bf16", True)
    code = _unpack2(planes["k_base"].reshape(T, H, D // 4)).astype(F32)
    if planes["k_scale"].dtype == np.int8:
        scale = np.ldexp(F32(1.0), planes["k_scale"].astype(np.int32)).astype(F32)
    else:
        scale = _plane_f32(planes["k_scale"], sb)
    zp = _plane_f32(planes["k_zp"], sb)
    Kd = code.reshape(G, 32, H, D) * scale[:, None] + zp[:, None]
    if k > 0:
        word = planes["k_obmp"].reshape(G, H, D, 4).copy().view(np.uint32)[..., 0]
        bits = ((word[..., None] >> np.arange(32, dtype=np.uint32)) & 1).astype(bool)   # [G,H,D,32]
        rank = np.cumsum(bits, -1) - 1
        stream = np.zeros((G, H, D), dtype=np.uint64)
        for i in range(planes["k_oval"].shape[-1]):
            stream |= planes["k_oval"][..., i].astype(np.uint64) << np.uint64(8 * i)
        nib = (stream[..., None] >> (4 * np.maximum(rank, 0)).astype(np.uint64)) & np.uint64(0xF)
        lvl = fp4_decode(nib)
        if planes["kv_outlier_map"]:
            ms = _plane_f32(planes["k_fp4_mapscale"], sb)[..., None]
            mc = _plane_f32(planes["k_fp4_mapcenter"], sb)[..., None]
            ov = (lvl / ms + mc).astype(F32)
        else:
            ov = (lvl * scale[..., None] + zp[..., None]).astype(F32)
        Kd = np.where(bits.transpose(0, 3, 1, 2), ov.transpose(0, 3, 1, 2), Kd)
    Kd = Kd.reshape(T, H, D).astype(F32)
    vcode = _unpack2(planes["v_main"].reshape(T, H, D // 4)).astype(F32).reshape(T, H, D // 32, 32)
    if planes["v_scale"].dtype == np.int8:
        vs = np.ldexp(F32(1.0), planes["v_scale"].astype(np.int32)).astype(F32)
    else:
        vs = _plane_f32(planes["v_scale"], sb)
    vz = _plane_f32(planes["v_zp"], sb)
    Vd = (vcode * vs.reshape(T, H, -1, 1) + vz.reshape(T, H, -1, 1)).reshape(T, H, D).astype(F32)
    return Kd, Vd


# ───────────────────────────── attention ─────────────────────────────

def attention_fp32(q, K, V, sm_scale):
    """One query row per head: ``q [Hq,D]``, ``K,V [T,Hkv,D]`` -> ``(o [Hq,D], lse [Hq])`` in fp64->fp32."""
    Hq, D = q.shape
    Hkv = K.shape[1]
    per = Hq // Hkv
    o = np.zeros((Hq, D), dtype=np.float64)
    lse = np.full((Hq,), -np.inf)
    if K.shape[0] == 0:
        return o.astype(F32), lse.astype(F32)
    for h in range(Hq):
        kh = h // per
        s = (K[:, kh, :].astype(np.float64) @ q[h].astype(np.float64)) * sm_scale
        m = s.max()
        w = np.exp(s - m)
        o[h] = (w[:, None] * V[:, kh, :].astype(np.float64)).sum(0) / w.sum()
        lse[h] = m + math.log(w.sum())
    return o.astype(F32), lse.astype(F32)


def split_ranges(seq, num_splits):
    """Token range of every split: per = ceil(ceil(seq/S)/32)*32 (paged_decode.py:1428-1432)."""
    per = -(-(-(-seq // num_splits)) // GROUP_TOKENS) * GROUP_TOKENS if seq > 0 else 0
    return [(s * per, min((s + 1) * per, seq)) for s in range(num_splits)]


def decode_split_kv(q, planes, k_tail, v_tail, sm_scale, num_splits, *, seq=None,
                    req_to_token=None, req_to_group=None, split_pv=False):
    """Reference-kernel arithmetic for one sequence (bf16 rounding points kept).

    ``q [Hq,D]`` bf16-representable fp32; ``planes`` as produced by :func:`pack_kv` (int8
    scales, dedicated map when k>0), possibly pooled and addressed through ``req_to_token``
    (page ids) / ``req_to_group`` (group slots); ``k_tail/v_tail [Ttail,Hkv,D]``.
    Returns ``(o [Hq,D], lse [Hq], attn_logits [Hq,S,D+1])``.
    """
    Hq, D = q.shape
    H = planes["n_kv_heads"]
    per_h = Hq // H
    ps = planes["page_size"]
    k = planes["outliers_per_vector"]
    if seq is None:
        seq = planes["num_tokens"]
    n_pages, n_groups = -(-seq // ps), seq // 32
    r2t = np.arange(n_pages) if req_to_token is None else np.asarray(req_to_token)
    r2g = np.arange(n_groups) if req_to_group is None else np.asarray(req_to_group)
    kb = planes["k_base"].reshape(-1, planes["k_base"].shape[2], D // 4)     # [pages*ps, H, D/4]
    vm = planes["v_main"].reshape(-1, H, D // 4)
    vsc = planes["v_scale"].reshape(-1, H, D // 32)
    vzp = planes["v_zp"].reshape(-1, H, D // 32)
    mid = np.zeros((Hq, num_splits, D + 1), dtype=F32)
    mid[:, :, D] = -np.inf
    qc = bf16_round((q.astype(F32) * F32(sm_scale)).astype(F32))            # bf16(q*sm_scale)
    for s, (t0, t1) in enumerate(split_ranges(seq, num_splits)):
        if t1 <= t0:
            continue
        toks = np.arange(t0, t1)
        loc = r2t[toks // ps] * ps + toks % ps
        gslot = r2g[toks // 32]
        for kh in range(H):
            code = _unpack2(kb[loc, kh]).astype(F32)                        # [n, D]
            sc = np.ldexp(F32(1.0), planes["k_scale"][gslot, kh].astype(np.int32)).astype(F32)
            zp = bf16_from_bits(planes["k_zp"][gslot, kh])
            kbase = bf16_round(code * sc)                                   # exact: code*2^e
            delta = np.zeros_like(kbase)
            if k > 0:
                word = planes["k_obmp"][gslot, kh].reshape(len(toks), D, 4).copy().view(np.uint32)[..., 0]
                tpos = (toks % 32).astype(np.uint32)[:, None]
                isout = ((word >> tpos) & 1).astype(bool)
                below = word & ((np.uint32(1) << tpos) - np.uint32(1))
                rank = np.zeros_like(below)
                for b in range(32):
                    rank += (below >> np.uint32(b)) & 1
                stream = np.zeros(word.shape, dtype=np.uint64)
                ov = planes["k_oval"][gslot, kh]
                for i in range(ov.shape[-1]):
                    stream |= ov[..., i].astype(np.uint64) << np.uint64(8 * i)
                lvl = fp4_decode((stream >> (4 * rank).astype(np.uint64)) & np.uint64(0xF))
                if planes["kv_outlier_map"]:
                    ms = bf16_from_bits(planes["k_fp4_mapscale"][gslot, kh])
                    mc = bf16_from_bits(planes["k_fp4_mapcenter"][gslot, kh])
                    ov = (lvl / ms + mc).astype(F32)
                else:
                    ov = (lvl * sc + zp).astype(F32)
                d = bf16_round((ov - (kbase + zp)).astype(F32))
                delta = np.where(isout, d, F32(0))
            vcode = _unpack2(vm[loc, kh]).astype(F32).reshape(len(toks), D // 32, 32)
            vs = np.ldexp(F32(1.0), vsc[loc, kh].astype(np.int32)).astype(F32)[..., None]
            vz = bf16_from_bits(vzp[loc, kh])[..., None]
            if split_pv:
                vdq = bf16_round(vcode * vs).reshape(len(toks), D)
                vbias = np.repeat(vz, 32, axis=-1).reshape(len(toks), D)
            else:
                vdq = bf16_round((vcode * vs + vz).astype(F32)).reshape(len(toks), D)
                vbias = None
            kfull = kbase.astype(np.float64) + delta.astype(np.float64)
            for j in range(per_h):
                h = kh * per_h + j
                qzp = (zp.astype(np.float64) @ q[h].astype(np.float64)).astype(F32) * F32(sm_scale)
                logit = (kfull @ qc[h].astype(np.float64)).astype(F32) + qzp
                # online softmax over 32-token tiles, as the kernel runs it (paged_decode.py:2060-2068)
                e_max, e_sum = F32(-np.inf), 0.0
                acc = np.zeros(D, dtype=np.float64)
                for g0 in range(0, len(toks), GROUP_TOKENS):
                    x = logit[g0:g0 + GROUP_TOKENS]
                    n_max = max(e_max, x.max())
                    re = math.exp(float(e_max) - float(n_max)) if np.isfinite(e_max) else 0.0
                    p = np.exp((x - n_max).astype(F32)).astype(F32)
                    pb = bf16_round(p).astype(np.float64)
                    acc = acc * re + pb @ vdq[g0:g0 + GROUP_TOKENS].astype(np.float64)
                    if vbias is not None:
                        acc = acc + pb @ vbias[g0:g0 + GROUP_TOKENS].astype(np.float64)
                    e_sum = e_sum * re + float(p.astype(np.float64).sum())
                    e_max = n_max
                mid[h, s, :D] = (acc / e_sum).astype(F32)
                mid[h, s, D] = F32(float(e_max) + math.log(e_sum))
    o_t, lse_t = attention_fp32(q, k_tail, v_tail, sm_scale)
    o = np.zeros((Hq, D), dtype=F32)
    lse = np.zeros((Hq,), dtype=F32)
    for h in range(Hq):
        parts_l = np.concatenate([mid[h, :, D], [lse_t[h]]]).astype(np.float64)
        parts_o = np.concatenate([mid[h, :, :D], o_t[h][None]], 0).astype(np.float64)
        m = parts_l.max()
        if not np.isfinite(m):
            lse[h] = -np.inf
            continue
        w = np.exp(parts_l - m)
        o[h] = ((w[:, None] * parts_o).sum(0) / w.sum()).astype(F32)
        lse[h] = F32(m + math.log(w.sum()))
    return o, lse, mid


def merge_states(o_parts, lse_parts):
    """Merge P partial softmax states ``[P,R,D]``, ``[P,R]`` (paged_decode.py:3556-3624)."""
    l = lse_parts.astype(np.float64)
    m = l.max(0)
    msafe = np.where(np.isfinite(m), m, 0.0)
    w = np.exp(l - msafe)
    den = w.sum(0)
    o = (w[..., None] * o_parts.astype(np.float64)).sum(0) / np.where(den > 0, den, 1.0)[..., None]
    with np.errstate(divide="ignore"):
        lse = msafe + np.log(den)
    return o.astype(F32), lse.astype(F32)


def compare(got, want):
    """(cosine, max_abs, rel_l2) as the reference's gate computes them (attention/oracle.py:53-63)."""
    g = np.asarray(got, dtype=np.float64).ravel()
    w = np.asarray(want, dtype=np.float64).ravel()
    cos = float(g @ w / max(np.linalg.norm(g) * np.linalg.norm(w), 1e-30))
    return cos, float(np.abs(g - w).max()), float(np.linalg.norm(g - w) / max(np.linalg.norm(w), 1e-12))


# ───────────────────────────── fake quantizer (timed CPU baseline) ─────────────────────────────

def fakequant_group(x, *, is_key, group=32, sink_front=8, sink_back=32, top=3, bottom=3,
                    use_pow2=True):
    """Fake-quantize ``x [Hkv, T, D]`` fp32 the way the accuracy-side CPU path does.

    K (``is_key``): vectors of ``group`` consecutive tokens per channel, ``top`` largest and
    ``bottom`` smallest values kept as FP4 through a dedicated [-6,6] map; V: vectors of ``group``
    consecutive channels per token, no outliers.  The first ``sink_front`` and last ``sink_back``
    tokens pass through.  Tokens that do not fill a whole vector are zero-padded exactly as the
    reference does (quant_function.py:264-274).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    Hh, T, D = x.shape
    lo, hi = (sink_front if T > sink_front else 0), (T - sink_back if T > sink_back else T)
    mid = x[:, lo:hi, :]
    if mid.shape[1] == 0:
        return x.copy()
    w = mid.transpose(0, 2, 1) if is_key else mid                      # [..., L] grouped along last
    L = w.shape[-1]
    pad = (-L) % group
    wp = np.pad(w, [(0, 0), (0, 0), (0, pad)])
    valid = np.pad(np.ones(w.shape, dtype=bool), [(0, 0), (0, 0), (0, pad)])
    g = wp.reshape(Hh, wp.shape[1], -1, group)
    gv = valid.reshape(g.shape)
    omask = np.zeros(g.shape, dtype=bool)
    if is_key and top > 0:
        thr = np.sort(np.where(gv, g, np.finfo(F32).min), -1)[..., -top][..., None]
        omask |= g >= thr
    if is_key and bottom > 0:
        thr = np.sort(np.where(gv, g, np.finfo(F32).max), -1)[..., bottom - 1][..., None]
        omask |= g <= thr
    qm = (~omask) & gv
    mn = np.where(qm, g, F32(0)) + np.where(qm, F32(0), F32(1e8))
    mxv = np.where(qm, g, F32(0)) - np.where(qm, F32(0), F32(1e8))
    mn = mn.min(-1, keepdims=True).astype(F32)
    mxv = mxv.max(-1, keepdims=True).astype(F32)
    rng = mxv - mn
    scale = (rng / F32(3.0)).astype(F32)
    scale = np.where(rng <= 1e-8, F32(1.0), scale)
    if use_pow2:
        scale = np.ldexp(F32(1.0), pow2_exponent(np.maximum(scale, F32(1e-12)))).astype(F32)
    qv = np.clip(np.rint((g - mn) / scale), 0, 3)
    out = np.where(qm, (qv * scale + mn).astype(F32), g)
    if omask.any():
        omn = np.where(omask, g, F32(1e8)).min(-1, keepdims=True)
        omx = np.where(omask, g, F32(-1e8)).max(-1, keepdims=True)
        center = ((omx + omn) / F32(2.0)).astype(F32)
        mscale = ((F32(1.0) / np.maximum(omx - omn, F32(1e-8))).astype(F32) * F32(12.0)).astype(F32)
        lvl = fp4_decode(fp4_encode(((g - center) * mscale).astype(F32)))
        out = np.where(omask, (lvl / mscale + center).astype(F32), out)
    res = out.reshape(Hh, wp.shape[1], -1)[..., :L]
    res = res.transpose(0, 2, 1) if is_key else res
    full = x.copy()
    full[:, lo:hi, :] = res
    return full


def fakequant_group_torch(x, *, is_key, group=32, sink_front=8, sink_back=32, top=3, bottom=3):
    """Same arithmetic as :func:`fakequant_group` with multi-threaded torch CPU ops - the form
    the benchmark times as the CPU baseline (``x`` is a torch fp32 tensor ``[Hkv, T, D]``)."""
    import torch
    Hh, T, D = x.shape
    lo, hi = (sink_front if T > sink_front else 0), (T - sink_back if T > sink_back else T)
    mid = x[:, lo:hi, :]
    if mid.shape[1] == 0:
        return x.clone()
    w = mid.transpose(1, 2) if is_key else mid
    L = w.shape[-1]
    pad = (-L) % group
    wp = torch.nn.functional.pad(w, (0, pad))
    valid = torch.ones(L + pad, dtype=torch.bool)
    valid[L:] = False
    g = wp.reshape(Hh, wp.shape[1], -1, group)
    gv = valid.reshape(1, 1, -1, group).expand_as(g)
    omask = torch.zeros_like(g, dtype=torch.bool)
    fmin, fmax = torch.finfo(torch.float32).min, torch.finfo(torch.float32).max
    if is_key and top > 0:
        thr = torch.topk(torch.where(gv, g, torch.tensor(fmin)), top, dim=-1).values[..., -1:]
        omask |= g >= thr
    if is_key and bottom > 0:
        thr = torch.topk(torch.where(gv, g, torch.tensor(fmax)), bottom, dim=-1, largest=False).values[..., -1:]
        omask |= g <= thr
    qm = (~omask) & gv
    base = g * qm
    far = (~qm).float() * 1e8
    mn = (base + far).min(-1, keepdim=True).values
    mxv = (base - far).max(-1, keepdim=True).values
    rng = mxv - mn
    scale = rng / 3
    scale = torch.where(rng <= 1e-8, torch.ones_like(scale), scale)
    scale = torch.pow(2.0, torch.round(torch.log2(scale.clamp(min=1e-12))))
    out = torch.where(qm, torch.round((g - mn) / scale).clamp(0, 3) * scale + mn, g)
    if bool(omask.any()):
        omn = torch.where(omask, g, torch.tensor(1e8)).min(-1, keepdim=True).values
        omx = torch.where(omask, g, torch.tensor(-1e8)).max(-1, keepdim=True).values
        center = (omx + omn) / 2.0
        mscale = 12.0 / (omx - omn).clamp_min(1e-8)
        m = (g - center) * mscale
        idx = torch.bucketize(m.abs().view(torch.int32), torch.from_numpy(FP4_THRESH.astype(np.int32)), right=True)
        lvl = torch.from_numpy(FP4_LEVELS)[idx] * torch.sign(m)
        out = torch.where(omask, lvl / mscale + center, out)
    res = out.reshape(Hh, wp.shape[1], -1)[..., :L]
    res = res.transpose(1, 2) if is_key else res
    full = x.clone()
    full[:, lo:hi, :] = res
    return full
