"""KV quantize + pack on the GPU, behind the reference's ``ommx_pack_kv_canonical_block``.

Mirrors ``ommx_gpu_serve/attention/pack.py:293-655`` of the reference: same keyword set, same
returned plane dict, planes bit-identical to the reference packer run on CPU.  The work is done
by ``ommx_b200_pack_kv`` in libommx_b200.so (csrc/ommx_pack.cu); nothing here computes.

``ommx_pack_kv_into`` is the form the stores use: it quantizes a block straight into slots of
existing pooled planes (what the reference does with a pack followed by per-plane copies,
``attention/kv_store.py:594-610``, ``attention/kv_pool.py:619-635``).
"""
from __future__ import annotations

import os
from typing import Any, Optional

import torch

from .. import _lib

CANONICAL_GROUP_TOKENS = 32
CANONICAL_GROUP_CHANNELS = 32
OUTLIER_REPRS = ("relidx7", "combinadic", "bitmap")
_FALSE = {"0", "false", "off", "no"}


def _env_flag(name: str, default: bool) -> bool:
    raw = os.environ.get(name)
    return (raw.strip().lower() not in _FALSE) if raw else default


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.OMMX_DT_F32
    if t.dtype == torch.bfloat16:
        return _lib.OMMX_DT_BF16
    if t.dtype == torch.float16:
        return _lib.OMMX_DT_F16
    raise ValueError(f"K/V dtype {t.dtype} is not supported (float32, bfloat16, float16)")


def _scale_kind(scale_dtype, use_int8: bool) -> int:
    if use_int8:
        return _lib.OMMX_SCALE_INT8_EXP
    if scale_dtype == torch.bfloat16:
        return _lib.OMMX_SCALE_BF16
    if scale_dtype == torch.float32:
        return _lib.OMMX_SCALE_F32
    raise NotImplementedError(f"scale_dtype {scale_dtype} is not supported (bfloat16, float32)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def planes_struct(planes: dict, *, k: int, outlier_map: bool, relidx7: bool = False) -> "_lib.KVPlanes":
    """Fill the C plane descriptor from a plane dict (every plane contiguous, same device).  With ``relidx7`` the
    outlier-index plane is ``k_oidx`` (the reference's 7-bit position stream) instead of the flat bitmask ``k_obmp``."""
    kb = planes["k_base"]
    for name in ("k_base", "k_scale", "k_zp", "k_obmp", "k_oval", "k_fp4_mapscale",
                 "k_fp4_mapcenter", "v_main", "v_scale", "v_zp"):
        t = planes.get(name)
        if t is not None and not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    ks = planes["k_scale"]
    if ks.dtype == torch.int8:
        kind = _lib.OMMX_SCALE_INT8_EXP
    elif ks.dtype == torch.bfloat16:
        kind = _lib.OMMX_SCALE_BF16
    elif ks.dtype == torch.float32:
        kind = _lib.OMMX_SCALE_F32
    else:
        raise ValueError(f"k_scale dtype {ks.dtype} not understood")
    s = _lib.KVPlanes()
    s.n_kv_heads = int(kb.shape[2])
    s.head_dim = int(kb.shape[3]) * 4
    s.page_size = int(kb.shape[1])
    s.num_pages = int(kb.shape[0])
    s.num_group_slots = int(ks.shape[0])
    s.outliers_per_vector = int(k)
    s.kv_outlier_map = 1 if (outlier_map and k > 0) else 0
    s.scale_kind = kind
    s.k_base, s.k_scale, s.k_zp = _ptr(kb), _ptr(ks), _ptr(planes["k_zp"])
    if relidx7 and k > 0:
        idx = planes.get("k_oidx")
        if idx is None or not idx.is_contiguous() or idx.dtype != torch.uint8 or int(idx.shape[-1]) != (7 * int(k) + 7) // 8:
            raise ValueError(f"k_oidx must be a contiguous uint8 plane of ceil(7k/8)={(7 * int(k) + 7) // 8} bytes per frame")
        s.k_obmp, s.outlier_index = _ptr(idx), _lib.OMMX_OIDX_RELIDX7
    else:
        s.k_obmp, s.outlier_index = _ptr(planes.get("k_obmp")), _lib.OMMX_OIDX_BITMASK
    s.k_oval = _ptr(planes.get("k_oval"))
    s.k_mapscale, s.k_mapcenter = _ptr(planes.get("k_fp4_mapscale")), _ptr(planes.get("k_fp4_mapcenter"))
    s.v_main, s.v_scale, s.v_zp = _ptr(planes["v_main"]), _ptr(planes["v_scale"]), _ptr(planes["v_zp"])
    return s


def alloc_planes(num_pages: int, num_group_slots: int, n_kv_heads: int, head_dim: int, *,
                 page_size: int = 16, outliers_per_vector: int = 6, kv_outlier_map: bool = True,
                 scale_kind: int = _lib.OMMX_SCALE_INT8_EXP, device="cuda") -> dict:
    """Allocate an empty plane set (the ABI of ``ommx_gpu_serve/attention/paged_decode.py:2856-2887``)."""
    H, D, k = int(n_kv_heads), int(head_dim), int(outliers_per_vector)
    sdt = {_lib.OMMX_SCALE_INT8_EXP: torch.int8, _lib.OMMX_SCALE_BF16: torch.bfloat16,
           _lib.OMMX_SCALE_F32: torch.float32}[scale_kind]
    zdt = torch.float32 if scale_kind == _lib.OMMX_SCALE_F32 else torch.bfloat16
    z = dict(device=device)
    out = {
        "k_base": torch.zeros(num_pages, page_size, H, D // 4, dtype=torch.uint8, **z),
        "k_scale": torch.zeros(num_group_slots, H, D, dtype=sdt, **z),
        "k_zp": torch.zeros(num_group_slots, H, D, dtype=zdt, **z),
        "k_oidx": None, "k_crank": None, "k_obmp": None, "k_oval": None,
        "k_fp4_mapscale": None, "k_fp4_mapcenter": None,
        "v_main": torch.zeros(num_pages, page_size, H, D // 4, dtype=torch.uint8, **z),
        "v_scale": torch.zeros(num_pages, page_size, H, D // 32, dtype=sdt, **z),
        "v_zp": torch.zeros(num_pages, page_size, H, D // 32, dtype=zdt, **z),
    }
    if k > 0:
        out["k_obmp"] = torch.zeros(num_group_slots, H, D, 4, dtype=torch.uint8, **z)
        out["k_oval"] = torch.zeros(num_group_slots, H, D, (k + 1) // 2, dtype=torch.uint8, **z)
        if kv_outlier_map:
            out["k_fp4_mapscale"] = torch.zeros(num_group_slots, H, D, dtype=zdt, **z)
            out["k_fp4_mapcenter"] = torch.zeros(num_group_slots, H, D, dtype=zdt, **z)
    return out


def ommx_pack_kv_into(K, V, planes: dict, *, dst_pages=None, dst_groups=None,
                      outliers_per_vector: int, outlier_select: str = "signed", use_pow2: bool = True,
                      kv_outlier_map: bool = True, status: Optional[torch.Tensor] = None) -> None:
    """Quantize ``K``/``V`` ``[32*n, H, D]`` into ``planes`` at the given page ids / group slots.

    ``dst_pages`` int32 ``[T/page_size]`` and ``dst_groups`` int32 ``[T/32]`` are device tensors
    (``None`` = 0,1,2,...).  No host synchronisation; errors the device sees (page or slot out of
    range, non-finite input) are OR-ed into ``status`` (int32 ``[1]``) when it is given.
    """
    lib = _lib.load()
    if not K.is_cuda:
        raise RuntimeError("ommx_pack_kv_into needs CUDA tensors (no CPU path)")
    if tuple(K.shape) != tuple(V.shape) or K.dim() != 3:
        raise ValueError(f"K/V shape mismatch: {tuple(K.shape)} vs {tuple(V.shape)}")
    if K.dtype != V.dtype:
        raise ValueError("K and V must share a dtype")
    if K.stride(-1) != 1 or V.stride(-1) != 1 or K.stride() != V.stride():
        K, V = K.contiguous(), V.contiguous()
    sel = str(outlier_select).lower()
    if sel not in ("signed", "abs"):
        raise ValueError(f"outlier_select must be signed|abs; got {outlier_select!r}")
    a = _lib.PackArgs()
    a.k, a.v = K.data_ptr(), V.data_ptr()
    a.in_dtype = _dtype_code(K)
    a.num_tokens = int(K.shape[0])
    a.stride_token, a.stride_head = int(K.stride(0)), int(K.stride(1))
    for name, t in (("dst_pages", dst_pages), ("dst_groups", dst_groups)):
        if t is not None and (t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous int32 CUDA tensor")
    a.dst_pages, a.dst_groups = _ptr(dst_pages), _ptr(dst_groups)
    a.outlier_select = 1 if sel == "signed" else 0
    a.use_pow2 = 1 if use_pow2 else 0
    a.planes = planes_struct(planes, k=int(outliers_per_vector), outlier_map=bool(kv_outlier_map))
    if a.planes.n_kv_heads != int(K.shape[1]) or a.planes.head_dim != int(K.shape[2]):
        raise ValueError("K/V geometry does not match the destination planes")
    a.status = _ptr(status)
    with torch.cuda.device(K.device):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.ommx_b200_pack_kv(a, stream), "ommx_b200_pack_kv")


def ommx_pack_kv_canonical_block(
    K, V, *,
    outliers_per_vector: int = 3,
    scale_dtype: Any = None,
    page_size: int = 16,
    device: Any = None,
    outlier_repr: str = "relidx7",
    outlier_select: str = "abs",
    k_format: str = "i2f4",
    use_pow2: bool = False,
    kv_outlier_map: Any = None,
    kv_int8_scale: Any = None,
    group_tokens: int = CANONICAL_GROUP_TOKENS,
    group_channels: int = CANONICAL_GROUP_CHANNELS,
    v_format: str = "i2",
    check_finite: bool = True,
):
    """Pack a K/V block of exactly ``32*n`` tokens into fresh planes (reference signature).

    ``K``/``V`` are ``[num_tokens, n_kv_heads, head_dim]`` float32 / bfloat16 / float16; CPU
    tensors are copied to ``device`` (default: the current CUDA device) first.  The returned
    dict has the reference's keys (``attention/pack.py:628-655``).  Served here: the flat
    bitmask and the relidx7 outlier index (``outlier_repr='bitmap'`` / ``'relidx7'``, k <= 16),
    32-token / 32-channel groups, INT2 V.
    Anything else raises ``NotImplementedError`` - there is no slower fallback.
    ``check_finite`` reads one status word back (a host sync, as the reference's own finite
    check is) and raises ``ValueError`` on NaN/Inf input.
    """
    if scale_dtype is None:
        scale_dtype = torch.bfloat16
    repr_l = str(outlier_repr).lower()
    if repr_l not in OUTLIER_REPRS:
        raise ValueError(f"outlier_repr must be one of {OUTLIER_REPRS}; got {outlier_repr!r}")
    kfmt = str(k_format).lower()
    if kfmt not in ("i2f4", "itf4"):
        raise ValueError(f"k_format must be i2f4|itf4; got {k_format!r}")
    vfmt = str(v_format).lower()
    if vfmt not in ("i2", "bf16"):
        raise ValueError(f"v_format must be i2|bf16; got {v_format!r}")
    if kv_outlier_map is None:
        kv_outlier_map = _env_flag("OMMX_KV_OUTLIER_MAP", True)
    if kv_int8_scale is None:
        kv_int8_scale = _env_flag("OMMX_KV_INT8_SCALE", True)
    use_int8 = bool(kv_int8_scale) and bool(use_pow2)
    T, H, D = (int(s) for s in K.shape)
    if tuple(V.shape) != (T, H, D):
        raise ValueError(f"K/V shape mismatch: {tuple(K.shape)} vs {tuple(V.shape)}")
    gt, gc, k = int(group_tokens), int(group_channels), int(outliers_per_vector)
    if gt not in (16, 32, 64, 128):
        raise ValueError(f"group_tokens (K vector_length) must be in {{16,32,64,128}}; got {gt}")
    if gc not in (16, 32, 64, 128):
        raise ValueError(f"group_channels (V vector_length) must be in {{16,32,64,128}}; got {gc}")
    if T % gt != 0 or T % int(page_size) != 0:
        raise ValueError(f"num_tokens={T} must be a multiple of {gt} and page_size")
    if D % gc != 0 or D % 4 != 0:
        raise ValueError(f"head_dim={D} must be a multiple of {gc}")
    if k < 0 or k > gt:
        raise ValueError(f"outliers_per_vector={k} out of range [0, {gt}]")
    if k > 0 and repr_l == "combinadic":
        raise NotImplementedError(
            "outlier_repr='combinadic': this build packs the flat-bitmask and relidx7 outlier indices")
    if k > 16 and repr_l == "relidx7":
        raise NotImplementedError("relidx7 planes are packed for up to 16 outliers per vector")
    if gt != 32 or gc != 32:
        raise NotImplementedError("this build packs 32-token K groups and 32-channel V groups only")
    if vfmt != "i2":
        raise NotImplementedError("this build packs INT2 V only")
    if device is None:
        device = K.device if K.is_cuda else torch.device("cuda", torch.cuda.current_device()) \
            if torch.cuda.is_available() else None
    if device is None or torch.device(device).type != "cuda":
        raise RuntimeError("ommx_pack_kv_canonical_block runs on a CUDA device only (no CPU path)")
    device = torch.device(device)
    Kd, Vd = K.to(device), V.to(device)
    use_map = bool(kv_outlier_map) and k > 0
    planes = alloc_planes(T // int(page_size), T // gt, H, D, page_size=int(page_size),
                          outliers_per_vector=k, kv_outlier_map=use_map,
                          scale_kind=_scale_kind(scale_dtype, use_int8), device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device) if check_finite else None
    ommx_pack_kv_into(Kd, Vd, planes, outliers_per_vector=k, outlier_select=outlier_select,
                      use_pow2=bool(use_pow2), kv_outlier_map=use_map, status=status)
    if check_finite:
        bits = int(status.item())
        if bits & _lib.ST_NONFINITE:
            raise ValueError("KV pack: non-finite input (NaN/inf) - it would poison a whole group's scale")
        if bits:
            raise RuntimeError(f"KV pack: device reported {_lib.status_text(bits)}")
    G, pages = T // gt, T // int(page_size)
    if k > 0 and repr_l == "relidx7":
        # same outlier set, other index encoding: k ascending 7-bit positions per frame (the value plane is shared)
        lib = _lib.load()
        oidx = torch.zeros(G, H, D, (7 * k + 7) // 8, dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            _lib.check(lib.ommx_b200_outlier_index_convert(planes["k_obmp"].data_ptr(), oidx.data_ptr(), G * H * D, k, 1, None,
                                                           torch.cuda.current_stream().cuda_stream),
                       "ommx_b200_outlier_index_convert")
        planes["k_oidx"], planes["k_obmp"] = oidx, None
    planes.update({
        "k_field_bytes": (4 if repr_l == "bitmap" else (7 * k + 7) // 8) if k > 0 else 0,
        "req_to_token": torch.arange(pages, dtype=torch.int32, device=device).reshape(1, pages),
        "req_to_group": torch.arange(G, dtype=torch.int32, device=device).reshape(1, G),
        "head_dim": D, "n_kv_heads": H, "num_tokens": T, "n_groups": G, "page_size": int(page_size),
        "outliers_per_vector": k, "outlier_repr": repr_l, "outlier_select": str(outlier_select).lower(),
        "group_tokens": gt, "group_channels": gc, "k_format": kfmt, "v_format": vfmt,
        "k_base_bits": 2, "oval_bits": 4, "use_pow2": bool(use_pow2),
        "kv_outlier_map": use_map, "kv_int8_scale": use_int8,
    })
    return planes


__all__ = ["CANONICAL_GROUP_TOKENS", "CANONICAL_GROUP_CHANNELS", "OUTLIER_REPRS",
           "ommx_pack_kv_canonical_block", "ommx_pack_kv_into", "alloc_planes", "planes_struct"]
