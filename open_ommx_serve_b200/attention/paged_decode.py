"""Paged decode attention over OMMX-quantized KV, behind the reference's launcher signature.

Mirrors the public surface of ``ommx_gpu_serve/attention/paged_decode.py`` of the reference:
``ommx_paged_decode_attention_canonical`` (:2768-3549), ``merge_attention_states`` (:3556-3624),
``is_available`` (:118), ``_auto_num_kv_splits`` (:409-461), ``launch_stats`` /
``reset_launch_stats`` (:2728-2739), ``abl_flag_names`` / ``active_recipe_altering_env``
(:2755-2765).  The kernels are hand-written sm_100a CUDA in libommx_b200.so
(csrc/ommx_decode.cu); nothing here computes, and there is no Triton, CPU or eager fallback.

Differences from the reference launcher, all refusals rather than silent changes: the outlier
index must be the flat bitmask (``bitmap_read`` with ``k_obmp``); scales must be the int8
power-of-two exponents; K groups are 32 tokens, V groups 32 channels; head_dim 128; at most 8
query heads per kv head; ``packed_start_offset`` must be 0.  The Triton scheduling knobs
(``num_stages``, ``num_warps``, the ``OMMX_ATTN_*`` environment) are accepted and ignored.
"""
from __future__ import annotations

import os
from typing import Any, Optional

import torch

from .. import _lib
from .pack import planes_struct

_LAUNCHES = {"stage1": 0, "bitmap": 0, "abl": 0}

ABL_FLAG_NAMES = ("OMMX_ABL_NO_OUTLIER", "OMMX_ABL_V_NODEQUANT", "OMMX_ABL_K_NODEQUANT",
                  "OMMX_ABL_NO_UNPACK",          # here bit 3 streams the planes and computes nothing
                  "OMMX_ABL_TEST_STALL")         # tests of the give-up path: short waits, one ring fill announced but not issued
RECIPE_ALTERING_ENV_PREFIXES = ("OMMX_ABL_", "OMMX_W_ABL_")
RECIPE_ALTERING_ENV_KEYS = ("OMMX_ATTN_V_BF16", "OMMX_ATTN_FP8_QK")


def is_available() -> bool:
    """True when the CUDA library loads and a CUDA device is present."""
    try:
        _lib.load()
    except RuntimeError:
        return False
    return bool(torch.cuda.is_available())


def launch_stats() -> dict:
    """Copy of the per-process launch counters (decode calls served, of which bitmap reads)."""
    return dict(_LAUNCHES)


def reset_launch_stats() -> None:
    for key in _LAUNCHES:
        _LAUNCHES[key] = 0


def env_truthy(v) -> bool:
    return v is not None and str(v).strip().lower() not in ("", "0", "false", "off", "no")


def active_recipe_altering_env(environ=None) -> list:
    """Sorted names of the environment keys that would change what a kernel computes."""
    env = os.environ if environ is None else environ
    return sorted(k for k, v in env.items()
                  if (k.startswith(RECIPE_ALTERING_ENV_PREFIXES) or k in RECIPE_ALTERING_ENV_KEYS)
                  and env_truthy(v))


def abl_flag_names(mask: int) -> list:
    return [n for i, n in enumerate(ABL_FLAG_NAMES) if int(mask) & (1 << i)]


def _env_int(name: str, default: int, *, allow_zero: bool = False) -> int:
    """Strict integer read of an environment knob: blank = default, anything malformed raises."""
    raw = os.environ.get(name)
    if raw is None or not str(raw).strip():
        return int(default)
    try:
        val = int(str(raw).strip())
    except ValueError:
        raise ValueError(f"{name}={raw!r} is not an integer (default would be {default})") from None
    if val < 0 or (val == 0 and not allow_zero):
        raise ValueError(f"{name}={raw!r} must be a positive integer (default would be {default})")
    return val


def _auto_num_kv_splits(seq_len: int, batch_size: int, device: Any = None, kv_heads: int = 8) -> int:
    """Split count for (max context, batch): sized so that batch x splits fills the 148 SMs.

    One CTA serves one (split, sequence) with all local kv heads, so ``kv_heads`` does not
    enter.  ``OMMX_ATTN_NUM_KV_SPLITS`` overrides, as in the reference.
    """
    if str(os.environ.get("OMMX_ATTN_NUM_KV_SPLITS") or "").strip():
        return _env_int("OMMX_ATTN_NUM_KV_SPLITS", 1)
    lib = _lib.load()
    if device is not None and torch.device(device).type == "cuda" and torch.cuda.is_available():
        with torch.cuda.device(device):
            return int(lib.ommx_b200_auto_num_kv_splits(int(seq_len), int(batch_size), int(kv_heads)))
    return int(lib.ommx_b200_auto_num_kv_splits(int(seq_len), int(batch_size), int(kv_heads)))


def _make_attn_logits(batch, head_num, num_kv_splits, head_dim, device):
    return torch.empty((batch, head_num, num_kv_splits, head_dim + 1), dtype=torch.float32, device=device)


def _o_dtype(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.OMMX_DT_F32
    if t.dtype == torch.bfloat16:
        return _lib.OMMX_DT_BF16
    raise NotImplementedError(f"o dtype {t.dtype}: float32 or bfloat16")


def ommx_paged_decode_attention_canonical(
    q,
    k_base, k_scale, k_zp, k_oidx, k_oval,
    v_main, v_scale, v_zp,
    k_tail, v_tail, b_tail_len,
    o, lse,
    req_to_token, req_to_group, b_seq_len,
    *,
    sm_scale: float = 1.0,
    page_size: int = 16,
    logit_cap: float = 0.0,
    k_outliers_per_vector: int = 3,
    k_format: str = "i2f4",
    combinadic_read: bool = False,
    k_crank: Any = None,
    bitmap_read: bool = False,
    k_obmp: Any = None,
    k_fp4_mapscale: Any = None,
    k_fp4_mapcenter: Any = None,
    kv_outlier_map: bool = False,
    kv_int8_scale: bool = False,
    num_kv_splits: Optional[int] = None,
    num_stages: Optional[int] = None,
    num_warps: Optional[int] = None,
    max_seq_len: Optional[int] = None,
    max_tail_len: Optional[int] = None,
    attn_logits: Any = None,
    qzp_buf: Any = None,
    packed_start_offset: int = 0,
    seg_group_base: int = 0,
    status: Any = None,
    _stage: int = 0,
    static_workspace: bool = False,
    head_gather: Any = None,
) -> None:
    """Decode attention of one query row per sequence. Writes ``o`` / ``lse`` in place.

    Arguments and plane layout are the reference's (``paged_decode.py:2856-2902``): ``q``
    bf16 ``[B,Hq,D]``; page planes ``[pages, page_size, Hkv, .]``; group planes
    ``[group_slots, Hkv, D, .]``; ``k_tail/v_tail`` bf16 ``[B, T_tail, Hkv, D]`` with
    ``b_tail_len`` valid rows; ``req_to_token`` / ``req_to_group`` int32 or int64 tables;
    ``b_seq_len`` packed token counts.  Pass ``max_seq_len``, ``max_tail_len`` and
    ``attn_logits`` (f32 ``[B,Hq,S+1,D+1]``) to avoid every host sync and allocation, which
    is what CUDA-graph capture needs.  ``status`` (int32 ``[1]``, optional, not in the
    reference) collects device-side error bits instead of a trap.  ``_stage`` (1 or 2) runs one
    stage alone, for the benchmark's per-kernel timing.

    ``static_workspace=True`` (not in the reference) is for callers that may not allocate on
    the device while serving, e.g. under an engine whose memory pool is frozen after start-up:
    ``attn_logits`` is neither needed nor created, the split partials go to an 8 MiB array built
    into the library (``ommx_b200_decode_static_ws``).  ``batch * Hq * num_kv_splits * (D+1)`` must
    stay within 2 Mi floats (``ValueError`` beyond); calls that overlap on the GPU share the array
    and race; make the first call on a device outside stream capture.

    ``head_gather`` (not in the reference): the ``(PeerHeadGather, layer)`` plan of a kv-head sharded run
    (``sharding.PeerHeadGather.plan``); stage 2 then also stores this rank's rows into every rank's
    gathered buffer and returns when all ranks' rows of the layer have arrived in this rank's.
    """
    lib = _lib.load()
    if not q.is_cuda:
        raise RuntimeError("ommx_paged_decode_attention_canonical needs CUDA tensors (no CPU path)")
    kfmt = str(k_format).lower()
    if kfmt not in ("i2f4", "itf4"):
        raise ValueError(f"k_format must be i2f4|itf4; got {k_format!r}")
    pages, ngroups = int(k_base.shape[0]), int(k_scale.shape[0])
    if pages and ngroups:
        gt = (pages * int(page_size)) // ngroups
        if gt not in (16, 32, 64, 128):
            raise ValueError(f"derived GROUP_TOKENS={gt} (pages={pages} page_size={page_size} "
                             f"n_group_slots={ngroups}) must be in {{16,32,64,128}}")
        if gt != 32:
            raise NotImplementedError(f"GROUP_TOKENS={gt}: this build serves 32-token K groups")
    vsc = int(v_scale.shape[-1])
    if vsc:
        gc = (int(v_main.shape[-1]) * 4) // vsc
        if gc not in (16, 32, 64, 128):
            raise ValueError(f"derived GROUP_CHANNELS={gc} must be in {{16,32,64,128}}")
        if gc != 32:
            raise NotImplementedError(f"GROUP_CHANNELS={gc}: this build serves 32-channel V groups")
    combinadic_read = bool(combinadic_read) or env_truthy(os.environ.get("OMMX_VLLM_KV_COMBINADIC_READ"))
    bitmap_read = bool(bitmap_read) or env_truthy(os.environ.get("OMMX_VLLM_KV_BITMAP_READ"))
    if bitmap_read and combinadic_read:
        raise ValueError("combinadic_read and bitmap_read are mutually exclusive outlier-index sources.")
    batch, head_num = int(q.shape[0]), int(q.shape[1])
    n_kv_heads = int(k_base.shape[-2])
    if head_num < n_kv_heads or head_num % n_kv_heads != 0:
        raise NotImplementedError(
            f"q_head_num={head_num} must be an integer multiple of n_kv_heads={n_kv_heads}")
    if int(k_base.shape[1]) != int(page_size):
        raise ValueError(f"k_base is [pages, {k_base.shape[1]}, h, w] but page_size={page_size}")
    for name, t in (("k_base", k_base), ("v_main", v_main), ("v_scale", v_scale), ("v_zp", v_zp)):
        if pages and (t.stride(0) != int(page_size) * t.stride(1) or t.stride(-1) != 1):
            raise ValueError(f"{name} must be a contiguous [pages, page_size, h, w] plane")
    start_offset = int(packed_start_offset or 0)
    if start_offset < 0 or start_offset >= int(page_size):
        raise ValueError(f"packed_start_offset={start_offset} must be in [0, page_size={page_size})")
    seg_group_base = int(seg_group_base or 0)
    if seg_group_base < 0:
        raise ValueError(f"seg_group_base={seg_group_base} must be >= 0")
    k = int(k_outliers_per_vector)
    if k > 0 and k_oval is None:
        raise ValueError("k_outliers_per_vector > 0 requires the k_oval sidecar plane.")
    if bitmap_read and k > 0 and k_obmp is None:
        raise ValueError("bitmap_read=True requires the k_obmp flat-bitmask plane (pack with "
                         "ommx_pack_kv_canonical_block(..., outlier_repr='bitmap')).")
    # The reference's bitmask read stops at k = 8 (its value stream must fit one 32-bit word,
    # paged_decode.py:3055-3058); this kernel walks a 64-bit stream, so the 32-bit bitmask serves k <= 16.
    if bitmap_read and k > 16:
        raise ValueError(f"bitmap_read holds the k_oval stream in two 32-bit words, i.e. k <= 16; got k={k}.")
    relidx7_read = k > 0 and not bitmap_read
    if relidx7_read and combinadic_read:
        raise NotImplementedError("combinadic rank planes are not served: derive relidx7 planes at load time "
                                  "(the reference's derive_relidx7_from_combinadic) or pack with outlier_repr='bitmap'")
    if relidx7_read and k_oidx is None:
        raise ValueError("k_outliers_per_vector > 0 without bitmap_read requires the k_oidx (relidx7) sidecar plane.")
    if relidx7_read and k > 16:
        raise ValueError(f"the relidx7 read path serves k <= 16; got k={k}.")
    use_map = bool(kv_outlier_map) and k > 0
    if use_map and (k_fp4_mapscale is None or k_fp4_mapcenter is None):
        raise ValueError("kv_outlier_map=True requires k_fp4_mapscale + k_fp4_mapcenter planes.")
    if max_seq_len is not None:
        max_seq = max(1, int(max_seq_len)) if pages else 0
    else:
        max_seq = int(b_seq_len.max().item()) if int(b_seq_len.numel()) > 0 else 0
    if max_tail_len is not None:
        max_tail = int(max_tail_len)
    else:
        max_tail = int(b_tail_len.max().item()) if (b_tail_len is not None and int(b_tail_len.numel()) > 0) else 0
    D = int(v_main.shape[-1]) * 4
    if num_kv_splits is None:
        num_kv_splits = _auto_num_kv_splits(max(max_seq, 1), batch, device=q.device, kv_heads=n_kv_heads)
    num_kv_splits = max(1, int(num_kv_splits))
    if static_workspace:
        if int(_stage) != 0:
            raise ValueError("static_workspace=True runs both stages on the library's own workspace; _stage must be 0")
        attn_logits = None
    else:
        if attn_logits is None:
            attn_logits = _make_attn_logits(batch, head_num, num_kv_splits + 1, D, q.device)
        if attn_logits.dtype != torch.float32 or attn_logits.device != q.device or attn_logits.dim() != 4:
            raise ValueError("attn_logits must be a float32 [batch, heads, splits, head_dim+1] tensor on q's device")
        if int(attn_logits.shape[0]) < batch or int(attn_logits.shape[1]) < head_num:
            raise ValueError(f"attn_logits {tuple(attn_logits.shape)} is smaller than batch={batch} x heads={head_num}")
        if int(attn_logits.shape[-1]) != D + 1 or attn_logits.stride(-1) != 1:
            raise ValueError(f"attn_logits last dim must be head_dim+1={D + 1} and contiguous")
        if int(attn_logits.shape[2]) < num_kv_splits:
            raise ValueError(f"attn_logits holds {attn_logits.shape[2]} split slots, fewer than num_kv_splits={num_kv_splits}")
    if o.dim() != 3 or int(o.shape[0]) < batch or int(o.shape[1]) < head_num or int(o.shape[2]) != D:
        raise ValueError(f"o must be [batch>={batch}, heads>={head_num}, {D}]; got {tuple(o.shape)}")
    if lse.dim() != 2 or int(lse.shape[0]) < batch or int(lse.shape[1]) < head_num or lse.stride(1) != 1:
        raise ValueError(f"lse must be [batch>={batch}, heads>={head_num}] with a unit last stride; got {tuple(lse.shape)}")
    for name, t in (("o", o), ("lse", lse), ("b_seq_len", b_seq_len), ("req_to_token", req_to_token), ("req_to_group", req_to_group),
                    ("k_tail", k_tail), ("v_tail", v_tail), ("b_tail_len", b_tail_len)):
        if t is not None and t.device != q.device:
            raise ValueError(f"{name} is on {t.device}, q on {q.device}")
    if q.dtype != torch.bfloat16:
        raise NotImplementedError(f"q dtype {q.dtype}: this build serves bfloat16 queries")
    if q.stride(-1) != 1 or o.stride(-1) != 1:
        raise ValueError("q and o must have a unit last stride")
    tables64 = req_to_token.dtype == torch.int64
    if req_to_token.dtype not in (torch.int32, torch.int64) or req_to_group.dtype != req_to_token.dtype:
        raise ValueError("req_to_token / req_to_group must both be int32 or both int64")
    if b_seq_len.dtype != torch.int32 or (b_tail_len is not None and b_tail_len.dtype != torch.int32):
        raise ValueError("b_seq_len / b_tail_len must be int32")

    a = _lib.DecodeArgs()
    a.q, a.q_dtype, a.batch, a.n_q_heads = q.data_ptr(), _lib.OMMX_DT_BF16, batch, head_num
    a.q_stride_b, a.q_stride_h = int(q.stride(0)), int(q.stride(1))
    planes = {"k_base": k_base, "k_scale": k_scale, "k_zp": k_zp, "k_obmp": k_obmp if (k > 0 and bitmap_read) else None,
              "k_oidx": k_oidx if relidx7_read else None,
              "k_oval": k_oval if k > 0 else None,
              "k_fp4_mapscale": k_fp4_mapscale if use_map else None,
              "k_fp4_mapcenter": k_fp4_mapcenter if use_map else None,
              "v_main": v_main, "v_scale": v_scale, "v_zp": v_zp}
    a.planes = planes_struct(planes, k=k, outlier_map=use_map, relidx7=relidx7_read)
    if max_tail > 0:
        if k_tail is None or v_tail is None or b_tail_len is None:
            raise ValueError("max_tail_len > 0 needs k_tail, v_tail and b_tail_len")
        if k_tail.dtype != torch.bfloat16 or v_tail.dtype != torch.bfloat16:
            raise NotImplementedError("k_tail / v_tail must be bfloat16")
        if k_tail.stride() != v_tail.stride() or k_tail.stride(-1) != 1:
            raise ValueError("k_tail and v_tail must share strides, with a unit last stride")
        a.k_tail, a.v_tail = k_tail.data_ptr(), v_tail.data_ptr()
        a.tail_stride_b, a.tail_stride_t, a.tail_stride_h = (int(s) for s in k_tail.stride()[:3])
        a.b_tail_len = b_tail_len.data_ptr()
    a.b_seq_len = b_seq_len.data_ptr()
    a.req_to_token, a.req_to_group = req_to_token.data_ptr(), req_to_group.data_ptr()
    a.table_is_int64 = 1 if tables64 else 0
    a.r2t_stride_b, a.r2g_stride_b = int(req_to_token.stride(0)), int(req_to_group.stride(0))
    a.o, a.o_dtype = o.data_ptr(), _o_dtype(o)
    a.o_stride_b, a.o_stride_h = int(o.stride(0)), int(o.stride(1))
    a.lse, a.lse_stride_b = lse.data_ptr(), int(lse.stride(0))
    if lse.dtype != torch.float32:
        raise ValueError("lse must be float32")
    if attn_logits is not None:
        a.attn_logits = attn_logits.data_ptr()
        a.al_stride_b, a.al_stride_h, a.al_stride_s = (int(s) for s in attn_logits.stride()[:3])
    a.num_kv_splits, a.max_seq_len, a.max_tail_len = num_kv_splits, max_seq, max_tail
    a.seg_group_base, a.packed_start_offset = seg_group_base, start_offset
    a.sm_scale, a.logit_cap = float(sm_scale), float(logit_cap)
    a.status = None if status is None else status.data_ptr()
    # ablation knobs (differential timing only; recorded so a leaked export cannot pass as served)
    abl = sum(1 << i for i, n in enumerate(ABL_FLAG_NAMES) if env_truthy(os.environ.get(n)))
    a.abl_flags = abl
    if head_gather is not None:
        if int(_stage) == 1:
            raise ValueError("head_gather belongs to stage 2; _stage=1 runs stage 1 alone")
        a.gather = head_gather.check(batch, head_num, D, q.device)
    _LAUNCHES["abl"] |= abl
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        if static_workspace:
            entry, what = lib.ommx_b200_decode_static_ws, "ommx_b200_decode_static_ws"
        else:
            entry = (lib.ommx_b200_decode, lib.ommx_b200_decode_stage1, lib.ommx_b200_decode_stage2)[int(_stage)]
            what = "ommx_b200_decode"
        _lib.check(entry(a, stream), what)
    _LAUNCHES["stage1"] += 1
    if bitmap_read:
        _LAUNCHES["bitmap"] += 1


def merge_attention_states(o_parts, lse_parts, *, valid_lens=None, out=None, lse_out=None):
    """Merge ``P`` partial softmax states over disjoint KV segments: ``[P,R,D]``, ``[P,R]`` -> ``[R,D]``, ``[R]``.

    ``m = max_p lse_p; w_p = exp(lse_p - m); o = sum w_p o_p / sum w_p; lse = m + log sum w_p``.
    ``valid_lens`` int ``[R]`` limits the parts of a row to its first ``valid_lens[r]`` (negative =
    all).  Same contract as the reference (``paged_decode.py:3556-3624``).
    """
    lib = _lib.load()
    if o_parts.dim() != 3:
        raise ValueError(f"o_parts must be [P, R, D]; got shape {tuple(o_parts.shape)}. "
                         "Reshape any [P, ..., D] structure to a flat row axis R first.")
    if lse_parts.dim() != 2 or tuple(lse_parts.shape) != tuple(o_parts.shape[:2]):
        raise ValueError(f"lse_parts must be [P, R] matching o_parts[:2]; got "
                         f"{tuple(lse_parts.shape)} vs {tuple(o_parts.shape[:2])}.")
    if not o_parts.is_cuda:
        raise RuntimeError("merge_attention_states needs CUDA tensors (no CPU path)")
    P, R, D = (int(s) for s in o_parts.shape)
    op = o_parts.contiguous().to(torch.float32)
    lp = lse_parts.contiguous().to(torch.float32)
    res = torch.empty(R, D, dtype=torch.float32, device=o_parts.device)
    if lse_out is None:
        lse_out = torch.empty(R, dtype=torch.float32, device=o_parts.device)
    elif (lse_out.dtype != torch.float32 or lse_out.device != o_parts.device or not lse_out.is_contiguous()
          or int(lse_out.numel()) != R):
        raise ValueError(f"lse_out must be a contiguous float32 tensor of {R} entries on {o_parts.device}")
    if out is not None and (tuple(out.shape) != (R, D) or out.device != o_parts.device):
        raise ValueError(f"out must be [R={R}, D={D}] on {o_parts.device}; got {tuple(out.shape)} on {out.device}")
    valid = None
    if valid_lens is not None:
        valid = valid_lens.to(device=o_parts.device, dtype=torch.int32).contiguous()
        if int(valid.numel()) != R:
            raise ValueError(f"valid_lens must have R={R} entries; got {valid.numel()}.")
    with torch.cuda.device(o_parts.device):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.ommx_b200_merge_states(op.data_ptr(), lp.data_ptr(),
                                              None if valid is None else valid.data_ptr(),
                                              P, R, D, res.data_ptr(), lse_out.data_ptr(), stream),
                   "ommx_b200_merge_states")
    if out is None:
        out = res.to(o_parts.dtype)
    else:
        out.copy_(res)
    return out, lse_out


__all__ = ["ommx_paged_decode_attention_canonical", "merge_attention_states", "is_available"]
