"""ctypes binding of libommx_b200.so (the C ABI declared in include/ommx_b200.h).

There is no fallback: if the library is missing or cannot be loaded, every entry point of the
package raises ``RuntimeError``.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libommx_b200.so")

OMMX_DT_F32, OMMX_DT_BF16, OMMX_DT_F16 = 0, 1, 2
OMMX_SCALE_INT8_EXP, OMMX_SCALE_BF16, OMMX_SCALE_F32 = 0, 1, 2
OMMX_OIDX_BITMASK, OMMX_OIDX_RELIDX7 = 0, 1
ST_BAD_PAGE, ST_BAD_GROUP, ST_NONFINITE, ST_TIMEOUT, ST_BAD_LENGTH, ST_SCALE_RANGE = 1, 2, 4, 8, 16, 32
STATUS_NAMES = {ST_BAD_PAGE: "page id out of range", ST_BAD_GROUP: "group slot out of range",
                ST_NONFINITE: "non-finite K/V value", ST_TIMEOUT: "a bounded device wait ran out",
                ST_BAD_LENGTH: "a split holds more groups than one CTA can index",
                ST_SCALE_RANGE: "a scale exponent above 11 was clamped"}


class KVPlanes(C.Structure):
    _fields_ = [("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("page_size", C.c_int32),
                ("num_pages", C.c_int32), ("num_group_slots", C.c_int32),
                ("outliers_per_vector", C.c_int32), ("kv_outlier_map", C.c_int32),
                ("scale_kind", C.c_int32),
                ("k_base", C.c_void_p), ("k_scale", C.c_void_p), ("k_zp", C.c_void_p),
                ("k_obmp", C.c_void_p), ("k_oval", C.c_void_p), ("k_mapscale", C.c_void_p),
                ("k_mapcenter", C.c_void_p), ("v_main", C.c_void_p), ("v_scale", C.c_void_p),
                ("v_zp", C.c_void_p), ("outlier_index", C.c_int32)]


class PackArgs(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("in_dtype", C.c_int32),
                ("num_tokens", C.c_int32), ("stride_token", C.c_int64), ("stride_head", C.c_int64),
                ("dst_pages", C.c_void_p), ("dst_groups", C.c_void_p),
                ("outlier_select", C.c_int32), ("use_pow2", C.c_int32),
                ("planes", KVPlanes), ("status", C.c_void_p)]


class HeadGather(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("recv", C.c_void_p), ("out", C.c_void_p), ("state", C.c_void_p)]


class DecodeArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_dtype", C.c_int32), ("batch", C.c_int32), ("n_q_heads", C.c_int32),
                ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64),
                ("planes", KVPlanes),
                ("k_tail", C.c_void_p), ("v_tail", C.c_void_p),
                ("tail_stride_b", C.c_int64), ("tail_stride_t", C.c_int64), ("tail_stride_h", C.c_int64),
                ("b_tail_len", C.c_void_p), ("b_seq_len", C.c_void_p),
                ("req_to_token", C.c_void_p), ("req_to_group", C.c_void_p), ("table_is_int64", C.c_int32),
                ("r2t_stride_b", C.c_int64), ("r2g_stride_b", C.c_int64),
                ("o", C.c_void_p), ("o_dtype", C.c_int32), ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64),
                ("lse", C.c_void_p), ("lse_stride_b", C.c_int64),
                ("attn_logits", C.c_void_p),
                ("al_stride_b", C.c_int64), ("al_stride_h", C.c_int64), ("al_stride_s", C.c_int64),
                ("num_kv_splits", C.c_int32), ("max_seq_len", C.c_int32), ("max_tail_len", C.c_int32),
                ("seg_group_base", C.c_int32), ("packed_start_offset", C.c_int32),
                ("sm_scale", C.c_float), ("logit_cap", C.c_float), ("status", C.c_void_p),
                ("abl_flags", C.c_int32), ("gather", C.c_void_p)]


class KVPool(C.Structure):
    _fields_ = [("planes", KVPlanes), ("k_hist", C.c_void_p), ("v_hist", C.c_void_p),
                ("num_seqs", C.c_int32), ("ring_cap", C.c_int32),
                ("sink_tokens", C.c_int32), ("recent_window", C.c_int32),
                ("seq_len", C.c_void_p), ("req_to_token", C.c_void_p), ("req_to_group", C.c_void_p),
                ("pages_per_seq", C.c_int32), ("groups_per_seq", C.c_int32)]


class KVAppendArgs(C.Structure):
    _fields_ = [("pool", KVPool), ("k_new", C.c_void_p), ("v_new", C.c_void_p),
                ("new_stride_b", C.c_int64), ("new_stride_h", C.c_int64),
                ("slots", C.c_void_p), ("batch", C.c_int32), ("advance", C.c_int32),
                ("outlier_select", C.c_int32), ("use_pow2", C.c_int32),
                ("k_tail", C.c_void_p), ("v_tail", C.c_void_p), ("max_tail", C.c_int32),
                ("b_seq_len", C.c_void_p), ("b_tail_len", C.c_void_p), ("status", C.c_void_p),
                ("write_pos", C.c_void_p), ("index_is_int64", C.c_int32)]


#: every symbol include/ommx_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "ommx_b200_pack_kv": (C.c_int, [C.POINTER(PackArgs), C.c_void_p]),
    "ommx_b200_outlier_index_convert": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "ommx_b200_decode": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "ommx_b200_decode_stage1": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "ommx_b200_decode_stage2": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "ommx_b200_decode_static_ws": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "ommx_b200_kv_append_decode": (C.c_int, [C.POINTER(KVAppendArgs), C.c_void_p]),
    "ommx_b200_kv_gather_tail": (C.c_int, [C.POINTER(KVPool), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                           C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ommx_b200_peer_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]),
    "ommx_b200_peer_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "ommx_b200_peer_close": (C.c_int, [C.c_void_p]),
    "ommx_b200_peer_free": (C.c_int, [C.c_void_p]),
    "ommx_b200_auto_num_kv_splits": (C.c_int, [C.c_int32, C.c_int32, C.c_int32]),
    "ommx_b200_min_num_kv_splits": (C.c_int, [C.c_int32, C.c_int32]),
    "ommx_b200_merge_states": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ommx_b200_host_pow2_exponent": (C.c_int, [C.c_float]),
    "ommx_b200_host_fp4_encode": (C.c_int, [C.c_float]),
    "ommx_b200_abi_version": (C.c_int, []),
    "ommx_b200_last_error": (C.c_char_p, []),
    "ommx_b200_launch_count": (C.c_int64, []),
    "ommx_b200_reset_launch_count": (None, []),
}

_LIB = None


def load():
    """Load the shared library once; raise ``RuntimeError`` when it is not there."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m open_ommx_serve_b200.build` "
            "(nvcc, sm_100a). There is no CPU or Triton fallback.")
    try:
        lib = C.CDLL(LIB_PATH)
    except OSError as e:  # pragma: no cover - depends on the host
        raise RuntimeError(f"cannot load {LIB_PATH}: {e}") from e
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def last_error() -> str:
    return load().ommx_b200_last_error().decode("utf-8", "replace")


def check(rc: int, what: str):
    """Map a negative C return code onto the exception the reference raises for that case."""
    if rc == 0:
        return
    msg = f"{what}: {last_error()}"
    if rc == -2:
        raise NotImplementedError(msg)
    if rc == -1:
        raise ValueError(msg)
    raise RuntimeError(msg)


def status_text(bits: int) -> str:
    return ", ".join(v for k, v in STATUS_NAMES.items() if bits & k) or "ok"
