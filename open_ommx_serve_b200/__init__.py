"""B200-native OMMX paged decode attention (sm_100a CUDA behind the reference's Python surface).

Drop-in for the hot path of Youngmin17/open_ommx_serve: the KV quantize/pack store, the split-KV
decode attention and its log-sum-exp combine.  ``attention.pack`` / ``attention.paged_decode`` /
``attention.kv_window`` mirror the reference modules of the same names under
``ommx_gpu_serve/attention/``.
"""
from .attention.kv_window import WindowSpec, packed_boundary  # noqa: F401
from .attention.pack import ommx_pack_kv_canonical_block, ommx_pack_kv_into  # noqa: F401
from .attention.paged_decode import (  # noqa: F401
    ommx_paged_decode_attention_canonical, merge_attention_states, is_available,
    launch_stats, reset_launch_stats)

__all__ = [
    "ommx_pack_kv_canonical_block", "ommx_pack_kv_into", "ommx_paged_decode_attention_canonical",
    "merge_attention_states", "is_available", "launch_stats", "reset_launch_stats",
    "WindowSpec", "packed_boundary",
]
