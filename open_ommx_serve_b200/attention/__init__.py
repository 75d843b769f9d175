"""Mirror of the reference package ``ommx_gpu_serve.attention`` for the decode hot path."""
from .kv_pool import MultiSeqKVPool  # noqa: F401
from .kv_window import WindowSpec, packed_boundary  # noqa: F401
from .pack import ommx_pack_kv_canonical_block, ommx_pack_kv_into  # noqa: F401
from .paged_decode import (  # noqa: F401
    ommx_paged_decode_attention_canonical, merge_attention_states, is_available)

__all__ = ["ommx_paged_decode_attention_canonical", "merge_attention_states", "is_available",
           "ommx_pack_kv_canonical_block", "ommx_pack_kv_into", "WindowSpec", "packed_boundary",
           "MultiSeqKVPool"]
