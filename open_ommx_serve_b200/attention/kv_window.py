"""Sink / packed-prefix / recent-tail arithmetic of the OMMX KV layout (host integers only).

Same names and meaning as the reference module ``ommx_gpu_serve/attention/kv_window.py``
(:35-141).  A sequence of ``seq`` tokens is served from three places:

    [0, sink)             bf16 rows (attention sink)
    [sink, boundary)      quantized planes, a whole number of ``group_tokens``-token groups
    [boundary, seq)       bf16 rows (recent window plus the group still filling up)

``boundary`` depends on ``seq`` alone, so no per-request state can drift.
"""
from __future__ import annotations

from dataclasses import dataclass

CANONICAL_GROUP_TOKENS = 32


def packed_boundary(seq_len: int, sink_tokens: int, recent_window: int,
                    group_tokens: int = CANONICAL_GROUP_TOKENS) -> int:
    """First token index after the quantized prefix."""
    seq_len, sink_tokens = int(seq_len), int(sink_tokens)
    recent_window, group_tokens = int(recent_window), int(group_tokens)
    if group_tokens <= 0:
        raise ValueError(f"group_tokens must be > 0; got {group_tokens}")
    spare = seq_len - sink_tokens - recent_window
    if spare <= 0:
        return min(sink_tokens, seq_len)
    return sink_tokens + spare // group_tokens * group_tokens


def packed_len(seq_len, sink_tokens, recent_window, group_tokens=CANONICAL_GROUP_TOKENS) -> int:
    """Quantized tokens (a multiple of ``group_tokens``)."""
    return max(0, packed_boundary(seq_len, sink_tokens, recent_window, group_tokens) - int(sink_tokens))


def num_packed_groups(seq_len, sink_tokens, recent_window, group_tokens=CANONICAL_GROUP_TOKENS) -> int:
    return packed_len(seq_len, sink_tokens, recent_window, group_tokens) // int(group_tokens)


def newly_completed_groups(prev_seq_len, new_seq_len, sink_tokens, recent_window,
                           group_tokens=CANONICAL_GROUP_TOKENS) -> int:
    """Groups that became packable when the sequence grew from ``prev`` to ``new`` tokens."""
    before = num_packed_groups(prev_seq_len, sink_tokens, recent_window, group_tokens)
    after = num_packed_groups(new_seq_len, sink_tokens, recent_window, group_tokens)
    return max(0, after - before)


def tail_token_indices(seq_len, sink_tokens, recent_window, group_tokens=CANONICAL_GROUP_TOKENS):
    """Token indices kept in bf16: the sink first, then everything from the boundary on."""
    seq_len, sink_tokens = int(seq_len), int(sink_tokens)
    edge = packed_boundary(seq_len, sink_tokens, recent_window, group_tokens)
    return [*range(min(sink_tokens, seq_len)), *range(edge, seq_len)]


def sink_page_shift(sink_tokens: int, page_size: int) -> int:
    return int(sink_tokens) // max(1, int(page_size))


def sink_token_offset(sink_tokens: int, page_size: int) -> int:
    return int(sink_tokens) % max(1, int(page_size))


@dataclass(frozen=True)
class WindowSpec:
    """The four constants of the residual window, with the helpers bound to them."""

    sink_tokens: int = 8
    recent_window: int = 32
    group_tokens: int = CANONICAL_GROUP_TOKENS
    page_size: int = 16

    def boundary(self, seq_len: int) -> int:
        return packed_boundary(seq_len, self.sink_tokens, self.recent_window, self.group_tokens)

    def packed_len(self, seq_len: int) -> int:
        return packed_len(seq_len, self.sink_tokens, self.recent_window, self.group_tokens)

    def num_groups(self, seq_len: int) -> int:
        return num_packed_groups(seq_len, self.sink_tokens, self.recent_window, self.group_tokens)

    def newly_completed_groups(self, prev_seq_len: int, new_seq_len: int) -> int:
        return newly_completed_groups(prev_seq_len, new_seq_len, self.sink_tokens,
                                      self.recent_window, self.group_tokens)

    def tail_indices(self, seq_len: int):
        return tail_token_indices(seq_len, self.sink_tokens, self.recent_window, self.group_tokens)

    def packed_start_offset(self) -> int:
        return sink_token_offset(self.sink_tokens, self.page_size)

    def sink_page_shift(self) -> int:
        return sink_page_shift(self.sink_tokens, self.page_size)

    def max_tail_len(self, max_seq_len: int = 0) -> int:
        """Most bf16 rows a request can hold: sink + recent + one group still filling."""
        return int(self.sink_tokens) + int(self.recent_window) + int(self.group_tokens)


__all__ = ["CANONICAL_GROUP_TOKENS", "WindowSpec", "packed_boundary", "packed_len",
           "num_packed_groups", "newly_completed_groups", "tail_token_indices",
           "sink_page_shift", "sink_token_offset"]
