"""Host arithmetic of the residual window (reference: attention/kv_window.py)."""
import pytest

from open_ommx_serve_b200.attention import kv_window as W


def test_boundary_invariants():
    spec = W.WindowSpec()
    for seq in range(0, 400):
        b = spec.boundary(seq)
        assert b <= seq or seq < 8
        assert (b - 8) % 32 == 0 or b == min(8, seq)
        if seq >= 40:
            assert 32 <= seq - b < 64
        assert spec.packed_len(seq) == max(0, b - 8)
        assert len(spec.tail_indices(seq)) == seq - spec.packed_len(seq)
    assert spec.max_tail_len(0) == 72


def test_known_values():
    assert W.packed_len(4096, 8, 32) == 4032
    assert W.packed_len(65536, 8, 32) == 65472
    assert W.packed_len(71, 8, 32) == 0 and W.packed_len(72, 8, 32) == 32
    assert W.newly_completed_groups(71, 72, 8, 32) == 1
    assert W.newly_completed_groups(72, 103, 8, 32) == 0
    assert W.sink_token_offset(8, 16) == 8 and W.sink_page_shift(40, 16) == 2
    with pytest.raises(ValueError):
        W.packed_boundary(10, 8, 32, 0)
