"""The allocation-free decode entry point (``ommx_b200_decode_static_ws``).

Some callers cannot allocate device memory on their serving path - an engine that froze its
memory pool after start-up, a plug-in that is given buffers but no allocator.  For them the
library carries its own 8 MiB split workspace.  This test drives that entry point through the C
ABI and holds it to the ordinary entry point: same inputs, same split count, twice in a row
(the workspace is shared and keeps the previous call's contents, so the second call proves
nothing stale leaks in).  The two paths launch the same kernels, so the match is exact.
"""
import pytest
import torch

from helpers import Case

pytestmark = pytest.mark.gpu


def test_static_workspace_matches_caller_workspace_twice():
    case = Case([3000, 500, 72, 9000], seed=91)
    want_o, want_lse = case.run(num_kv_splits=37)
    for call in range(2):
        o, lse = case.run(num_kv_splits=37, static_workspace=True)
        assert torch.isfinite(o).all(), f"call {call}"
        assert (o - want_o).abs().max().item() <= 1e-6, f"call {call}"
        assert (lse - want_lse).abs().max().item() <= 1e-6, f"call {call}"
    # a different problem right after: nothing of the previous contents may show
    other = Case([5000], seed=92, H=2, Hq=8)
    want_o, want_lse = other.run(num_kv_splits=148)
    o, lse = other.run(num_kv_splits=148, static_workspace=True)
    assert (o - want_o).abs().max().item() <= 1e-6 and (lse - want_lse).abs().max().item() <= 1e-6


def test_static_workspace_rejects_oversize():
    case = Case([2000], seed=93)
    # 1 * 32 heads * 600 splits * 129 floats = 2.48 M floats > 2 Mi
    with pytest.raises(ValueError, match="built-in workspace"):
        case.run(num_kv_splits=600, static_workspace=True)
