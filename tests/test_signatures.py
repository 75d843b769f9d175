"""Drop-in check: every mirrored function and method takes the reference's parameters, by name and
order.  Runs when the reference package is importable (baseline/_ref, built by oracle/build_ref.py
next to a reference checkout); skipped otherwise.  Extra trailing keyword parameters with defaults
are allowed on this side (status words and the like); nothing the reference accepts may be missing."""
import inspect
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _ref():
    if not os.path.isdir(os.path.join(REF, "ommx_gpu_serve")):
        pytest.skip("baseline/_ref is not built")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import ommx_gpu_serve.attention as ra
    return ra


def _params(fn):
    return [p for p in inspect.signature(fn).parameters.values() if p.name != "self"]


def _assert_accepts(ours, theirs, what):
    mine = {p.name: p for p in _params(ours)}
    ref = _params(theirs)
    for p in ref:
        assert p.name in mine, f"{what}: parameter {p.name!r} of the reference is missing"
        q = mine[p.name]
        pos_ok = q.kind == p.kind or (p.kind == p.KEYWORD_ONLY and q.kind in (q.KEYWORD_ONLY, q.POSITIONAL_OR_KEYWORD))
        assert pos_ok, f"{what}: {p.name!r} is {q.kind.description} here, {p.kind.description} in the reference"
    positional = [p.name for p in ref if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    mine_pos = [p.name for p in _params(ours) if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    assert mine_pos[:len(positional)] == positional, f"{what}: positional order {mine_pos} vs {positional}"
    for name, p in mine.items():
        if name not in {r.name for r in ref}:
            assert p.default is not inspect.Parameter.empty, f"{what}: extra parameter {name!r} needs a default"


def test_function_signatures():
    ra = _ref()
    import open_ommx_serve_b200.attention as oa
    from ommx_gpu_serve.attention import paged_decode as rp, pack as rk, kv_window as rw
    from open_ommx_serve_b200.attention import paged_decode as op, pack as ok, kv_window as ow
    for name in ("ommx_paged_decode_attention_canonical", "merge_attention_states", "is_available",
                 "_auto_num_kv_splits", "launch_stats", "reset_launch_stats", "abl_flag_names",
                 "active_recipe_altering_env"):
        _assert_accepts(getattr(op, name), getattr(rp, name), name)
    _assert_accepts(ok.ommx_pack_kv_canonical_block, rk.ommx_pack_kv_canonical_block, "ommx_pack_kv_canonical_block")
    for name in ("packed_boundary", "WindowSpec"):
        _assert_accepts(getattr(ow, name), getattr(rw, name), name)
    for name in ("ommx_paged_decode_attention_canonical", "merge_attention_states", "is_available",
                 "ommx_pack_kv_canonical_block"):
        assert hasattr(oa, name) and hasattr(ra, name)


@pytest.mark.parametrize("cls,methods", [
    ("MultiSeqKVPool", ["__init__", "append_block", "append", "append_decode_batched", "append_decode_device",
                        "append_decode_captured", "regroup", "pool_planes", "request_planes", "tail_bf16_batched",
                        "decode_inputs_captured", "decode_inputs_batched", "decode_seed_seq_device",
                        "advance_seq_device", "decode_inputs_device"]),
    ("CanonicalKVStore", ["__init__", "reset_inplace", "append", "write_token", "advance_to", "gather_tail_into",
                          "append_block", "maybe_regroup", "decode_planes", "decode_planes_full", "tail_bf16",
                          "decode_inputs"]),
])
def test_class_method_signatures(cls, methods):
    _ref()
    import importlib
    mod = "kv_pool" if cls == "MultiSeqKVPool" else "kv_store"
    theirs = getattr(importlib.import_module("ommx_gpu_serve.attention." + mod), cls)
    ours = getattr(importlib.import_module("open_ommx_serve_b200.attention." + mod), cls)
    for m in methods:
        _assert_accepts(getattr(ours, m), getattr(theirs, m), f"{cls}.{m}")
