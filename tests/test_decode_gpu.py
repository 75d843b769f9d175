"""CUDA decode attention (stage 1 + stage 2) vs the CPU oracle.

Gate: max-abs <= 2e-2 and cosine >= 0.9999 against fp32 attention over the dequantized cache
(the reference's own gate is cos >= 0.999, rel-L2 <= 0.02: tests/test_decode_kernel_parity.py).
"""
import numpy as np
import pytest
import torch

from oracle import ommx_oracle as O
from helpers import Case, check_close, check_fp32, load_golden

pytestmark = pytest.mark.gpu


def _run_and_check(case, **kw):
    """Two gates: (1) max-abs 2e-2 / cosine 0.9999 against the reference kernel's arithmetic
    restated on CPU (its bf16 rounding points kept); (2) the reference's own kernel-vs-fp32
    gate, cosine 0.999 / rel-L2 0.02, against fp64 attention over the dequantized cache."""
    lse_atol = kw.pop("lse_atol", 2e-2)
    max_abs = kw.pop("max_abs", 2e-2)
    lse_atol_fp32 = kw.pop("lse_atol_fp32", 5e-2)
    o, lse = case.run(**kw)
    ctx = str(case.seq_lens[:6])
    # every GQA width runs the reference's split-PV arithmetic (exact code*scale products, zero-point bias
    # summed apart)
    want_o, want_lse = case.oracle_kernel_arith(num_kv_splits=int(kw.get("num_kv_splits") or 1), split_pv=True)
    check_close(o, want_o, max_abs=max_abs, ctx="kernel-arith " + ctx)
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=lse_atol, rtol=0)
    f_o, f_lse = case.oracle()
    check_fp32(o, f_o, ctx="fp32 " + ctx)
    # against exact attention the reference's own rounding of q*sm_scale to bf16 shows in lse in proportion to the
    # logit magnitude (|q.k| * 2^-9): a few 1e-2 with the x12 outlier channels, up to ~0.1 at x30
    np.testing.assert_allclose(lse.cpu().numpy(), f_lse, atol=lse_atol_fp32, rtol=0)
    return o, lse


@pytest.mark.parametrize("name", ["attn_seq168", "attn_seq300_gqa8"])
def test_decode_matches_reference_oracle_fixture(name):
    """Output of the reference's fp32 oracle on the committed inputs."""
    g = load_golden(name)
    seq, H, Hq, D, sink, recent = (int(x) for x in g["cfg"])
    K, V, q = (torch.from_numpy(O.bf16_from_bits(g[n])) for n in ("K", "V", "q"))
    case = Case([seq], H=H, Hq=Hq, seed=0, permute=False)
    # overwrite the seeded content with the fixture's tensors
    edge = O.packed_boundary(seq, sink, recent)
    planes = O.pack_kv(K[sink:edge].numpy(), V[sink:edge].numpy())
    from helpers import plane_to_torch, PLANES
    for n in PLANES:
        case.planes[n][: planes[n].shape[0]] = plane_to_torch(n, planes[n], "cuda")
    tail = list(range(sink)) + list(range(edge, seq))
    case.k_tail[0, :len(tail)] = K[tail].bfloat16().cuda()
    case.v_tail[0, :len(tail)] = V[tail].bfloat16().cuda()
    case.q_dev = q.bfloat16()[None].cuda()
    for splits in (1, 2, 5):
        o, _ = case.run(num_kv_splits=splits)
        check_fp32(o[0], g["o"], ctx=f"{name} S={splits}")
        check_close(o[0], g["o"], ctx=f"{name} S={splits}")


@pytest.mark.parametrize("seq", [72, 104, 136, 200, 232, 1024, 4096])
def test_decode_single_sequence(seq):
    _run_and_check(Case([seq], seed=seq))


@pytest.mark.parametrize("splits", [1, 2, 4, 7, 16, 64, 148])
def test_decode_forced_splits(splits):
    _run_and_check(Case([4136], seed=5), num_kv_splits=splits)


def test_decode_16k_auto_splits_and_bf16_output():
    case = Case([16384], seed=42)
    o, _ = _run_and_check(case)
    ob, _ = case.run(o_dtype=torch.bfloat16)
    assert (ob.float() - o).abs().max().item() <= 2e-2


@pytest.mark.parametrize("H,Hq", [(1, 4), (2, 8), (4, 16), (8, 32), (1, 8), (8, 64), (2, 2), (4, 12)])
def test_decode_head_geometries(H, Hq):
    """kv-head shards of 1/2/4/8 heads per device and GQA groups of 1, 3, 4 and 8."""
    _run_and_check(Case([1500], H=H, Hq=Hq, seed=H * 100 + Hq))


@pytest.mark.parametrize("k", [0, 2, 3, 4, 6, 8, 9, 10, 12, 16])
@pytest.mark.parametrize("mag", [4.0, 30.0])
def test_decode_outlier_sweep(k, mag):
    _run_and_check(Case([2048], seed=k + 1, k=k, mag=mag), lse_atol_fp32=5e-2 if mag < 20 else 0.2)


def test_decode_base_shared_outlier_map():
    _run_and_check(Case([1000], seed=3, outlier_map=False))


@pytest.mark.parametrize("ps", [8, 16, 32])
def test_decode_page_sizes(ps):
    _run_and_check(Case([3000], seed=ps, page_size=ps))


def test_decode_ragged_batch_int64_tables():
    lens = [40, 71, 72, 1024, 5000, 333, 8, 2049]
    _run_and_check(Case(lens, seed=11, tables_dtype=torch.int64))


def test_decode_batch32_ragged_partition_512():
    lens = torch.randint(1024, 8193, (32,), generator=torch.Generator().manual_seed(42)).tolist()
    case = Case(lens, seed=12)
    _run_and_check(case, num_kv_splits=(max(case.packed) + 511) // 512)


def test_decode_tail_only_and_empty():
    case = Case([30, 8, 71], seed=2)                 # nothing quantized anywhere
    o, lse = case.run()
    want_o, want_lse = case.oracle()
    check_close(o, want_o, max_abs=1e-4)
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, atol=1e-3)
    # a sequence with no rows at all: o = 0, lse = -inf (reference: paged_decode.py:2393)
    case = Case([200], seed=2)
    case.b_seq_len.zero_()
    case.b_tail_len.zero_()
    o, lse = case.run()
    assert (o == 0).all() and torch.isinf(lse).all() and (lse < 0).all()


def test_decode_page_permutation_is_bit_invariant():
    """Where a page lives must not change a single bit of the result."""
    a = Case([6000, 3000], seed=21, permute=True)
    b = Case([6000, 3000], seed=21, permute=False)
    oa, la = a.run(num_kv_splits=13)
    ob, lb = b.run(num_kv_splits=13)
    assert torch.equal(oa, ob) and torch.equal(la, lb)


def test_decode_is_deterministic_and_workspace_reuse():
    case = Case([9000], seed=8)
    ws = torch.full((1, 32, 149, 129), float("nan"), device="cuda")
    o1, _ = case.run(num_kv_splits=148, attn_logits=ws)
    o2, _ = case.run(num_kv_splits=148, attn_logits=ws)
    assert torch.equal(o1, o2)


def test_decode_64k_split_invariance():
    """Full benchmark size: results agree across split counts and with the oracle."""
    case = Case([65536], seed=42)
    o148, l148 = case.run(num_kv_splits=148)
    o16, l16 = case.run(num_kv_splits=16)
    assert (o148 - o16).abs().max().item() < 5e-3          # bf16 P rounding against different running maxima
    assert (l148 - l16).abs().max().item() < 5e-3
    check_fp32(o148, case.oracle()[0], ctx="64K fp32")
    check_close(o148, case.oracle_kernel_arith(num_kv_splits=16, split_pv=True)[0], ctx="64K kernel-arith")


def test_decode_segments_and_merge_states():
    """seg_group_base partial states merged by merge_attention_states == one full call."""
    from open_ommx_serve_b200 import merge_attention_states
    case = Case([2000], seed=31, permute=True)
    full_o, full_lse = case.run(num_kv_splits=4)
    packed = case.packed[0]
    cut_g = (packed // 32) // 3
    parts_o, parts_l = [], []
    saved_seq, saved_tail = case.b_seq_len.clone(), case.b_tail_len.clone()
    for base, ntok, tail in ((0, cut_g * 32, 0), (cut_g, packed - cut_g * 32, 0), (0, 0, int(saved_tail[0]))):
        case.b_seq_len[0] = ntok
        case.b_tail_len[0] = tail
        o, l = case.run(num_kv_splits=3, seg_group_base=base, max_seq_len=packed, pass_max=False,
                        max_tail_len=72, pass_max_tail=False)
        parts_o.append(o[0])
        parts_l.append(l[0])
    case.b_seq_len.copy_(saved_seq)
    case.b_tail_len.copy_(saved_tail)
    o, l = merge_attention_states(torch.stack(parts_o), torch.stack(parts_l))
    assert (o - full_o[0]).abs().max().item() < 2e-3        # different split boundaries, bf16 P rounding
    assert (l - full_lse[0]).abs().max().item() < 2e-3
    # ragged merge: only the first part counts for row 0
    valid = torch.tensor([1] + [3] * (o.shape[0] - 1), dtype=torch.int32, device="cuda")
    o2, l2 = merge_attention_states(torch.stack(parts_o), torch.stack(parts_l), valid_lens=valid)
    assert torch.allclose(o2[0], parts_o[0][0], atol=1e-6) and torch.allclose(o2[1:], o[1:], atol=1e-6)
    want = O.merge_states(torch.stack(parts_o).cpu().numpy(), torch.stack(parts_l).cpu().numpy())
    np.testing.assert_allclose(o.cpu().numpy(), want[0], atol=1e-5)


def test_decode_logit_cap():
    case = Case([600], seed=4)
    o, _ = case.run(logit_cap=5.0)
    rec = case.per_seq[0]
    Kd, Vd = O.dequant_kv(rec["planes"])
    Kf = np.concatenate([Kd, rec["K"][rec["tail_idx"]].numpy()])
    Vf = np.concatenate([Vd, rec["V"][rec["tail_idx"]].numpy()])
    q = case.q[0].float().numpy()
    want = np.zeros((case.Hq, case.D), dtype=np.float32)
    for h in range(case.Hq):
        s = (Kf[:, h // 4].astype(np.float64) @ q[h]) * case.sm_scale
        s = 5.0 * np.tanh(s / 5.0)
        w = np.exp(s - s.max())
        want[h] = (w[:, None] * Vf[:, h // 4]).sum(0) / w.sum()
    check_fp32(o[0], want, ctx="logit_cap")


def test_decode_status_word_on_bad_tables():
    from open_ommx_serve_b200 import _lib
    case = Case([1000], seed=6)
    case.req_to_token[0, 3] = 10 ** 6
    case.req_to_group[0, 1] = -1
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o, _ = case.run(status=status)
    bits = int(status.item())
    assert bits & _lib.ST_BAD_PAGE and bits & _lib.ST_BAD_GROUP
    assert torch.isfinite(o).all()                  # the access was skipped, nothing trapped


def test_decode_scale_exponent_out_of_fp16_range_is_clamped_and_reported():
    """Scale factors travel as fp16 powers of two: exponents above 11 are clamped and flagged,
    tiny ones (below 2^-18) drop their term; neither traps nor produces a non-finite output."""
    from open_ommx_serve_b200 import _lib
    case = Case([500], seed=12)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o_ref, _ = case.run(status=status)
    assert int(status.item()) == 0
    vs = case.planes["v_scale"]
    vs.view(-1)[5] = 13                              # one V scale step of 2^13
    ks = case.planes["k_scale"]
    ks.view(-1)[7] = -40                             # one K scale step of 2^-40
    o, _ = case.run(status=status)
    assert int(status.item()) & _lib.ST_SCALE_RANGE
    assert torch.isfinite(o).all()


def test_decode_128k_one_kv_head_shard():
    """The 8-way sharded long-context shape: 128K tokens, one local kv head (4 query heads), 8 groups
    in flight per CTA.  Checked through split-count invariance and the fp32 oracle."""
    case = Case([131072], H=1, Hq=4, seed=77)
    o148, l148 = case.run(num_kv_splits=148)
    o32, l32 = case.run(num_kv_splits=32)
    assert (o148 - o32).abs().max().item() < 5e-3
    assert (l148 - l32).abs().max().item() < 5e-3
    check_fp32(o148, case.oracle()[0], ctx="128K fp32")


def test_decode_refusals():
    case = Case([200], seed=1)
    with pytest.raises(NotImplementedError):
        case.run(packed_start_offset=8)
    with pytest.raises(ValueError):
        case.run(attn_logits=torch.zeros(1, 32, 5, 128, device="cuda"), num_kv_splits=4)
    with pytest.raises(ValueError):
        case.run(num_kv_splits=1, max_seq_len=10 ** 6, pass_max=False)
    with pytest.raises(ValueError):
        case.run(seg_group_base=-1)


def test_store_then_decode_end_to_end():
    """CUDA store kernel feeding the CUDA decode kernels (no oracle-made planes in the loop)."""
    from open_ommx_serve_b200 import ommx_pack_kv_canonical_block
    case = Case([3000], seed=77, permute=False)
    rec = case.per_seq[0]
    edge = 8 + case.packed[0]
    out = ommx_pack_kv_canonical_block(rec["K"][8:edge].bfloat16().cuda(), rec["V"][8:edge].bfloat16().cuda(),
                                       outliers_per_vector=6, outlier_repr="bitmap", outlier_select="signed",
                                       use_pow2=True, kv_outlier_map=True, page_size=16)
    for n in case.planes:
        case.planes[n] = out[n]
    case.req_to_token, case.req_to_group = out["req_to_token"], out["req_to_group"]
    o, _ = case.run()
    check_close(o, case.oracle_kernel_arith(split_pv=True)[0], ctx="store->decode")
    from open_ommx_serve_b200 import launch_stats
    assert launch_stats()["stage1"] > 0 and launch_stats()["bitmap"] > 0


@pytest.fixture
def tensor_core_stage1(monkeypatch):
    """Route stage 1 through the tcgen05 kernel (the launcher reads the variable per call)."""
    monkeypatch.setenv("OMMX_B200_STAGE1", "tc")
    yield


@pytest.mark.parametrize("H,Hq,seq,splits", [(8, 32, 4136, None), (8, 32, 16384, 37), (4, 16, 8232, 4), (2, 8, 8232, 16),
                                             (1, 4, 4136, 4), (1, 8, 8232, 8), (2, 16, 3000, None), (4, 12, 1500, None)])
def test_tensor_core_stage1_matches_oracle(tensor_core_stage1, H, Hq, seq, splits):
    """The tcgen05 / tensor-memory stage 1 (opt-in) against the same two gates as the default kernel."""
    _run_and_check(Case([seq], H=H, Hq=Hq, seed=H * 7 + Hq + seq), num_kv_splits=splits)


@pytest.mark.parametrize("k,mag", [(0, 12.0), (2, 4.0), (6, 30.0), (8, 12.0), (12, 12.0)])
def test_tensor_core_stage1_outlier_sweep(tensor_core_stage1, k, mag):
    _run_and_check(Case([2048], seed=k + 1, k=k, mag=mag), lse_atol_fp32=5e-2 if mag < 20 else 0.2)


def test_tensor_core_stage1_ragged_batch_and_segments(tensor_core_stage1):
    lens = [40, 71, 72, 1024, 5000, 333, 8, 2049]
    _run_and_check(Case(lens, seed=11, tables_dtype=torch.int64))
    _run_and_check(Case([1000], seed=3, outlier_map=False))
    _run_and_check(Case([3000], seed=32, page_size=32))


def test_tensor_core_stage1_agrees_with_default_kernel(monkeypatch):
    case = Case([9000, 700], seed=8)
    monkeypatch.setenv("OMMX_B200_STAGE1", "legacy")
    o1, l1 = case.run(num_kv_splits=24)
    monkeypatch.setenv("OMMX_B200_STAGE1", "tc")
    o2, l2 = case.run(num_kv_splits=24)
    assert (o1 - o2).abs().max().item() < 2e-3 and (l1 - l2).abs().max().item() < 2e-3


def test_bounded_waits_give_up_and_the_device_stays_usable(monkeypatch):
    """The give-up path of stage 1: with the test knob the producer announces one ring fill without issuing its
    copies and every wait has a 2 ms limit, so all three warp roles run out of patience, report it in the status
    word and leave through the epilogue.  Nothing traps or hangs; the next call on the device is an ordinary one."""
    from open_ommx_serve_b200 import _lib
    from open_ommx_serve_b200.attention import paged_decode as pd
    case = Case([3000], seed=3)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    monkeypatch.setenv("OMMX_ABL_TEST_STALL", "1")
    o, lse = case.run(num_kv_splits=4, status=status)
    assert int(status.item()) & _lib.ST_TIMEOUT
    assert torch.isfinite(o).all()                                   # what is left is the attention over the bf16 rows
    monkeypatch.delenv("OMMX_ABL_TEST_STALL")
    assert "OMMX_ABL_TEST_STALL" in pd.abl_flag_names(pd.launch_stats()["abl"])   # a knob that ran is on record
    pd.reset_launch_stats()
    status.zero_()
    o2, lse2 = case.run(num_kv_splits=4, status=status)
    assert int(status.item()) == 0
    want_o, want_lse = case.oracle_kernel_arith(num_kv_splits=4, split_pv=True)
    check_close(o2, want_o, ctx="after a timed-out call")
