"""This package's CUDA decode against the reference's own Triton kernels, on the same planes.

The path's tolerance is stated against the reference's Triton path: max-abs <= 2e-2 and cosine
>= 0.9999 on the same seeded inputs.  Here the unmodified reference package (installed under
baseline/_ref by oracle/build_ref.py; it is not part of this repository) packs the cache with
its own packer on the CPU, its Triton launcher (attention/paged_decode.py:2768) decodes it on
the GPU, and this package's launcher decodes the very same plane tensors, page tables and
residual rows.  Skipped when baseline/_ref or Triton is not there.
"""
import math
import os
import sys

import numpy as np
import pytest
import torch

from helpers import gaussian_kv, check_close

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
SINK, RECENT, PAGE, H, HQ, D = 8, 32, 16, 8, 32, 128


def _reference():
    if not os.path.isfile(os.path.join(REF, "ommx_gpu_serve", "attention", "paged_decode.py")):
        pytest.skip("baseline/_ref is not built (python oracle/build_ref.py next to a reference checkout)")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    try:
        import triton  # noqa: F401
        from ommx_gpu_serve.attention import paged_decode as rdec, pack as rpack
    except Exception as exc:                                  # pragma: no cover - environment dependent
        pytest.skip(f"reference package or triton not importable: {exc}")
    if not rdec.is_available():
        pytest.skip("the reference reports its Triton backend unavailable")
    return rdec, rpack


def _build(rpack, ctx, *, k=6, mag=12.0, seed=42, h=H, hq=HQ, batch=1, permute=True, repr_="bitmap"):
    """Pack `batch` sequences with the REFERENCE packer into one pooled, permuted plane set."""
    packed = max(0, (ctx - SINK - RECENT) // 32 * 32)
    edge = SINK + packed
    n_pages, n_groups = packed // PAGE, packed // 32
    tot_pages, tot_groups = batch * n_pages + 4, batch * n_groups + 2
    gp = torch.randperm(tot_groups, generator=torch.Generator().manual_seed(4243)) if permute else torch.arange(tot_groups)
    pp = torch.randperm(tot_pages, generator=torch.Generator().manual_seed(4242)) if permute else torch.arange(tot_pages)
    pooled, meta = {}, None
    r2t = torch.zeros(batch, n_pages, dtype=torch.int64)
    r2g = torch.zeros(batch, n_groups, dtype=torch.int64)
    tail_len = ctx - packed
    k_tail = torch.zeros(batch, tail_len, h, D, dtype=torch.bfloat16)
    v_tail = torch.zeros(batch, tail_len, h, D, dtype=torch.bfloat16)
    page_planes = ("k_base", "v_main", "v_scale", "v_zp")
    names = page_planes + ("k_scale", "k_zp", "k_obmp", "k_oidx", "k_oval", "k_fp4_mapscale", "k_fp4_mapcenter")
    for b in range(batch):
        K, V = gaussian_kv(seed + 1000 * b, ctx, h, D, mag=mag)
        pl = rpack.ommx_pack_kv_canonical_block(
            K[SINK:edge], V[SINK:edge], outliers_per_vector=k, group_tokens=32, group_channels=32,
            page_size=PAGE, k_format="i2f4", outlier_repr=repr_, use_pow2=True, outlier_select="signed")
        meta = pl
        mine_p, mine_g = pp[b * n_pages:(b + 1) * n_pages], gp[b * n_groups:(b + 1) * n_groups]
        for n in names:
            t = pl.get(n)
            if not torch.is_tensor(t):
                continue
            lead = tot_pages if n in page_planes else tot_groups
            if n not in pooled:
                pooled[n] = torch.zeros((lead,) + tuple(t.shape[1:]), dtype=t.dtype)
            pooled[n][mine_p if n in page_planes else mine_g] = t
        r2t[b], r2g[b] = mine_p, mine_g
        tail = list(range(SINK)) + list(range(edge, ctx))
        k_tail[b], v_tail[b] = K[tail].bfloat16(), V[tail].bfloat16()
    dev = "cuda"
    q = torch.randn(batch, hq, D, generator=torch.Generator().manual_seed(seed + 7)).bfloat16()
    return dict(planes={n: t.to(dev) for n, t in pooled.items()}, meta=meta, q=q.to(dev),
                k_tail=k_tail.to(dev), v_tail=v_tail.to(dev), r2t=r2t.to(dev), r2g=r2g.to(dev),
                b_seq_len=torch.full((batch,), packed, dtype=torch.int32, device=dev),
                b_tail_len=torch.full((batch,), tail_len, dtype=torch.int32, device=dev),
                packed=packed, tail=tail_len, k=k, batch=batch, hq=hq)


def _decode(fn, c, **extra):
    p = c["planes"]
    o = torch.full((c["batch"], c["hq"], D), float("nan"), dtype=torch.float32, device="cuda")
    lse = torch.full((c["batch"], c["hq"]), float("nan"), dtype=torch.float32, device="cuda")
    fn(c["q"], p["k_base"], p["k_scale"], p["k_zp"], p.get("k_oidx"), p.get("k_oval"),
       p["v_main"], p["v_scale"], p["v_zp"], c["k_tail"], c["v_tail"], c["b_tail_len"],
       o, lse, c["r2t"], c["r2g"], c["b_seq_len"],
       sm_scale=1.0 / math.sqrt(D), page_size=PAGE, k_outliers_per_vector=c["k"], k_format="i2f4",
       bitmap_read=c["k"] > 0 and p.get("k_obmp") is not None, k_obmp=p.get("k_obmp"),
       k_fp4_mapscale=p.get("k_fp4_mapscale"), k_fp4_mapcenter=p.get("k_fp4_mapcenter"),
       kv_outlier_map=bool(c["meta"].get("kv_outlier_map", False)) and c["k"] > 0,
       kv_int8_scale=bool(c["meta"].get("kv_int8_scale", False)),
       max_seq_len=c["packed"], max_tail_len=c["tail"], **extra)
    torch.cuda.synchronize()
    return o, lse


def _compare(c, ctx_name):
    rdec, _ = _reference()
    from open_ommx_serve_b200.attention.paged_decode import ommx_paged_decode_attention_canonical as ours
    o_ref, lse_ref = _decode(rdec.ommx_paged_decode_attention_canonical, c)
    o, lse = _decode(ours, c)
    assert torch.isfinite(o_ref).all(), "the reference's Triton output is not finite"
    # the path's gate, against the reference's Triton output
    check_close(o, o_ref.cpu().numpy(), cos_min=0.9999, max_abs=2e-2, ctx="vs triton " + ctx_name)
    np.testing.assert_allclose(lse.cpu().numpy(), lse_ref.cpu().numpy(), atol=2e-2, rtol=0)


@pytest.mark.parametrize("ctx", [1024, 4096, 16384])
def test_matches_triton_reference(ctx):
    _, rpack = _reference()
    _compare(_build(rpack, ctx), f"ctx {ctx}")


@pytest.mark.parametrize("mag", [4.0, 12.0, 30.0])
@pytest.mark.parametrize("k", [0, 6, 8])
def test_matches_triton_reference_outlier_magnitudes(k, mag):
    _, rpack = _reference()
    _compare(_build(rpack, 2048, k=k, mag=mag, seed=7 + k), f"ctx 2048 k={k} mag={mag}")


@pytest.mark.parametrize("k", [6, 10])
def test_matches_triton_reference_relidx7(k):
    """The reference's relidx7 read path (attention/paged_decode.py:640-706), which also serves k > 8."""
    _, rpack = _reference()
    _compare(_build(rpack, 2048, k=k, seed=30 + k, repr_="relidx7"), f"ctx 2048 relidx7 k={k}")


def test_matches_triton_reference_batch_gqa8():
    """Llama-70B head geometry (64 query heads over 8 kv heads), four sequences."""
    _, rpack = _reference()
    _compare(_build(rpack, 3000, hq=64, batch=4, seed=3), "ctx 3000 x4 gqa8")


def test_matches_triton_reference_64k():
    """The headline context.  The planes come from this package's CUDA packer, after it has been held
    equal, plane for plane, to the reference packer on the first 4 096 tokens of the same data."""
    rdec, rpack = _reference()
    from open_ommx_serve_b200.attention.pack import ommx_pack_kv_canonical_block as our_pack
    ctx = 65536
    packed = (ctx - SINK - RECENT) // 32 * 32
    edge = SINK + packed
    K, V = gaussian_kv(42, ctx, H, D)
    kw = dict(outliers_per_vector=6, page_size=PAGE, outlier_repr="bitmap", outlier_select="signed", use_pow2=True)
    pl = our_pack(K[SINK:edge].bfloat16().cuda(), V[SINK:edge].bfloat16().cuda(), kv_outlier_map=True, **kw)
    ref_head = rpack.ommx_pack_kv_canonical_block(K[SINK:SINK + 4096], V[SINK:SINK + 4096], group_tokens=32,
                                                  group_channels=32, k_format="i2f4", **kw)
    for n in ("k_base", "v_main", "v_scale", "v_zp"):
        assert torch.equal(pl[n][:4096 // PAGE].cpu(), ref_head[n]), n
    for n in ("k_scale", "k_zp", "k_obmp", "k_oval", "k_fp4_mapscale", "k_fp4_mapcenter"):
        assert torch.equal(pl[n][:4096 // 32].cpu(), ref_head[n]), n
    tail = list(range(SINK)) + list(range(edge, ctx))
    c = dict(planes={n: t for n, t in pl.items() if torch.is_tensor(t)}, meta=ref_head,
             q=torch.randn(1, HQ, D, generator=torch.Generator().manual_seed(49)).bfloat16().cuda(),
             k_tail=K[tail].bfloat16()[None].cuda(), v_tail=V[tail].bfloat16()[None].cuda(),
             r2t=torch.arange(packed // PAGE, dtype=torch.int64, device="cuda")[None],
             r2g=torch.arange(packed // 32, dtype=torch.int64, device="cuda")[None],
             b_seq_len=torch.tensor([packed], dtype=torch.int32, device="cuda"),
             b_tail_len=torch.tensor([ctx - packed], dtype=torch.int32, device="cuda"),
             packed=packed, tail=ctx - packed, k=6, batch=1, hq=HQ)
    _compare(c, "ctx 65536")
