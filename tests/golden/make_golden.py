#!/usr/bin/env python3
"""Generate the golden fixtures in this folder by running the REFERENCE project's own CPU code.

    python tests/golden/make_golden.py /path/to/open_ommx_serve [case ...]

(with case names given, only those files are rewritten)

It imports, unmodified, from the reference checkout:
  * ommx_gpu_serve.attention.pack.ommx_pack_kv_canonical_block / dequant_kv_canonical
  * ommx_gpu_serve.attention.oracle.synth_kv / reference_output
  * ommx_fakequant/quant_function.py::_apply_group_quantization_vectorized   (loaded by path)
and writes one ``.npz`` per case: the seeded inputs plus every output plane; for the two benchmark-sized
blocks it writes the SHA-256 of every reference-made plane to ``plane_sha256.json`` instead.  The fixtures are
the pin that tests/test_oracle.py holds the CPU oracle to (bit for bit), and that the GPU parity
tests hold the CUDA kernels to.  The reference is needed only here; the tests read the files.
bf16 tensors are stored as uint16 bit patterns.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/open_ommx_serve")
REF = sys.argv[1]
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

from ommx_gpu_serve.attention.pack import ommx_pack_kv_canonical_block, dequant_kv_canonical  # noqa: E402
from ommx_gpu_serve.attention.oracle import synth_kv, reference_output  # noqa: E402

_spec = importlib.util.spec_from_file_location(
    "ref_quant_function", os.path.join(REF, "ommx_fakequant", "quant_function.py"))
_qf = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_qf)

PLANES = ("k_base", "k_scale", "k_zp", "k_obmp", "k_oval", "k_fp4_mapscale", "k_fp4_mapcenter",
          "v_main", "v_scale", "v_zp")


def gaussian_kv(seed, T, H, D, mag=12.0, bf16=True):
    """N(0,1) K/V with 4 K channels per head scaled by ``mag`` (the benchmark's distribution)."""
    g = torch.Generator().manual_seed(seed)
    K = torch.randn(T, H, D, generator=g)
    V = torch.randn(T, H, D, generator=g)
    for h in range(H):
        idx = torch.randperm(D, generator=torch.Generator().manual_seed(seed + 1 + h))[:4]
        K[:, h, idx] *= mag
    if bf16:
        K, V = K.bfloat16().float(), V.bfloat16().float()
    return K, V


def _np(t):
    if t is None:
        return None
    return t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def pack_case(name, K, V, *, k=6, select="signed", use_pow2=True, omap=True, page_size=16,
              with_dequant=True):
    ref = ommx_pack_kv_canonical_block(
        K, V, outliers_per_vector=k, outlier_repr="bitmap", outlier_select=select,
        use_pow2=use_pow2, kv_outlier_map=omap, page_size=page_size)
    out = {"K": K.numpy(), "V": V.numpy(),
           "cfg": np.array([k, int(select == "signed"), int(use_pow2), int(omap), page_size])}
    for p in PLANES:
        if ref[p] is not None:
            out[p] = _np(ref[p])
    if with_dequant:
        Kd, Vd = dequant_kv_canonical(ref)
        out["K_dq"], out["V_dq"] = Kd.numpy(), Vd.numpy()
    _save(name, out)
    return ref


def _save(name, arrays):
    if len(sys.argv) > 2 and name not in sys.argv[2:]:
        return
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    h = hashlib.sha256(open(path, "rb").read()).hexdigest()[:16]
    print(f"{name:24s} {os.path.getsize(path) / 1024:8.1f} KiB  sha256:{h}")


def main():
    torch.set_num_threads(1)
    pack_case("pack_default", *gaussian_kv(42, 64, 2, 128))
    pack_case("pack_fp32_inputs", *gaussian_kv(1, 64, 2, 128, bf16=False))
    for k in (0, 2, 4, 8):
        pack_case(f"pack_k{k}", *gaussian_kv(3, 32, 1, 128), k=k)
    for k in (9, 12, 16):       # value streams longer than one 32-bit word
        pack_case(f"pack_k{k}", *gaussian_kv(3, 32, 1, 128), k=k)
    pack_case("pack_abs_k3", *gaussian_kv(4, 32, 2, 128), k=3, select="abs")
    pack_case("pack_shared_map", *gaussian_kv(5, 32, 2, 128), omap=False)
    pack_case("pack_bf16_scale", *gaussian_kv(5, 32, 2, 128), use_pow2=False)
    pack_case("pack_page32", *gaussian_kv(6, 64, 2, 128, mag=30.0), page_size=32)
    Ks, Vs = synth_kv(64, 2, 128, seed=42)
    pack_case("pack_spiked", Ks.float(), Vs.float())
    # edge cases: all-zero vectors, exact ties, constant vectors, tiny and huge magnitudes
    K, V = gaussian_kv(7, 64, 2, 128)
    K[:32, 0] = 0.0
    K[32:, 0, :5] = 1.5
    K[40:50, 1, 7] = K[40, 1, 7]
    K[:32, 1, 64:] *= 1e-6
    K[32:, 1, 64:] *= 3e4
    K[:32, 1, 10] = torch.tensor([1.0, 2.0] * 16)
    V[:8] = 0.0
    V[8:16] = 3.25
    V[16:24] *= 1e-5
    V[24:32] *= 1e5
    pack_case("pack_edge", K.bfloat16().float(), V.bfloat16().float())

    # fake quantizer (the timed CPU baseline): fp32 inputs, front 8 / back 32 full precision
    K, V = gaussian_kv(11, 200, 2, 128, bf16=False)
    Kb, Vb = K.permute(1, 0, 2)[None].contiguous(), V.permute(1, 0, 2)[None].contiguous()
    kw = dict(group_size=32, bits=2, use_pow2=True, attention_sink_num=32, attention_sink_num_front=8,
              debug_mode=False, outlier_method="fp4", outliers_per_group=0, is_prefill=False)
    fk = _qf._apply_group_quantization_vectorized(
        Kb, is_key=True, outlier_percent_topk=3 / 32, outlier_percent_bottomk=3 / 32, **kw)[0]
    fv = _qf._apply_group_quantization_vectorized(
        Vb, is_key=False, outlier_percent_topk=0.0, outlier_percent_bottomk=0.0, **kw)[0]
    _save("fakequant_t200", {"K": K.numpy(), "V": V.numpy(), "K_fq": fk.numpy(), "V_fq": fv.numpy()})

    # the other outlier-index encoding the reference's presets name: relidx7 (k = 6 and the k = 10 recipe)
    for k in (6, 10):
        K, V = gaussian_kv(20 + k, 64, 2, 128)
        ref = ommx_pack_kv_canonical_block(K, V, outliers_per_vector=k, outlier_repr="relidx7", outlier_select="signed",
                                           use_pow2=True, kv_outlier_map=True, page_size=16)
        out = {"K": K.numpy(), "V": V.numpy(), "cfg": np.array([k, 1, 1, 1, 16]), "k_oidx": _np(ref["k_oidx"])}
        for p in PLANES:
            if ref[p] is not None:
                out[p] = _np(ref[p])
        Kd, Vd = dequant_kv_canonical(ref)
        out["K_dq"], out["V_dq"] = Kd.numpy(), Vd.numpy()
        _save(f"pack_relidx7_k{k}", out)

    # attention: the reference's fp32 oracle over (dequantized packed prefix + bf16 residual rows)
    for name, seed, seq, H, Hq in (("attn_seq168", 42, 168, 2, 8), ("attn_seq300_gqa8", 9, 300, 1, 8)):
        D, sink, recent = 128, 8, 32
        K, V = gaussian_kv(seed, seq, H, D)
        q = torch.randn(Hq, D, generator=torch.Generator().manual_seed(seed + 100)).bfloat16()
        boundary = sink + ((seq - sink - recent) // 32) * 32
        ref = ommx_pack_kv_canonical_block(
            K[sink:boundary], V[sink:boundary], outliers_per_vector=6, outlier_repr="bitmap",
            outlier_select="signed", use_pow2=True, kv_outlier_map=True, page_size=16)
        Kd, Vd = dequant_kv_canonical(ref)
        tail = list(range(sink)) + list(range(boundary, seq))
        Kf = torch.cat([Kd, K[tail]])
        Vf = torch.cat([Vd, V[tail]])
        o = reference_output(q, Kf, Vf, Hq, H, D ** -0.5)
        _save(name, {"K": _np(K.bfloat16()), "V": _np(V.bfloat16()), "q": _np(q),
                     "o": o.numpy(), "cfg": np.array([seq, H, Hq, D, sink, recent])})


def plane_hashes():
    """SHA-256 of every plane the reference packer makes for the benchmark-sized blocks (too large to commit as
    arrays): config 1's 4 032 x 8 x 128 block (seed 42, bf16-valued) and an 8 192-token prefill chunk (seed 43)."""
    import json
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    out = {}
    for name, seed, T, skip in (("config1_ctx4096", 42, 4096, 8), ("prefill_chunk_8192", 43, 8192 + 8, 8)):
        K, V = gaussian_kv(seed, T, 8, 128)
        n = (T - skip - 32) // 32 * 32 if name.startswith("config1") else 8192
        ref = ommx_pack_kv_canonical_block(
            K[skip:skip + n], V[skip:skip + n], outliers_per_vector=6, outlier_repr="bitmap",
            outlier_select="signed", use_pow2=True, kv_outlier_map=True, page_size=16)
        out[name] = {"seed": seed, "tokens": n, "first_token": skip,
                     "sha256": {p: hashlib.sha256(np.ascontiguousarray(_np(ref[p])).tobytes()).hexdigest()
                                for p in PLANES if ref[p] is not None}}
        print(name, n, "tokens hashed")
    with open(os.path.join(HERE, "plane_sha256.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
    if len(sys.argv) <= 2 or "plane_sha256" in sys.argv[2:]:
        plane_hashes()
