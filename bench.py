#!/usr/bin/env python3
"""Benchmark of the OMMX paged decode-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): one decode step of the attention path through a 32-layer stack,
Llama-3.1-8B geometry (32 query heads, 8 KV heads, head_dim 128), batch 1, context 64K, OMMX
recipe k=6 / sink 8 / recent 32, 16-token pages behind a seeded random page table.  Each layer
has its own packed planes, so one step streams 32 x 69 MB - far more than the 126 MB L2; L2
is flushed between timed steps as well.  Metric: microseconds per layer (lower is better); the
achieved HBM GB/s (packed-KV bytes / time) and the contexts 1K..128K are reported beside it.

  value      device-resident inputs, the whole step replayed as one CUDA graph
  roofline   stage-1 kernel alone: algorithmic bytes per launch / its average duration
             (CUDA events on the launching stream), against the measured copy bandwidth
  e2e        the public Python entry with HOST buffers: per step the q and new K/V rows of
             every layer are copied from pinned memory and the outputs are copied back
  contexts   per context: whole step, stage 1, stage 2, the all-gather (N > 1), and the
             reference's own Triton kernels timed on the same planes of the same GPU
             (baseline/_ref, the reference's microbenchmark protocol: graph replay, 3 + 20, median)
  workloads  the other configurations as sub-records: batch 32 ragged with the per-step store,
             Llama-70B head geometry (batch 8 x 32K), the prefill-time bulk pack of 8 192 tokens
  cpu_baseline / --impl reference
             the reference's CPU path - its own fake quantizer (oracle/_ref, unmodified) on K and V,
             then dense attention - timed on the host cores on ONE layer of the same context

With N > 1 (torchrun) the 8 KV heads are sharded over the ranks and nothing is exchanged during
attention; the head outputs of a layer are exchanged inside stage 2 (--gather peer, the default:
every rank's stage 2 stores its rows into all ranks' buffers through peer-mapped memory) or by one
NCCL all-gather per layer (--gather nccl); both are timed on every run, inside the step or beside it.
Synthetic data throughout: seeded N(0,1) K/V with 4 K channels per head scaled x12.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, HQ, HKV, D, PAGE = 32, 32, 8, 128, 16
SINK, RECENT, K_OUT = 8, 32, 6
MAG = 12.0                # factor on the 4 outlier channels of every K head
CONTEXTS = (1024, 4096, 16384, 32768, 65536, 131072)
HEADLINE_CTX = 65536
H200_PUBLISHED_US = {65536: 563.2, 32768: 284.1, 16384: 162.3, 4096: 147.3, 1024: 469.6}
TRITON_BUDGET_S = 240.0   # wall-clock cap on the Triton legs of one run (JIT compiles dominate)


def packed_len(ctx):
    return max(0, (ctx - SINK - RECENT) // 32 * 32)


# dram__bytes_read.sum + dram__bytes_write.sum of one stage-1 launch under ncu over its algorithmic
# bytes (profiles/decode_stage1_64k_b1.md): the planes are read once, nothing is re-read
NCU_TRAFFIC_RATIO = (69.261312e6 + 1.031936e6) / 69138432.0


def unit_bytes(k):
    """Packed bytes per (token, kv head): codes 32 + K scale 4 + K zero-point 8 (+ map scale 8, map centre 8, bitmask
    16 and 4 bytes per pair of outliers when k > 0) + V 44; 132 at k = 6."""
    return 32 + 4 + 8 + ((8 + 8 + 16 + 4 * ((k + 1) // 2)) if k > 0 else 0) + 44


def algorithmic_bytes(ctx, batch, hkv):
    """Bytes the path must read per layer: every plane handed to the kernel + the bf16 rows."""
    p = packed_len(ctx)
    return batch * (p * hkv * unit_bytes(K_OUT) + (ctx - p) * hkv * D * 2 * 2)


def measured_peak_gbs():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ───────────────────────────── reference arm / CPU baseline ─────────────────────────────

def _reference_fakequant():
    """The reference's own fake quantizer, loaded by path from oracle/_ref (None when not built)."""
    path = os.path.join(ROOT, "oracle", "_ref", "ommx_fakequant", "quant_function.py")
    if not os.path.isfile(path):
        return None
    spec = importlib.util.spec_from_file_location("ref_quant_function", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod._apply_group_quantization_vectorized


def cpu_reference_layer(ctx, steps=3, warmup=1, seed=42):
    """The reference's CPU path on one layer: fake-quantize K (outliers kept as FP4) and V
    (ommx_fakequant/quant_function.py:152, run unmodified from oracle/_ref when it is there, else
    the restatement in oracle/ommx_oracle.py), then dense attention of one query row over the
    result (ommx_fakequant/quant_attention.py:688,957).  All host cores."""
    import numpy as np
    import torch
    from oracle import ommx_oracle as O
    torch.set_num_threads(host_cores())          # torchrun exports OMP_NUM_THREADS=1; undo that here
    ref_fq = _reference_fakequant()
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(HQ, D, generator=g)
    K = torch.randn(ctx, HKV, D, generator=g)
    V = torch.randn(ctx, HKV, D, generator=g)
    for h in range(HKV):
        idx = torch.randperm(D, generator=torch.Generator().manual_seed(seed + 1 + h))[:4]
        K[:, h, idx] *= MAG
    Kh, Vh = K.permute(1, 0, 2).contiguous(), V.permute(1, 0, 2).contiguous()
    kw = dict(group_size=32, bits=2, use_pow2=True, attention_sink_num=RECENT, attention_sink_num_front=SINK,
              debug_mode=False, outlier_method="fp4", outliers_per_group=0, is_prefill=False)

    def quantize():
        if ref_fq is not None:
            Kq = ref_fq(Kh[None], is_key=True, outlier_percent_topk=3 / 32, outlier_percent_bottomk=3 / 32, **kw)[0]
            Vq = ref_fq(Vh[None], is_key=False, outlier_percent_topk=0.0, outlier_percent_bottomk=0.0, **kw)[0]
            return Kq, Vq
        return (O.fakequant_group_torch(Kh, is_key=True),
                O.fakequant_group_torch(Vh, is_key=False, top=0, bottom=0))

    times, qt, at = [], [], []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        Kq, Vq = quantize()
        t1 = time.perf_counter()
        Kr = Kq.repeat_interleave(HQ // HKV, dim=0)[None]
        Vr = Vq.repeat_interleave(HQ // HKV, dim=0)[None]
        out = torch.nn.functional.scaled_dot_product_attention(q[None, :, None, :], Kr, Vr)
        t2 = time.perf_counter()
        if i >= warmup:
            times.append(t2 - t0)
            qt.append(t1 - t0)
            at.append(t2 - t1)
    # correctness of what was timed: dense fp64 attention over the same fake-quantized cache
    want, _ = O.attention_fp32(q.numpy(), Kq.permute(1, 0, 2).numpy(), Vq.permute(1, 0, 2).numpy(), D ** -0.5)
    err = float(np.abs(out[0, :, 0].numpy() - want).max())
    mean = sum(times) / len(times)
    return {"us_per_layer": mean * 1e6, "median_us": sorted(times)[len(times) // 2] * 1e6,
            "quant_ms": sorted(qt)[len(qt) // 2] * 1e3, "attn_ms": sorted(at)[len(at) // 2] * 1e3,
            "max_abs_vs_dense": err, "threads": torch.get_num_threads(), "cpu_count": os.cpu_count(),
            "kind": "reference" if ref_fq is not None else "port"}


def cpu_baseline_record(res, ctx, steps):
    what = ("the reference's ommx_fakequant/quant_function.py run unmodified" if res["kind"] == "reference"
            else "the restatement of ommx_fakequant/quant_function.py in oracle/")
    return {"value": res["us_per_layer"], "unit": "us", "cores": res["threads"], "kind": res["kind"],
            "sample": f"1 of {LAYERS} layers at ctx {ctx} per step ({what}): fake-quantize K+V ({res['quant_ms']:.0f} ms) + "
                      f"dense attention ({res['attn_ms']:.1f} ms), mean of {steps}; host has {res['cpu_count']} cpus",
            "max_abs_vs_dense_attention": res["max_abs_vs_dense"]}


def run_reference(args, rank, world):
    """`--impl reference`: rank 0 alone times the reference's CPU path; a step is ONE layer of the
    configured context (the layers of a stack are independent and identical in cost)."""
    if rank != 0:
        return
    ctx = args.ctx
    res = cpu_reference_layer(ctx, steps=max(1, args.steps), warmup=max(0, args.warmup))
    us = res["us_per_layer"]
    line = {
        "impl": "reference", "metric": "ommx_decode_attn_us_per_layer", "value": us, "unit": "us",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"llama3.1-8b geometry, {LAYERS}-layer stack, batch 1, ctx {ctx}, OMMX k={K_OUT} (outlier channels x{MAG:g}) sink 8 "
                               f"recent 32, {PAGE}-token pages, random page table",
                   "ctx": ctx, "batch": 1,
                   "step": "one timed step = ONE layer of the stack on the host cores (a bounded sample: the layers are "
                           "independent and cost the same); value is per layer, like the GPU arm's"},
        "extrapolated_stack_ms": us * LAYERS / 1e3,
        "cpu_baseline": cpu_baseline_record(res, ctx, max(1, args.steps)),
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "hbm_gbs": algorithmic_bytes(ctx, 1, HKV) / us / 1e3, "gpu_launches": 0,
    }
    print(json.dumps(line))


# ───────────────────────────── our arm ─────────────────────────────

class LayerStack:
    """`layers` layers of pooled planes for one rank's share of the KV heads."""

    def __init__(self, ctx, batch, hkv, hq, device, seed=42, layers=None):
        import torch
        from open_ommx_serve_b200.attention.pack import alloc_planes, ommx_pack_kv_into
        self.n_layers = LAYERS if layers is None else layers
        self.ctx, self.batch, self.hkv, self.hq, self.device = ctx, batch, hkv, hq, device
        P = packed_len(ctx)
        self.max_packed, self.max_tail = P, ctx - P
        pages_per_seq, groups_per_seq = P // PAGE, P // 32
        n_groups = batch * groups_per_seq
        n_pages = n_groups * (32 // PAGE)
        gen = torch.Generator().manual_seed(4242)
        pperm = torch.randperm(n_pages, generator=gen).to(torch.int32)
        gperm = torch.randperm(n_groups, generator=torch.Generator().manual_seed(4243)).to(torch.int32)
        self.req_to_token = pperm.reshape(batch, pages_per_seq).contiguous().to(device)
        self.req_to_group = gperm.reshape(batch, groups_per_seq).contiguous().to(device)
        self.layers = []
        cg = torch.Generator(device=device)
        chunk = 16384
        # residual rows of all layers in one tensor each, so that a step's new rows land with one copy
        self.k_tail_all = torch.empty(self.n_layers, batch, 72, hkv, D, dtype=torch.bfloat16, device=device)
        self.v_tail_all = torch.empty_like(self.k_tail_all)
        ch_idx = [torch.randperm(D, generator=torch.Generator().manual_seed(seed + 1 + h))[:4].to(device) for h in range(hkv)]
        for layer in range(self.n_layers):
            pl = alloc_planes(n_pages, n_groups, hkv, D, page_size=PAGE, outliers_per_vector=K_OUT,
                              kv_outlier_map=True, device=device)
            cg.manual_seed(seed + layer)
            tails_k, tails_v = self.k_tail_all[layer], self.v_tail_all[layer]
            for b in range(batch):
                for t0 in range(0, P, chunk):
                    n = min(chunk, P - t0)
                    K = torch.randn(n, hkv, D, generator=cg, device=device)
                    V = torch.randn(n, hkv, D, generator=cg, device=device)
                    for h in range(hkv):
                        K[:, h, ch_idx[h]] *= MAG
                    ommx_pack_kv_into(K.bfloat16(), V.bfloat16(), pl,
                                      dst_pages=self.req_to_token[b, t0 // PAGE:(t0 + n) // PAGE].contiguous(),
                                      dst_groups=self.req_to_group[b, t0 // 32:(t0 + n) // 32].contiguous(),
                                      outliers_per_vector=K_OUT)
                tails_k[b] = torch.randn(72, hkv, D, generator=cg, device=device).bfloat16()
                tails_v[b] = torch.randn(72, hkv, D, generator=cg, device=device).bfloat16()
            q = torch.randn(batch, hq, D, generator=cg, device=device).bfloat16()
            self.layers.append({"planes": pl, "k_tail": tails_k, "v_tail": tails_v, "q": q})
        self.b_seq_len = torch.full((batch,), P, dtype=torch.int32, device=device)
        self.b_tail_len = torch.full((batch,), ctx - P, dtype=torch.int32, device=device)
        self.o = torch.zeros(self.n_layers, batch, hq, D, dtype=torch.float32, device=device)
        self.lse = torch.zeros(self.n_layers, batch, hq, dtype=torch.float32, device=device)
        self.ws = None
        self.splits = 0

    def set_context(self, ctx):
        """Serve a shorter context out of the same planes (a prefix of every sequence)."""
        from open_ommx_serve_b200.attention.paged_decode import _auto_num_kv_splits
        import torch
        P = packed_len(ctx)
        self.cur_ctx, self.cur_packed, self.cur_tail = ctx, P, ctx - P
        self.b_seq_len.fill_(P)
        self.b_tail_len.fill_(ctx - P)
        self.splits = _auto_num_kv_splits(max(P, 1), self.batch, device=self.device, kv_heads=self.hkv)
        self.ws = torch.empty(self.batch, self.hq, self.splits + 1, D + 1, dtype=torch.float32, device=self.device)

    def decode_layer(self, i, q=None, stage=0, fn=None, o=None, lse=None, head_gather=None):
        """One decode call on layer i through this package's entry, or through `fn` (the reference's
        Triton launcher, which takes the same arguments)."""
        L = self.layers[i]
        p = L["planes"]
        kw = {}
        if fn is None:
            from open_ommx_serve_b200.attention.paged_decode import ommx_paged_decode_attention_canonical as fn
            kw = dict(num_kv_splits=self.splits, attn_logits=self.ws, _stage=stage, head_gather=head_gather)
        fn(L["q"] if q is None else q, p["k_base"], p["k_scale"], p["k_zp"], None, p["k_oval"],
           p["v_main"], p["v_scale"], p["v_zp"], L["k_tail"], L["v_tail"], self.b_tail_len,
           self.o[i] if o is None else o, self.lse[i] if lse is None else lse,
           self.req_to_token, self.req_to_group, self.b_seq_len,
           sm_scale=D ** -0.5, page_size=PAGE, k_outliers_per_vector=K_OUT, bitmap_read=True,
           k_obmp=p["k_obmp"], k_fp4_mapscale=p["k_fp4_mapscale"], k_fp4_mapcenter=p["k_fp4_mapcenter"],
           kv_outlier_map=True, kv_int8_scale=True,
           max_seq_len=self.cur_packed, max_tail_len=self.cur_tail, **kw)


def timed_graph(fn, steps, warmup, flush, torch):
    """Capture ``fn`` (one step) in a CUDA graph; return per-step device times in ms."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        fn()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return times


class TritonReference:
    """The reference's own Triton launcher (baseline/_ref, unmodified) on this GPU, same planes."""

    def __init__(self):
        self.fn, self.why, self.spent = None, None, 0.0
        ref = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isfile(os.path.join(ref, "ommx_gpu_serve", "attention", "paged_decode.py")):
            self.why = "baseline/_ref not built"
            return
        try:
            if ref not in sys.path:
                sys.path.insert(0, ref)
            import triton  # noqa: F401
            from ommx_gpu_serve.attention import paged_decode as rdec
            if not rdec.is_available():
                raise RuntimeError("reference reports its Triton backend unavailable")
            self.fn = rdec.ommx_paged_decode_attention_canonical
        except Exception as exc:
            self.why = f"{type(exc).__name__}: {str(exc)[:160]}"

    def time_layer(self, stack, flush, torch, layer=0):
        """Median µs of one layer's decode by the reference's protocol (bench/bench_decode_kernel.py:233-256:
        CUDA-graph replay, 3 warm-up + 20 measured, median) with L2 flushed before every replay; also
        returns max-abs / cosine of this package's output against the Triton output on that layer."""
        if self.fn is None or self.spent > TRITON_BUDGET_S:
            return None
        t_wall = time.time()
        try:
            o = torch.zeros_like(stack.o[layer])
            lse = torch.zeros_like(stack.lse[layer])

            def launch():
                stack.decode_layer(layer, fn=self.fn, o=o, lse=lse)

            launch()                                   # JIT compile + autotune outside the capture
            torch.cuda.synchronize()
            ms = sorted(timed_graph(launch, 20, 3, flush, torch))
            stack.decode_layer(layer)
            torch.cuda.synchronize()
            diff = float((stack.o[layer] - o).abs().max().item())
            cos = float(torch.nn.functional.cosine_similarity(stack.o[layer].flatten().double(), o.flatten().double(), dim=0).item())
            return {"us": 0.5 * (ms[9] + ms[10]) * 1e3, "max_abs_ours_vs_triton": diff, "cos_ours_vs_triton": cos}
        except Exception as exc:
            self.why = f"{type(exc).__name__}: {str(exc)[:160]}"
            self.fn = None
            return None
        finally:
            self.spent += time.time() - t_wall


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from open_ommx_serve_b200 import _lib, sharding

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    hkv, hq = HKV // world, HQ // world
    contexts = [c for c in CONTEXTS if c <= max(args.ctx, args.max_ctx)] if args.all_contexts else [args.ctx]
    stack = LayerStack(max(contexts), 1, hkv, hq, device)
    if args.profile:
        # plain eager launches for a profiler: no graph, no timing, no JSON line
        stack.set_context(args.ctx)
        for _ in range(args.steps):
            for i in range(LAYERS):
                stack.decode_layer(i)
        torch.cuda.synchronize()
        print(f"profile run: {args.steps} x {LAYERS} decode calls at ctx {args.ctx}, splits {stack.splits}", file=sys.stderr)
        return
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    gathered = torch.zeros(LAYERS, world, 1, hq, D, dtype=torch.float32, device=device) if world > 1 else None
    lib = _lib.load()
    triton_ref = TritonReference() if (rank == 0 and not args.no_triton) else None

    peer, peer_note = None, None
    if world > 1 and args.gather == "peer":
        try:
            peer = sharding.PeerHeadGather(world, rank, max(2, LAYERS), 1, hq, D, device)
        except RuntimeError as exc:                                # every rank raises together: all fall back together
            peer_note = f"peer-mapped exchange unavailable ({exc}); NCCL all-gather used"

    def step_full():
        for i in range(LAYERS):
            if peer is not None:
                stack.decode_layer(i, head_gather=peer.plan(i))       # stage 2 stores the rows into every rank's buffer
            else:
                stack.decode_layer(i)
                if world > 1:
                    sharding.gather_head_outputs(stack.o[i], world, out=gathered[i])

    def step_stage2_gather():
        for i in range(LAYERS):
            stack.decode_layer(i, stage=2, head_gather=peer.plan(i))

    def step_stage1():
        for i in range(LAYERS):
            stack.decode_layer(i, stage=1)

    def step_stage2():
        for i in range(LAYERS):
            stack.decode_layer(i, stage=2)

    def step_gather():
        for i in range(LAYERS):
            sharding.gather_head_outputs(stack.o[i], world, out=gathered[i])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    per_ctx = {}
    results = {}
    sampler = ClockSampler(local_rank)
    for ctx in contexts:
        stack.set_context(ctx)
        head = ctx == args.ctx
        k_steps = args.steps if head else max(3, min(args.steps, 5))
        barrier()
        lib.ommx_b200_reset_launch_count()
        if head:
            sampler.__enter__()
        t_full = timed_graph(step_full, k_steps, args.warmup, flush, torch)
        barrier()
        launches_step = int(lib.ommx_b200_launch_count()) // 2   # eager warm-up + capture each ran the step once
        t_s1 = timed_graph(step_stage1, k_steps, args.warmup, flush, torch)
        barrier()
        if head:
            sampler.__exit__()
        t_s2 = timed_graph(step_stage2, max(3, k_steps // 2), args.warmup, flush, torch)
        barrier()
        ms_ag = ms_nccl = None
        if world > 1:
            t_ag = timed_graph(step_gather, max(3, k_steps // 2), args.warmup, flush, torch)
            barrier()
            ms_nccl = ms_ag = reduce_max(sum(t_ag) / len(t_ag))
            if peer is not None:
                # what the exchange adds to stage 2: stage 2 with the peer stores and the arrival wait, minus stage 2 alone
                t_pg = timed_graph(step_stage2_gather, max(3, k_steps // 2), args.warmup, flush, torch)
                barrier()
                ms_ag = max(0.0, reduce_max(sum(t_pg) / len(t_pg)) - reduce_max(sum(t_s2) / len(t_s2)))
        ms_step = reduce_max(sum(t_full) / len(t_full))
        ms_s1 = reduce_max(sum(t_s1) / len(t_s1))
        ms_s2 = reduce_max(sum(t_s2) / len(t_s2))
        bytes_layer = algorithmic_bytes(ctx, 1, HKV)             # whole job (all ranks)
        bytes_launch = algorithmic_bytes(ctx, 1, hkv) - (ctx - packed_len(ctx)) * hkv * D * 4   # stage 1 reads planes only
        tri = triton_ref.time_layer(stack, flush, torch) if (triton_ref is not None and world == 1) else None
        per_ctx[str(ctx)] = {
            "us_per_layer": ms_step * 1e3 / LAYERS, "hbm_gbs": bytes_layer / (ms_step / LAYERS) / 1e6,
            "stage1_us": ms_s1 * 1e3 / LAYERS, "stage1_gbs": bytes_launch / (ms_s1 / LAYERS) / 1e6,
            "stage2_us": ms_s2 * 1e3 / LAYERS,
            "allgather_us": None if ms_ag is None else ms_ag * 1e3 / LAYERS,
            "nccl_allgather_us": None if ms_nccl is None else ms_nccl * 1e3 / LAYERS,
            "splits": stack.splits, "bytes_per_layer": bytes_layer,
            "triton_b200_us": None if tri is None else tri["us"],
            "triton_b200": tri,
            "h200_published_us": H200_PUBLISHED_US.get(ctx)}
        if head:
            results = {"ms_step": ms_step, "ms_s1": ms_s1, "bytes_layer": bytes_layer,
                       "bytes_launch": bytes_launch, "launches_step": launches_step}

    # ---- end to end through the public Python entry with host buffers ----
    stack.set_context(args.ctx)
    # the step's inputs (q and the new K/V row of every layer) in one pinned buffer, its outputs in another
    n_q, n_kv = hq * D, hkv * D
    in_host = torch.randn(LAYERS, n_q + 2 * n_kv).bfloat16().pin_memory()
    in_dev = torch.empty(LAYERS, n_q + 2 * n_kv, dtype=torch.bfloat16, device=device)
    o_host = torch.empty((LAYERS, world, 1, hq, D) if world > 1 else (LAYERS, 1, hq, D), dtype=torch.float32).pin_memory()
    new_row = stack.cur_tail - 1

    def step_e2e():
        in_dev.copy_(in_host, non_blocking=True)                                  # host -> device, once per step
        stack.k_tail_all[:, 0, new_row].copy_(in_dev[:, n_q:n_q + n_kv].view(LAYERS, hkv, D))
        stack.v_tail_all[:, 0, new_row].copy_(in_dev[:, n_q + n_kv:].view(LAYERS, hkv, D))
        for i in range(LAYERS):
            if peer is not None:
                stack.decode_layer(i, q=in_dev[i, :n_q].view(1, hq, D), head_gather=peer.plan(i))
            else:
                stack.decode_layer(i, q=in_dev[i, :n_q].view(1, hq, D))
                if world > 1:
                    sharding.gather_head_outputs(stack.o[i], world, out=gathered[i])
        # device -> host, once per step
        o_host.copy_(peer.all_buffers()[:LAYERS] if peer is not None else (gathered if world > 1 else stack.o), non_blocking=True)

    for _ in range(max(3, args.warmup)):
        step_e2e()
    barrier()
    e2e_times = []
    for _ in range(args.steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step_e2e()
        b.record()
        b.synchronize()
        e2e_times.append(a.elapsed_time(b))
    barrier()
    ms_e2e_eager = reduce_max(sum(e2e_times) / len(e2e_times))
    # the same step - pinned-host copies in, public entry, copy out - replayed from one CUDA graph, which is
    # how a serving loop drives the entry point (it allocates nothing and never synchronises with the host)
    e2e_graph_times = timed_graph(step_e2e, args.steps, max(3, args.warmup), flush, torch)
    barrier()
    ms_e2e = reduce_max(sum(e2e_graph_times) / len(e2e_graph_times))

    gather_check = None
    used_peer = peer is not None
    if peer is not None:
        # the exchanged rows against an NCCL all-gather of the same outputs, once, outside any timed region
        for i in range(LAYERS):
            stack.decode_layer(i, head_gather=peer.plan(i))
            sharding.gather_head_outputs(stack.o[i], world, out=gathered[i])
        torch.cuda.synchronize()
        same = all(torch.equal(peer.gathered(i), gathered[i]) for i in range(LAYERS))
        gather_check = "equal to the NCCL all-gather" if reduce_max(0.0 if same else 1.0) == 0.0 else "MISMATCH against the NCCL all-gather"
        peer.close()
        peer = None
    # ---- the other configurations, as sub-records of the same line ----
    workloads = {}
    del stack
    torch.cuda.empty_cache()
    if not args.no_workloads:
        peak, _ = measured_peak_gbs()
        workloads["llama70b_b8_32k"] = workload_llama70b(args, device, world, flush, reduce_max, barrier, peak, gathered_world=world)
        if world == 1:
            workloads["batch32_store_decode"] = workload_batch32(args, device, flush, peak)
            workloads["prefill_pack_8k"] = workload_prefill_pack(args, device, flush, peak)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peak_gbs()
    us_layer = results["ms_step"] * 1e3 / LAYERS
    ach = results["bytes_launch"] / (results["ms_s1"] / LAYERS) / 1e6
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_record(cpu_reference_layer(args.ctx, steps=2, warmup=1), args.ctx, 2)
    line = {
        "metric": "ommx_decode_attn_us_per_layer", "value": us_layer, "unit": "us", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": results["ms_step"],
        "higher_is_better": False, "scaling": "strong",
        "vs_baseline": us_layer / H200_PUBLISHED_US[args.ctx] if args.ctx in H200_PUBLISHED_US else None,
        "vs_baseline_note": "value / the reference's published H200-NVL microbench time for the same context (other hardware, page 32)",
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"llama3.1-8b geometry, {LAYERS}-layer stack, batch 1, ctx {args.ctx}, OMMX k={K_OUT} (outlier channels x{MAG:g}) sink 8 "
                               f"recent 32, {PAGE}-token pages, random page table",
                   "ctx": args.ctx, "batch": 1, "kv_heads_per_gpu": hkv, "splits": per_ctx[str(args.ctx)]["splits"],
                   "l2": "flushed between timed steps (256 MiB memset); one step reads 32 distinct plane sets",
                   "timing": "CUDA-graph replay of the whole step, CUDA events per step, mean of K, max over ranks",
                   "collective": ("none" if world == 1 else
                                  "stage 2 stores its [1, Hq/N, D] f32 rows into every rank's buffer (peer-mapped memory over NVLink, "
                                  "one arrival count per rank, bounded wait); nccl_allgather_us is the NCCL all-gather of the same rows timed alone"
                                  if used_peer else "one NCCL all-gather of [1, Hq/N, D] f32 per layer inside the step")},
        "hbm_gbs": results["bytes_layer"] / (results["ms_step"] / LAYERS) / 1e6,
        "tokens_per_s": 1.0 / (results["ms_step"] * 1e-3),
        "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                     "traffic": results["bytes_launch"] * NCU_TRAFFIC_RATIO, "peak_kind": peak_kind,
                     "traffic_note": "dram__bytes_read+write of one stage-1 launch under ncu at ctx 65536, 8 kv heads "
                                     "over its algorithmic bytes (profiles/decode_stage1_64k_b1.md), scaled by algorithmic bytes for other shapes",
                     "kernel": "decode_stage1_kernel",
                     "algorithmic_bytes_per_launch": results["bytes_launch"],
                     "us_per_launch": results["ms_s1"] * 1e3 / LAYERS,
                     "frac_of_nominal_8TBs": ach / 8000.0},
        "cpu_baseline": cpu,
        "e2e": {"value": ms_e2e * 1e3 / LAYERS, "unit": "us",
                "h2d_bytes_per_step": LAYERS * (hq * D * 2 + 2 * hkv * D * 2),
                "d2h_bytes_per_step": LAYERS * hq * D * 4 * world,
                "eager_value": ms_e2e_eager * 1e3 / LAYERS,
                "note": "one pinned-host copy in per step (q and the new K/V row of all layers), the public Python entry "
                        "per layer, one copy of all outputs back; the whole step replayed from a CUDA graph; "
                        "eager_value is the same step launched from Python"},
        "gpu_launches": results["launches_step"] * args.steps,
        "gather_check": gather_check if peer_note is None else peer_note,
        "contexts": per_ctx,
        "triton_reference": None if triton_ref is None else {"available": triton_ref.fn is not None, "note": triton_ref.why,
                                                             "seconds_spent": round(triton_ref.spent, 1)},
        "workloads": workloads,
        "clocks": sampler.summary(),
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ───────────────────────────── sub-record workloads ─────────────────────────────

def workload_llama70b(args, device, world, flush, reduce_max, barrier, peak, gathered_world=1):
    """Llama-3.1-70B head geometry (64 query heads, 8 kv heads, GQA 8), batch 8 at 32K context, the kv heads
    sharded over the ranks (all 8 on one GPU at N=1, one per GPU at N=8).  A 4-layer stack stands for the
    80 layers (each layer's planes exceed L2 many times over at N=1; L2 is flushed between steps)."""
    import torch
    from open_ommx_serve_b200 import sharding
    layers, B, ctx = (4 if world == 1 else 8), 8, 32768
    hkv, hq = HKV // world, 64 // world
    stack = LayerStack(ctx, B, hkv, hq, device, seed=7, layers=layers)
    stack.set_context(ctx)
    gathered = torch.zeros(layers, world, B, hq, D, dtype=torch.float32, device=device) if world > 1 else None
    peer = None
    if world > 1 and args.gather == "peer":
        try:
            peer = sharding.PeerHeadGather(world, int(os.environ.get("RANK", "0")), layers, B, hq, D, device)
        except RuntimeError:
            peer = None                                               # every rank raises together: NCCL for all

    def step():
        for i in range(layers):
            if peer is not None:
                stack.decode_layer(i, head_gather=peer.plan(i))
            else:
                stack.decode_layer(i)
                if world > 1:
                    sharding.gather_head_outputs(stack.o[i], world, out=gathered[i])

    def step_s1():
        for i in range(layers):
            stack.decode_layer(i, stage=1)

    steps = max(3, min(args.steps, 10))
    barrier()
    ms = reduce_max(sum(t := timed_graph(step, steps, args.warmup, flush, torch)) / len(t))
    barrier()
    ms1 = reduce_max(sum(t := timed_graph(step_s1, steps, args.warmup, flush, torch)) / len(t))
    barrier()
    p = packed_len(ctx)
    bytes_layer = B * (p * HKV * unit_bytes(K_OUT) + (ctx - p) * HKV * D * 4)
    bytes_launch = B * p * hkv * unit_bytes(K_OUT)
    ach = bytes_launch / (ms1 / layers) / 1e6
    rec = {"config": {"workload": f"llama3.1-70b head geometry (64 q heads, 8 kv heads), batch {B}, ctx {ctx}, {layers}-layer stack "
                                  f"standing for 80 layers, {hkv} kv head(s) per GPU", "splits": stack.splits,
                      "collective": "none" if world == 1 else ("head outputs exchanged inside stage 2 (peer-mapped memory)"
                                                                if peer is not None else "NCCL all-gather per layer")},
           "us_per_layer": ms * 1e3 / layers, "hbm_gbs": bytes_layer / (ms / layers) / 1e6,
           "tokens_per_s_80_layers": B / (ms / layers * 80 * 1e-3),
           "roofline": {"bound": "hbm", "kernel": "decode_stage1_kernel", "achieved": ach, "peak": peak, "unit": "GB/s",
                        "frac": ach / peak, "us_per_launch": ms1 * 1e3 / layers, "algorithmic_bytes_per_launch": bytes_launch}}
    if peer is not None:
        peer.close()
    del stack
    torch.cuda.empty_cache()
    return rec


def workload_batch32(args, device, flush, peak, layers=8):
    """Batch 32, ragged contexts 1K..32K (seed 42), split partition 512; every step stores one new token per
    sequence through the device-resident pool and decodes, per layer."""
    import torch
    from open_ommx_serve_b200 import _lib, ommx_paged_decode_attention_canonical
    from open_ommx_serve_b200.attention.kv_pool import MultiSeqKVPool
    from open_ommx_serve_b200.attention.kv_window import WindowSpec

    B, max_len, part = 32, 32768 + 256, 512
    lens = torch.randint(1024, 32769, (B,), generator=torch.Generator().manual_seed(42)).tolist()
    win = WindowSpec(8, 32, 32, PAGE)
    pools = []
    cg = torch.Generator(device=device)
    for layer in range(layers):
        pool = MultiSeqKVPool(D, HKV, B, max_len, outliers_per_vector=K_OUT, window=win, device=device)
        cg.manual_seed(1000 + layer)
        for r, T in enumerate(lens):
            K = torch.randn(T, HKV, D, generator=cg, device=device)
            V = torch.randn(T, HKV, D, generator=cg, device=device)
            K[:, :, :4] *= 12.0
            pool.append_block(r, K.bfloat16(), V.bfloat16())
        pools.append(pool)
    max_packed = win.packed_len(max_len)
    splits = (max_packed + part - 1) // part
    ws = torch.empty(B, HQ, splits + 1, D + 1, dtype=torch.float32, device=device)
    q = torch.randn(layers, B, HQ, D, generator=cg, device=device).bfloat16()
    kn = torch.randn(layers, B, HKV, D, generator=cg, device=device).bfloat16()
    vn = torch.randn(layers, B, HKV, D, generator=cg, device=device).bfloat16()
    o = torch.zeros(layers, B, HQ, D, dtype=torch.float32, device=device)
    lse = torch.zeros(layers, B, HQ, dtype=torch.float32, device=device)

    def step():
        for i, pool in enumerate(pools):
            pool.append_decode_device(kn[i], vn[i], B)
            d = pool.decode_inputs_device(B, max_packed)
            ommx_paged_decode_attention_canonical(
                q[i], d["k_base"], d["k_scale"], d["k_zp"], None, d["k_oval"], d["v_main"], d["v_scale"], d["v_zp"],
                d["k_tail"], d["v_tail"], d["b_tail_len"], o[i], lse[i], d["req_to_token"], d["req_to_group"],
                d["b_seq_len"], sm_scale=D ** -0.5, page_size=PAGE, k_outliers_per_vector=K_OUT, bitmap_read=True,
                k_obmp=d["k_obmp"], k_fp4_mapscale=d["k_fp4_mapscale"], k_fp4_mapcenter=d["k_fp4_mapcenter"],
                kv_outlier_map=True, kv_int8_scale=True, num_kv_splits=splits, max_seq_len=max_packed,
                max_tail_len=d["max_tail_len"], attn_logits=ws)

    lib = _lib.load()
    lib.ommx_b200_reset_launch_count()
    steps = max(3, min(args.steps, 10))
    times = timed_graph(step, steps, args.warmup, flush, torch)
    ms = sum(times) / len(times)
    packed = sum(win.packed_len(T + args.warmup + steps // 2) for T in lens)
    bytes_layer = packed * HKV * unit_bytes(K_OUT) + sum(T - win.packed_len(T) for T in lens) * HKV * D * 4
    status = max(int(p.status.item()) for p in pools)
    ach = bytes_layer / (ms / layers) / 1e6
    rec = {"config": {"workload": f"llama3.1-8b geometry, {layers}-layer stack, batch 32, contexts uniform 1K..32K (seed 42), "
                                  f"split partition 512 ({splits} splits), one new token stored per sequence per step "
                                  "(device-resident pool), then decode; CUDA-graph replay, L2 flushed between steps",
                      "sum_ctx": sum(lens), "splits": splits},
           "us_per_layer": ms * 1e3 / layers, "hbm_gbs": ach, "tokens_per_s_32_layers": B / (ms / layers * 32 * 1e-3),
           "roofline": {"bound": "hbm", "kernel": "store + stage 1 + stage 2 of one layer", "achieved": ach, "peak": peak,
                        "unit": "GB/s", "frac": ach / peak, "algorithmic_bytes_per_layer": bytes_layer},
           "gpu_launches": int(lib.ommx_b200_launch_count()), "device_status": status}
    del pools
    torch.cuda.empty_cache()
    return rec


def workload_prefill_pack(args, device, flush, peak, tokens=8192):
    """Prefill-time bulk quantize + pack of one 8 192-token K/V chunk (8 kv heads) straight into 16-token pages."""
    import torch
    from open_ommx_serve_b200.attention.pack import alloc_planes, ommx_pack_kv_into
    n_sets = 4
    g = torch.Generator(device=device).manual_seed(5)
    Ks = [torch.randn(tokens, HKV, D, generator=g, device=device) for _ in range(n_sets)]
    for K in Ks:
        K[:, :, :4] *= MAG
    Ks = [K.bfloat16() for K in Ks]
    Vs = [torch.randn(tokens, HKV, D, generator=g, device=device).bfloat16() for _ in range(n_sets)]
    pls = [alloc_planes(tokens // PAGE, tokens // 32, HKV, D, page_size=PAGE, outliers_per_vector=K_OUT,
                        kv_outlier_map=True, device=device) for _ in range(n_sets)]
    pages = torch.randperm(tokens // PAGE, generator=torch.Generator().manual_seed(1)).to(torch.int32).to(device)
    groups = torch.randperm(tokens // 32, generator=torch.Generator().manual_seed(2)).to(torch.int32).to(device)

    def step():
        for K, V, pl in zip(Ks, Vs, pls):
            ommx_pack_kv_into(K, V, pl, dst_pages=pages, dst_groups=groups, outliers_per_vector=K_OUT)

    steps = max(3, min(args.steps, 10))
    times = timed_graph(step, steps, args.warmup, flush, torch)
    us = sum(times) / len(times) * 1e3 / n_sets
    nbytes = tokens * HKV * D * 4 + tokens * HKV * unit_bytes(K_OUT)
    ach = nbytes / us / 1e3
    return {"config": {"workload": f"bulk quantize + pack of {tokens} tokens x {HKV} kv heads (bf16 K and V in, packed planes out, "
                                   f"{PAGE}-token pages through a random page table); {n_sets} chunks per step, L2 flushed between steps"},
            "us_per_chunk": us, "hbm_gbs": ach,
            "roofline": {"bound": "hbm", "kernel": "pack_k_lane_kernel + pack_v_kernel", "achieved": ach, "peak": peak,
                         "unit": "GB/s", "frac": ach / peak, "algorithmic_bytes_per_chunk": nbytes}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--ctx", type=int, default=HEADLINE_CTX, help="context of the headline value")
    ap.add_argument("--max-ctx", type=int, default=max(CONTEXTS), help="longest context of the per-context table")
    ap.add_argument("--no-all-contexts", dest="all_contexts", action="store_false")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-triton", action="store_true", help="skip timing the reference's Triton kernels")
    ap.add_argument("--no-workloads", action="store_true", help="skip the sub-record workloads")
    ap.add_argument("--gather", default="peer", choices=("peer", "nccl"),
                    help="N > 1: head outputs exchanged by stage 2's peer stores (default) or by an NCCL all-gather")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers in the stack (32 = the benchmark)")
    ap.add_argument("--profile", action="store_true", help="eager launches only, for ncu (use a small --layers)")
    ap.add_argument("--k", type=int, default=K_OUT, help="outliers per K vector (the headline recipe has 6)")
    ap.add_argument("--mag", type=float, default=MAG, help="factor on the 4 outlier channels of every K head")
    args = ap.parse_args()
    globals()["LAYERS"] = args.layers
    globals()["K_OUT"] = args.k
    globals()["MAG"] = args.mag
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(3, args.warmup)
    if args.profile:
        args.all_contexts = False
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
