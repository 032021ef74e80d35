#!/usr/bin/env python
"""Per-op timing at model shapes with roofline fractions.

Each op is captured into a CUDA graph of ``--iters`` launches that rotate over
distinct weight / KV buffers (larger than L2 in total, so every launch streams from
HBM), replayed after warm-up and timed with CUDA events.  Fractions are against the
measured peaks in MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 throughput).

    python bench_ops.py [--only gemm|attn|small] [--iters 16] [--json out.json]
    python bench_ops.py --single gemm:64x4096x4096      # one op, few launches (ncu target)

Plays the role of the reference's kernel/op report binaries
(pegainfer-bench/src/lib.rs:22-273, docs/subsystems/kernels/kernel-op-reports.md).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch

DEV = "cuda:0"


def peaks():
    p = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def time_graph(fn, n_variants, iters, reps=5):
    """fn(i) launches variant i; returns best ms per launch over `reps` graph replays."""
    for i in range(min(n_variants, 3)):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i % n_variants)
    g.replay()
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / iters)
    return best


def gemm_case(t, m, k, iters, lib=False):
    from pegainfer_b200.ops import cuda as K

    nvar = max(2, min(16, int(300e6 // (m * k * 2)) + 1))
    ws = [torch.randn(m, k, device=DEV).bfloat16() * 0.02 for _ in range(nvar)]
    x = torch.randn(t, k, device=DEV).bfloat16()
    out = torch.empty(t, m, device=DEV, dtype=torch.bfloat16)
    if lib:
        fn = lambda i: torch.nn.functional.linear(x, ws[i])
    else:
        fn = lambda i: K.linear(x, ws[i], out=out)
    ms = time_graph(fn, nvar, iters)
    return ms, (m * k + t * k + t * m) * 2, 2.0 * t * m * k


def attn_decode_case(bs, ctx, hq, hkv, d, page, iters):
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    ppb = (ctx + page - 1) // page
    nvar = 4
    npages = bs * ppb + 1
    kvs = [torch.randn(npages, 2, page, hkv, d, device=DEV).bfloat16() for _ in range(nvar)]
    seqs = [SeqStep(rid=i, input_tokens=[0], start_pos=ctx - 1, view=KvView(list(range(1 + i * ppb, 1 + (i + 1) * ppb)), ctx, page)) for i in range(bs)]
    _, meta = build_meta(seqs, page, DEV)
    meta.plan = K.plan_decode_splits(bs, hkv, ctx, DEV)
    q = torch.randn(bs, hq, d, device=DEV).bfloat16()
    out = torch.empty(bs, hq * d, device=DEV, dtype=torch.bfloat16)
    ms = time_graph(lambda i: K.paged_attention(q, kvs[i], meta, out=out), nvar, iters)
    return ms, bs * ctx * hkv * d * 2 * 2, 4.0 * bs * ctx * hq * d


def attn_prefill_case(nseq, qlen, hq, hkv, d, page, iters):
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    ppb = (qlen + page - 1) // page
    kv = torch.randn(nseq * ppb + 1, 2, page, hkv, d, device=DEV).bfloat16()
    seqs = [SeqStep(rid=i, input_tokens=[0] * qlen, start_pos=0, view=KvView(list(range(1 + i * ppb, 1 + (i + 1) * ppb)), qlen, page)) for i in range(nseq)]
    _, meta = build_meta(seqs, page, DEV)
    q = torch.randn(nseq * qlen, hq, d, device=DEV).bfloat16()
    out = torch.empty(nseq * qlen, hq * d, device=DEV, dtype=torch.bfloat16)
    ms = time_graph(lambda i: K.paged_attention(q, kv, meta, out=out), 1, iters)
    return ms, (nseq * qlen * (hq + 2 * hkv) * d * 2 + nseq * qlen * hq * d * 2), 4.0 * nseq * qlen * qlen / 2 * hq * d


def small_cases(iters):
    from pegainfer_b200.ops import cuda as K

    rows = []
    for t, h in ((64, 4096), (4096, 4096), (64, 5120), (64, 7168)):
        x = [torch.randn(t, h, device=DEV).bfloat16() for _ in range(4)]
        r = [torch.randn(t, h, device=DEV).bfloat16() for _ in range(4)]
        w = torch.ones(h, device=DEV).bfloat16()
        ms = time_graph(lambda i: K.add_rms_norm(x[i], r[i], w, 1e-6), 4, iters)
        rows.append((f"add_rms_norm {t}x{h}", ms, t * h * 2 * 4, 0))
    for t, i_ in ((64, 12288), (4096, 12288)):
        gu = [torch.randn(t, 2 * i_, device=DEV).bfloat16() for _ in range(4)]
        ms = time_graph(lambda i: K.swiglu(gu[i]), 4, iters)
        rows.append((f"swiglu {t}x{i_}", ms, t * i_ * 2 * 3, 0))
    for rws, v in ((64, 151936), (256, 151936), (64, 248320)):
        lg = [torch.randn(rws, v, device=DEV).bfloat16() for _ in range(3)]
        ms = time_graph(lambda i: K.argmax(lg[i]), 3, iters)
        rows.append((f"argmax {rws}x{v}", ms, rws * v * 2, 0))
        tp = torch.full((rws,), 0.9, device=DEV)
        tk = torch.full((rws,), 50, dtype=torch.int32, device=DEV)
        one = torch.ones(rws, device=DEV)
        z = torch.zeros(rws, device=DEV)
        u = torch.rand(rws, device=DEV)
        ms = time_graph(lambda i: K.sample(lg[i], one, tk, tp, z, u), 3, max(2, iters // 4))
        rows.append((f"sample(top-k 50, top-p .9) {rws}x{v}", ms, rws * v * 2, 0))
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=16)
    ap.add_argument("--json", default=None)
    ap.add_argument("--single", default=None, help="e.g. gemm:64x4096x4096, attn:64x1152, prefill:4x1024")
    ap.add_argument("--library", action="store_true", help="also time torch/cuBLAS for the GEMM rows")
    args = ap.parse_args()
    hbm, tf, src = peaks()
    rows = []
    if args.single:
        kind, shape = args.single.split(":")
        dims = [int(v) for v in shape.split("x")]
        if kind == "gemm":
            ms, by, fl = gemm_case(*dims, iters=args.iters)
        elif kind == "attn":
            ms, by, fl = attn_decode_case(dims[0], dims[1], 32, 8, 128, 16, args.iters)
        else:
            ms, by, fl = attn_prefill_case(dims[0], dims[1], 32, 8, 128, 16, args.iters)
        rows.append((args.single, ms, by, fl))
    else:
        if args.only in (None, "gemm"):
            shapes = [(64, 6144, 4096), (64, 4096, 4096), (64, 24576, 4096), (64, 4096, 12288), (64, 151936, 4096), (1, 4096, 4096), (16, 24576, 4096), (256, 24576, 4096),
                      (1024, 6144, 4096), (1024, 24576, 4096), (4096, 6144, 4096), (4096, 4096, 4096), (4096, 24576, 4096), (4096, 4096, 12288), (8192, 8192, 8192)]
            for t, m, k in shapes:
                ms, by, fl = gemm_case(t, m, k, args.iters)
                rows.append((f"gemm T{t} M{m} K{k}", ms, by, fl))
                if args.library:
                    ms2, _, _ = gemm_case(t, m, k, args.iters, lib=True)
                    rows.append((f"  cuBLAS T{t} M{m} K{k}", ms2, by, fl))
        if args.only in (None, "attn"):
            for bs, ctx in ((64, 1152), (1, 1152), (16, 1152), (256, 1152), (64, 4096)):
                ms, by, fl = attn_decode_case(bs, ctx, 32, 8, 128, 16, args.iters)
                rows.append((f"decode attn bs{bs} ctx{ctx} 32q/8kv hd128", ms, by, fl))
            ms, by, fl = attn_decode_case(32, 2304, 24, 4, 256, 16, args.iters)
            rows.append(("decode attn bs32 ctx2304 24q/4kv hd256", ms, by, fl))
            for ns, ql in ((4, 1024), (1, 4096)):
                ms, by, fl = attn_prefill_case(ns, ql, 32, 8, 128, 16, max(2, args.iters // 4))
                rows.append((f"prefill attn {ns}x{ql} 32q/8kv hd128", ms, by, fl))
        if args.only in (None, "small"):
            rows.extend(small_cases(args.iters))
    out = []
    print(f"{'op':58s} {'us':>9s} {'GB/s':>8s} {'%HBM':>6s} {'TFLOP/s':>8s} {'%bf16':>6s}   (peaks: {src} {hbm:.0f} GB/s, {tf:.0f} TFLOP/s)")
    for name, ms, by, fl in rows:
        gbs = by / ms / 1e6
        tfl = fl / ms / 1e9
        print(f"{name:58s} {ms * 1e3:9.1f} {gbs:8.0f} {100 * gbs / hbm:6.1f} {tfl:8.1f} {100 * tfl / tf:6.1f}")
        out.append(dict(op=name, us=ms * 1e3, gbs=gbs, frac_hbm=gbs / hbm, tflops=tfl, frac_bf16=tfl / tf, peaks=src))
    if args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)), exist_ok=True)
        json.dump(out, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
