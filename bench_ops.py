#!/usr/bin/env python
"""Per-op timing at model shapes with roofline fractions.

Each op is captured into a CUDA graph of ``--iters`` launches that rotate over
distinct weight / KV buffers (larger than L2 in total, so every launch streams from
HBM), replayed after warm-up and timed with CUDA events.  Fractions are against the
measured peaks in MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 throughput).

    python bench_ops.py [--only gemm|attn|small|gdn|kda|moe|mla] [--iters 16] [--json out.json]
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


def gemm_case(t, m, k, iters, lib=False, mode="auto"):
    from pegainfer_b200.ops import cuda as K

    nvar = max(2, min(16, int(300e6 // (m * k * 2)) + 1))
    ws = [torch.randn(m, k, device=DEV).bfloat16() * 0.02 for _ in range(nvar)]
    x = torch.randn(t, k, device=DEV).bfloat16()
    out = torch.empty(t, m, device=DEV, dtype=torch.bfloat16)
    if lib:
        fn = lambda i: torch.nn.functional.linear(x, ws[i])
    elif mode == "one_cta":  # a pinned split count keeps the problem on the one-CTA kernel
        fn = lambda i: K.linear(x, ws[i], out=out, force_splits=1)
    elif mode == "two_sm":
        fn = lambda i: K.linear_2sm(x, ws[i])
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


def _meta_for(q_lens, kv_lens, page):
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    seqs, nxt = [], 1
    for i, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        npg = (kl + page - 1) // page
        seqs.append(SeqStep(rid=i, input_tokens=[0] * ql, start_pos=kl - ql, view=KvView(list(range(nxt, nxt + npg)), kl, page)))
        nxt += npg
    _, meta = build_meta(seqs, page, DEV)
    return meta, nxt


def gdn_cases(iters, only=None):
    """Gated DeltaNet recurrence at the Qwen3.5-27B shape (16 K-heads, 48 V-heads, 128x128 state)."""
    from pegainfer_b200.ops import cuda as K

    rows = []
    hk, hv, dk, dv = 16, 48, 128, 128
    for name, q_lens in only or (("decode bs32", [1] * 32), ("decode bs64", [1] * 64), ("prefill 1x2048", [2048]), ("prefill 8x2048", [2048] * 8)):
        meta, _ = _meta_for(q_lens, q_lens, 16)
        meta.state_slots = torch.arange(len(q_lens), dtype=torch.int32, device=DEV)
        t = sum(q_lens)
        q = torch.randn(t, hk, dk, device=DEV).bfloat16()
        k = torch.randn(t, hk, dk, device=DEV).bfloat16()
        v = torch.randn(t, hv, dv, device=DEV).bfloat16()
        g = -torch.rand(t, hv, device=DEV) * 0.1
        beta = torch.rand(t, hv, device=DEV)
        states = [torch.zeros(len(q_lens), hv, dk, dv, device=DEV) for _ in range(3)]
        ms = time_graph(lambda i: K.gdn_recurrent(q, k, v, g, beta, states[i], meta), 3, max(2, iters // 4))
        state_bytes = len(q_lens) * hv * dk * dv * 4 * 2
        rows.append((f"gdn_recurrent {name} 48vh 128x128", ms, state_bytes + t * (2 * hk * dk + 2 * hv * dv) * 2, 4.0 * t * hv * dk * dv * 2))
        if max(q_lens) >= 64:  # the row above ran the chunk-wise scan; this one the token-by-token kernel
            ms = time_graph(lambda i: K.gdn_recurrent(q, k, v, g, beta, states[i], meta, chunked=False), 3, max(2, iters // 4))
            rows.append((f"  recurrence kernel {name}", ms, state_bytes + t * (2 * hk * dk + 2 * hv * dv) * 2, 4.0 * t * hv * dk * dv * 2))
    return rows


def kda_cases(iters, only=None):
    """KDA recurrence (decay per key channel, gate arithmetic in the kernel) and the attention-residual mix at the Kimi-K3
    shape: 96 heads with a 128x128 f32 state, hidden 7168, 8 snapshots."""
    from pegainfer_b200.ops import cuda as K

    rows = []
    heads, d, hidden = 96, 128, 7168
    inner = heads * d
    for name, q_lens in only or (("decode bs32", [1] * 32), ("decode bs64", [1] * 64), ("prefill 1x2048", [2048])):
        meta, _ = _meta_for(q_lens, q_lens, 16)
        meta.state_slots = torch.arange(len(q_lens), dtype=torch.int32, device=DEV)
        t = sum(q_lens)
        qkv = torch.randn(t, 3 * inner, device=DEV).bfloat16()
        q, k, v = (qkv[:, j * inner : (j + 1) * inner].view(t, heads, d) for j in range(3))
        f, b = torch.randn(t, inner, device=DEV).bfloat16(), torch.randn(t, heads, device=DEV).bfloat16()
        a_log, dt = torch.zeros(heads, device=DEV), torch.zeros(inner, device=DEV)
        states = [torch.zeros(len(q_lens), heads, d, d, device=DEV) for _ in range(3)]
        ms = time_graph(lambda i: K.kda_recurrent(q, k, v, f, b, a_log, dt, -5.0, states[i], meta), 3, max(2, iters // 4))
        rows.append((f"kda_recurrent {name} 96h 128x128", ms, len(q_lens) * heads * d * d * 4 * 2 + t * 5 * inner * 2, 4.0 * t * heads * d * d * 2))
    for t, nb in ((64, 8), (4096, 8)):
        cur = [torch.randn(t, hidden, device=DEV).bfloat16() for _ in range(3)]
        snaps = [torch.randn(t, 8, hidden, device=DEV).bfloat16() for _ in range(3)]
        sw = torch.randn(hidden, device=DEV)
        ms = time_graph(lambda i: K.attnres_mix(cur[i], snaps[i], nb, sw, 1e-5), 3, iters)
        rows.append((f"attnres_mix {t}x{hidden} {nb} snapshots", ms, t * hidden * 2 * (nb + 2), 0))
    return rows


def moe_cases(iters):
    """Routed-expert pipeline (align, gather, W13, SwiGLU, W2, combine) on one GPU."""
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.ops import reference as R

    rows = []
    for name, t, h, inter, e, k, quant in (("dsv2-lite bf16 64 exp top-6", 64, 2048, 1408, 64, 6, "bf16"), ("dsv2-lite fp8 64 exp top-6", 64, 2048, 1408, 64, 6, "fp8"),
                                            ("kimi-k2 int4 48 local exp top-8 (EP8 share)", 128, 7168, 2048, 48, 8, "int4")):
        x = torch.randn(t, h, device=DEV).bfloat16() * 0.5
        ids, w = R.router_topk(torch.randn(t, e, device=DEV), k, "softmax")
        nvar = 3
        if quant == "bf16":
            ws = [(torch.randn(e, 2 * inter, h, device=DEV).bfloat16() * 0.02, torch.randn(e, h, inter, device=DEV).bfloat16() * 0.02) for _ in range(nvar)]
            fn = lambda i: K.moe_experts(x, ids, w, ws[i][0], ws[i][1], 0)
            wbytes = e * 3 * inter * h * 2
        elif quant == "fp8":
            ws = [((torch.randn(e, 2 * inter, h, device=DEV) * 100).clamp(-448, 448).to(torch.float8_e4m3fn), torch.full((e, 2 * inter // 128, h // 128), 2e-4, device=DEV),
                   (torch.randn(e, h, inter, device=DEV) * 100).clamp(-448, 448).to(torch.float8_e4m3fn), torch.full((e, h // 128, inter // 128), 2e-4, device=DEV)) for _ in range(nvar)]
            fn = lambda i: K.moe_experts_fp8(x, ids, w, ws[i][0], ws[i][1], ws[i][2], ws[i][3], 0)
            wbytes = e * 3 * inter * h
        else:
            ws = [(torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, 2 * inter, h // 8), dtype=torch.int32, device=DEV), (torch.rand(e, 2 * inter, h // 32, device=DEV) * 0.004).bfloat16(),
                   torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, h, inter // 8), dtype=torch.int32, device=DEV), (torch.rand(e, h, inter // 32, device=DEV) * 0.004).bfloat16()) for _ in range(nvar)]
            fn = lambda i: K.moe_experts_int4(x, ids, w, ws[i][0], ws[i][1], ws[i][2], ws[i][3], 0)
            wbytes = e * 3 * inter * h // 2 + e * 3 * inter * h // 32 * 2
        ms = time_graph(fn, nvar, max(2, iters // 4))
        rows.append((f"moe experts {name} T{t}", ms, wbytes, 2.0 * t * k * 3 * inter * h))
    return rows


def mla_cases(iters):
    """Absorbed MLA decode attention over the paged latent cache (512 + 64 wide)."""
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.ops import reference as R

    rows = []
    c, rope, nope, vd = 512, 64, 128, 128
    for heads, bs, ctx in ((16, 64, 640), (64, 16, 1152), (64, 128, 1152)):
        meta, npages = _meta_for([1] * bs, [ctx] * bs, 16)
        latents = [torch.randn(npages, 16, c + rope, device=DEV).bfloat16() * 0.5 for _ in range(3)]
        q = torch.randn(bs, heads, nope + rope, device=DEV).bfloat16() * 0.5
        w_uk = torch.randn(heads, nope, c, device=DEV).bfloat16() * 0.05
        w_uv = torch.randn(heads, vd, c, device=DEV).bfloat16() * 0.05
        cos, sin = R.rope_tables(4096, rope, 10000.0, torch.bfloat16, DEV)
        qq = K.mla_rope_q(q, cos, sin, meta, nope)
        scale = (nope + rope) ** -0.5
        ms = time_graph(lambda i: K.mla_attention(qq, w_uk, w_uv, latents[i], meta, scale, c), 3, max(2, iters // 4))
        rows.append((f"mla decode (absorb + attn + v_up) {heads}h bs{bs} ctx{ctx}", ms, bs * ctx * (c + rope) * 2, 2.0 * bs * ctx * heads * (c + rope + c)))
    return rows


def time_eager(fn, iters, warm=3):
    """ms per call of a host-driven op (not graph-capturable: it uploads small index tensors), CUDA events around `iters` calls."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def mla_prefill_cases(iters, only=None):
    """MLA prefill, whole op (query absorb or K / V expansion included): the expanded form on the tcgen05 kernel against
    the absorbed form on the mma.sync kernel.  FLOPs counted in the expanded form: causal 4 x (192 + 128) / 2 per pair."""
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.ops import reference as R

    rows = []
    c, rope, nope, vd = 512, 64, 128, 128
    for heads, ns, ql in only or ((16, 4, 1024), (16, 1, 4096), (16, 1, 8192), (64, 1, 4096)):
        meta, npages = _meta_for([ql] * ns, [ql] * ns, 16)
        latent = torch.randn(npages, 16, c + rope, device=DEV).bfloat16() * 0.5
        q = torch.randn(ns * ql, heads, nope + rope, device=DEV).bfloat16() * 0.5
        w_uk = torch.randn(heads, nope, c, device=DEV).bfloat16() * 0.05
        w_uv = torch.randn(heads, vd, c, device=DEV).bfloat16() * 0.05
        cos, sin = R.rope_tables(max(4096, ql), rope, 10000.0, torch.bfloat16, DEV)
        qq = K.mla_rope_q(q, cos, sin, meta, nope)
        scale = (nope + rope) ** -0.5
        fl = 2.0 * ns * (ql * ql / 2) * heads * (nope + rope + vd)
        by = ns * ql * (c + rope) * 2
        ms = time_eager(lambda: K.mla_attention(qq, w_uk, w_uv, latent, meta, scale, c), max(2, iters // 2))
        rows.append((f"mla prefill {heads}h {ns}x{ql}, expanded on tcgen05 (gather + expand GEMMs + attention)", ms, by, fl))
        prev = K._PREFILL_TC
        K._PREFILL_TC = False
        try:
            ms = time_eager(lambda: K.mla_attention(qq, w_uk, w_uv, latent, meta, scale, c), max(2, iters // 4))
        finally:
            K._PREFILL_TC = prev
        rows.append((f"  absorbed on mma.sync (absorb GEMM + attention over 576 / 512 + v_up)", ms, by, fl))
    return rows


GEMM_PHASES = ["entry", "prologue done", "predecessor complete", "all loads issued", "first stage landed", "last MMA committed", "accumulator ready",
               "partial pushed", "cluster partials in", "reduced + stored", "roles done", "cluster released", "token tiles issued", "second stage landed", "seventh stage landed"]


def chain_case(t, h, inter, qkv, iters):
    """The four projections behind attention of one dense layer (o_proj + residual + norm weight, gate_up + SwiGLU,
    down + residual + norm weight, next qkv) as ONE persistent kernel; bytes = the four weight matrices."""
    from pegainfer_b200.ops import cuda as K

    nvar = 6
    ws = [dict(wo=(torch.randn(h, h, device=DEV) * 0.03).bfloat16(), gu=(torch.randn(2 * inter, h, device=DEV) * 0.03).bfloat16(), wd=(torch.randn(h, inter, device=DEV) * 0.02).bfloat16(),
               wq=(torch.randn(qkv, h, device=DEV) * 0.03).bfloat16()) for _ in range(nvar)]
    a = (torch.randn(t, h, device=DEV) * 0.5).bfloat16()
    n1 = torch.ones(h, device=DEV).bfloat16()
    res = torch.randn(t, h, device=DEV).bfloat16()

    def fn(i):
        w = ws[i]
        return K.decode_chain(a, [(w["wo"], K.CH_RESID_NORM, n1, False), (w["gu"], K.CH_SWIGLU, None, False), (w["wd"], K.CH_RESID_NORM, n1, False), (w["wq"], K.CH_PLAIN, None, False)],
                              residual=res, eps=1e-6)

    ms = time_graph(fn, nvar, iters)
    return ms, (h * h + 2 * inter * h + h * inter + qkv * h) * 2, 2.0 * t * (h * h + 2 * inter * h + h * inter + qkv * h)


def fp8_cases(iters, only=None):
    """Block-scaled FP8 GEMM (kind::f8f6f4) on decode shapes, with and without the activation quantiser; bytes
    count the e4m3 weights once."""
    from pegainfer_b200.loader.export import quantize_dense_to_fp8
    from pegainfer_b200.ops import cuda as K

    rows = []
    for t, m, k in only or ((64, 6144, 4096), (64, 24576, 4096), (64, 4096, 12288), (16, 24576, 4096), (64, 12288, 6144)):
        nvar = max(2, min(16, int(300e6 // (m * k)) + 1))
        ws = []
        for i in range(nvar):
            d = {"w": torch.randn(m, k) * 0.05}
            quantize_dense_to_fp8(d, ["w"])
            ws.append((d["w"].to(DEV).contiguous(), d["w_scale_inv"].to(DEV).contiguous()))
        x = torch.randn(t, k, device=DEV).bfloat16()
        xq, xs = K.quant_fp8_1x128(x)
        ms = time_graph(lambda i: K.linear_fp8_block(x, ws[i][0], ws[i][1], xq, xs), nvar, iters)
        rows.append((f"fp8 gemm T{t} M{m} K{k} (pre-quantised x)", ms, m * k + t * k + t * m * 2, 2.0 * t * m * k))
        ms = time_graph(lambda i: K.linear_fp8_block(x, ws[i][0], ws[i][1]), nvar, iters)
        rows.append((f"  with activation quantiser", ms, m * k + t * k * 3 + t * m * 2, 2.0 * t * m * k))
    return rows


def dsa_cases(iters, only=None):
    """Sparse-attention indexer on GLM-5 shapes (32 index heads x 128, keep 2048): tcgen05 scores, radix top-k, and the
    gathered sparse latent attention (64 heads, latent 512 + 64) at one decode row per sequence."""
    from pegainfer_b200.ops import cuda as K

    rows = []
    page, heads, d = 64, 32, 128
    for bs, ctx in only or ((16, 16384), (64, 8192), (64, 32768)):
        meta, npages = _meta_for([1] * bs, [ctx] * bs, page)
        cache = (torch.randn(npages, page, d, device=DEV) * 0.5).bfloat16()
        q = (torch.randn(bs, heads, d, device=DEV) * 0.3).bfloat16()
        w = (torch.randn(bs, heads, device=DEV) * 0.2).float()
        ms = time_graph(lambda i: K.dsa_index_scores(q, w, cache, meta), 1, iters)
        rows.append((f"dsa index scores bs{bs} ctx{ctx} 32h x 128", ms, bs * ctx * d * 2 + bs * ctx * 4, 2.0 * bs * ctx * heads * d))
        sc = K.dsa_index_scores(q, w, cache, meta)
        ms = time_graph(lambda i: K.dsa_topk(sc, 2048), 1, iters)
        rows.append((f"dsa top-2048 bs{bs} ctx{ctx}", ms, bs * ctx * 4 * 5, 0))
        sel = K.dsa_topk(sc, 2048)
        H, nope, vdim, c, rope = 64, 192, 256, 512, 64
        latent = (torch.randn(npages, page, c + rope, device=DEV) * 0.3).bfloat16()
        cos, sin = __import__("pegainfer_b200.ops.reference", fromlist=["rope_tables"]).rope_tables(ctx + 8, rope, 1e4, torch.bfloat16, DEV)
        qm = K.mla_rope_q((torch.randn(bs, H, nope + rope, device=DEV) * 0.3).bfloat16(), cos, sin, meta, nope)
        w_uk, w_uv = (torch.randn(H, nope, c, device=DEV) * 0.05).bfloat16(), (torch.randn(H, vdim, c, device=DEV) * 0.05).bfloat16()
        ms = time_graph(lambda i: K.mla_attention_sparse(qm, w_uk, w_uv, latent, meta, 0.0625, c, sel), 1, max(2, iters // 2))
        rows.append((f"sparse mla decode (gather + attn) bs{bs} keep 2048 of {ctx}", ms, bs * 2048 * (c + rope) * 2 * 3, 2.0 * bs * 2048 * H * (c + rope + c)))
        ms = time_graph(lambda i: K.mla_attention(qm, w_uk, w_uv, latent, meta, 0.0625, c), 1, max(2, iters // 4))
        rows.append((f"  dense mla decode over all {ctx} keys", ms, bs * ctx * (c + rope) * 2, 2.0 * bs * ctx * H * (c + rope + c)))
        del cache, latent
    return rows


def gemm_phase_timeline(t, m, k):
    """Per-CTA globaltimer stamps of one eager GEMM launch with cold L2 (profiling hook of the
    GEMM kernel): min / median / max over the CTAs, microseconds from the first CTA's entry."""
    import ctypes

    import numpy as np

    from pegainfer_b200 import _native
    from pegainfer_b200.ops import cuda as K

    lib = _native.load()
    x = (torch.randn(t, k, device=DEV) * 0.1).bfloat16()
    ws = [(torch.randn(m, k, device=DEV) * 0.02).bfloat16() for _ in range(4)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    timing = torch.zeros(148 * 16, dtype=torch.int64, device=DEV)
    for w in ws:
        K.linear(x, w)
    torch.cuda.synchronize()
    plan = K.gemm_plan(t, m, k)
    rows = None
    for rep in range(3):
        flush.zero_()
        timing.zero_()
        torch.cuda.synchronize()
        lib.pg_gemm_set_timing(ctypes.c_void_p(timing.data_ptr()))
        K.linear(x, ws[rep])
        torch.cuda.synchronize()
        lib.pg_gemm_set_timing(ctypes.c_void_p(0))
        tm = timing.view(148, 16).cpu().numpy().astype(np.float64)[: plan["grid"]]
        t0 = tm[:, 0].min()
        rows = []
        for i, name in enumerate(GEMM_PHASES):
            col = tm[:, i]
            col = col[col > 0]
            if len(col):
                rows.append((name, (col.min() - t0) / 1e3, (np.median(col) - t0) / 1e3, (col.max() - t0) / 1e3))
    print(f"gemm T{t} M{m} K{k}: plan {plan}")
    print(f"{'phase':26s} {'min us':>8s} {'median':>8s} {'max':>8s}")
    for name, a, b, c in rows:
        print(f"{name:26s} {a:8.2f} {b:8.2f} {c:8.2f}")


def gemm_phase_timeline_steady(t, m, k, launches=8):
    """The same stamps in steady state: a CUDA graph of ``launches`` back-to-back GEMMs (rotating
    weights, programmatic dependent launch between them), every launch writing its own stamp
    buffer.  Printed per phase: median over the CTAs, microseconds from the exit of the previous
    launch's last CTA (negative = overlapped with the predecessor)."""
    import ctypes

    import numpy as np

    from pegainfer_b200 import _native
    from pegainfer_b200.ops import cuda as K

    lib = _native.load()
    x = (torch.randn(t, k, device=DEV) * 0.1).bfloat16()
    nvar = max(2, min(16, int(300e6 // (m * k * 2)) + 1))
    ws = [(torch.randn(m, k, device=DEV) * 0.02).bfloat16() for _ in range(nvar)]
    out = torch.empty(t, m, device=DEV, dtype=torch.bfloat16)
    timing = torch.zeros(launches, 148 * 16, dtype=torch.int64, device=DEV)
    for w in ws[:3]:
        K.linear(x, w, out=out)
    torch.cuda.synchronize()
    plan = K.gemm_plan(t, m, k)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(launches):
            lib.pg_gemm_set_timing(ctypes.c_void_p(timing[i].data_ptr()))
            K.linear(x, ws[i % nvar], out=out)
    lib.pg_gemm_set_timing(ctypes.c_void_p(0))
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    tm = timing.view(launches, 148, 16).cpu().numpy().astype(np.float64)[:, : plan["grid"]]
    print(f"gemm T{t} M{m} K{k}: plan {plan}; steady state, launch i relative to the exit of launch i-1")
    print(f"{'phase':26s} " + " ".join(f"{'L%d' % i:>8s}" for i in range(2, launches)))
    ends = [max(tm[i][:, 11].max(), tm[i][:, 10].max()) for i in range(launches)]
    for j, name in enumerate(GEMM_PHASES):
        vals = []
        for i in range(2, launches):
            col = tm[i][:, j]
            col = col[col > 0]
            vals.append((np.median(col) - ends[i - 1]) / 1e3 if len(col) else float("nan"))
        print(f"{name:26s} " + " ".join(f"{v:8.2f}" for v in vals))
    per = [(ends[i] - ends[i - 1]) / 1e3 for i in range(2, launches)]
    print(f"{'exit to exit':26s} " + " ".join(f"{v:8.2f}" for v in per))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=16)
    ap.add_argument("--json", default=None)
    ap.add_argument("--single", default=None, help="e.g. gemm:64x4096x4096, attn:64x1152, prefill:4x1024, prefill256:1x4096, prefill512:4x1024, decode512:64x1152, gdn:8x2048 (sequences x tokens), chain:64x4096x12288x6144 (tokens x hidden x ffn x qkv), "
                    "fp8:64x24576x4096, dsa:16x16384 (sequences x context)")
    ap.add_argument("--library", action="store_true", help="also time torch/cuBLAS for the GEMM rows")
    ap.add_argument("--phases", default=None, help="gemm:TxMxK: print the per-CTA phase timeline of one GEMM launch")
    ap.add_argument("--phases-steady", default=None, help="gemm:TxMxK: the same stamps for back-to-back launches inside one CUDA graph")
    args = ap.parse_args()
    hbm, tf, src = peaks()
    rows = []
    if args.phases:
        gemm_phase_timeline(*[int(v) for v in args.phases.split(":")[1].split("x")])
        return
    if args.phases_steady:
        gemm_phase_timeline_steady(*[int(v) for v in args.phases_steady.split(":")[1].split("x")])
        return
    if args.single:
        kind, shape = args.single.split(":")
        dims = [int(v) for v in shape.split("x")]
        if kind in ("gemm", "gemm2sm", "gemm1cta"):
            ms, by, fl = gemm_case(*dims, iters=args.iters, mode={"gemm": "auto", "gemm2sm": "two_sm", "gemm1cta": "one_cta"}[kind])
        elif kind == "gdn":
            name, ms, by, fl = gdn_cases(args.iters, only=[("single", [dims[1]] * dims[0])])[0]
        elif kind == "chain":
            ms, by, fl = chain_case(dims[0], dims[1], dims[2], dims[3], args.iters)
        elif kind == "fp8":
            name, ms, by, fl = [r for r in fp8_cases(args.iters, only=[tuple(dims)])][0]
        elif kind == "dsa":
            name, ms, by, fl = dsa_cases(args.iters, only=[tuple(dims)])[0]
        elif kind == "attn":
            ms, by, fl = attn_decode_case(dims[0], dims[1], 32, 8, 128, 16, args.iters)
        elif kind == "mlaprefill":  # heads x sequences x tokens
            r2 = mla_prefill_cases(args.iters, only=[tuple(dims)])
            rows.extend(r2[:-1])
            name, ms, by, fl = r2[-1]
            args.single = name
        elif kind == "prefill512":  # global layers of the Gemma 4 line: 32 query / 4 KV heads of 512 (plain CUDA cores)
            ms, by, fl = attn_prefill_case(dims[0], dims[1], 32, 4, 512, 16, args.iters)
        elif kind == "decode512":
            ms, by, fl = attn_decode_case(dims[0], dims[1], 32, 4, 512, 16, args.iters)
        elif kind == "prefill256":  # the gated full-attention layers of Qwen3.5-27B: 24 query / 4 KV heads of 256
            ms, by, fl = attn_prefill_case(dims[0], dims[1], 24, 4, 256, 16, args.iters)
        else:
            ms, by, fl = attn_prefill_case(dims[0], dims[1], 32, 8, 128, 16, args.iters)
        rows.append((args.single, ms, by, fl))
    else:
        if args.only in (None, "chain"):
            for t in (64, 16):
                ms, by, fl = chain_case(t, 4096, 12288, 6144, args.iters)
                rows.append((f"decode chain T{t} (o, gate_up, down, qkv of Qwen3-8B)", ms, by, fl))
        if args.only in (None, "gemm"):
            shapes = [(64, 6144, 4096), (64, 4096, 4096), (64, 24576, 4096), (64, 4096, 12288), (64, 151936, 4096), (1, 4096, 4096), (16, 24576, 4096), (256, 24576, 4096),
                      (1024, 6144, 4096), (1024, 24576, 4096), (4096, 6144, 4096), (4096, 4096, 4096), (4096, 24576, 4096), (4096, 4096, 12288), (8192, 8192, 8192)]
            for t, m, k in shapes:
                ms, by, fl = gemm_case(t, m, k, args.iters)
                rows.append((f"gemm T{t} M{m} K{k}", ms, by, fl))
                if t >= 256:
                    ms1, _, _ = gemm_case(t, m, k, args.iters, mode="one_cta")
                    rows.append((f"  one-CTA kernel T{t} M{m} K{k}", ms1, by, fl))
                    if t < 512:
                        ms2, _, _ = gemm_case(t, m, k, args.iters, mode="two_sm")
                        rows.append((f"  two-SM kernel T{t} M{m} K{k}", ms2, by, fl))
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
        if args.only in (None, "gdn"):
            rows.extend(gdn_cases(args.iters))
        if args.only in (None, "kda"):
            rows.extend(kda_cases(args.iters))
        if args.only in (None, "moe"):
            rows.extend(moe_cases(args.iters))
        if args.only in (None, "mla"):
            rows.extend(mla_cases(args.iters))
        if args.only in (None, "fp8"):
            rows.extend(fp8_cases(args.iters))
        if args.only in (None, "dsa"):
            rows.extend(dsa_cases(args.iters))
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
