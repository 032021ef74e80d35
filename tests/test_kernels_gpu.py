"""sm_100a kernels against the PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch

from pegainfer_b200 import ops
from pegainfer_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def cu():
    from pegainfer_b200.ops import cuda

    return cuda


def bf16_close(a, b, rel=2 ** -7, abs_=1e-3):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = abs_ + rel * b.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{bad}/{a.numel()} elements off; max err {err.max().item():.4g}"


def status_clean():
    assert cu().read_status(DEV) == 0, f"device status word {cu().read_status(DEV):#x}"


@pytest.mark.parametrize(
    "t,m,k",
    [(1, 256, 128), (7, 384, 264), (16, 128, 64), (33, 1000, 520), (64, 4096, 4096), (64, 6144, 4096), (200, 512, 1024), (300, 1536, 2048), (1024, 2048, 1024)],
)
def test_gemm_matches_fp32(t, m, k):
    torch.manual_seed(t * 7 + m)
    x = (torch.randn(t, k, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(m, k, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().t()
    y = cu().linear(x, w)
    torch.cuda.synchronize()
    status_clean()
    assert y.shape == (t, m) and y.dtype == torch.bfloat16
    err = (y.float() - ref).abs()
    tol = 2 ** -7 * ref.abs() + 2e-2 * math.sqrt(k / 1024)
    assert (err <= tol).all(), f"max err {err.max().item()} (ref max {ref.abs().max().item()})"
    yf = cu().linear(x, w, out_dtype=torch.float32)
    assert (yf - ref).abs().max().item() < 1e-2 * math.sqrt(k / 64)
    # bit-identical rerun, also with a pinned split count
    assert torch.equal(y, cu().linear(x, w))
    for s in (1, 2, 3):
        if k // 64 >= s:
            ys = cu().linear(x, w, force_splits=s)
            assert (ys.float() - ref).abs().max().item() <= tol.max().item() * 2
    status_clean()


@pytest.mark.parametrize("t,m,k", [(256, 256, 64), (512, 1024, 256), (300, 700, 520), (1000, 1500, 1032), (2048, 4096, 4096), (4096, 6144, 1024), (777, 151936 // 16, 512), (1024, 6144, 512), (640, 2048, 256), (900, 1024, 320)])
def test_gemm_two_sm_pair_tiles(t, m, k):
    """cta_group::2 kernel (a CTA pair per 256 x 256 tile) called directly: full tiles, ragged
    edges in both dimensions, several tiles per pair (both accumulator buffers, ring wrap)."""
    torch.manual_seed(t + m + k)
    x = (torch.randn(t, k, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(m, k, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().t()
    y = cu().linear_2sm(x, w)
    torch.cuda.synchronize()
    status_clean()
    err = (y.float() - ref).abs()
    tol = 2 ** -7 * ref.abs() + 2e-2 * math.sqrt(max(k, 1024) / 1024)
    assert (err <= tol).all(), f"max err {err.max().item()} (ref max {ref.abs().max().item()})"
    assert torch.equal(y, cu().linear_2sm(x, w))
    # a strided activation view (row stride larger than K) goes through the tensor map
    big = (torch.randn(t, k + 64, device=DEV) * 0.5).bfloat16()
    y2 = cu().linear_2sm(big[:, :k], w)
    assert (y2.float() - big[:, :k].float() @ w.float().t()).abs().max().item() < 0.1 * math.sqrt(max(k, 1024) / 1024)
    status_clean()


@pytest.mark.parametrize("t,m,k,s", [(64, 4096, 4096, 4), (50, 1000, 2048, 8), (16, 24576, 1024, 3), (64, 24576, 4096, 0), (8, 30000, 512, 5), (64, 4096, 12288, 7), (33, 128, 8192, 6)])
def test_gemm_cluster_split_k(t, m, k, s):
    """Narrow token tiles reduce their k-splits across a thread-block cluster (several rounds per cluster included)."""
    torch.manual_seed(m + k)
    x = (torch.randn(t, k, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(m, k, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().t()
    tol = 2 ** -7 * ref.abs() + 2e-2 * math.sqrt(k / 1024)
    y = cu().linear(x, w, force_splits=s)
    y2 = cu().linear(x, w, force_splits=s)
    yf = cu().linear(x, w, out_dtype=torch.float32, force_splits=s)
    torch.cuda.synchronize()
    status_clean()
    assert ((y.float() - ref).abs() <= tol).all(), f"max err {(y.float() - ref).abs().max().item()}"
    assert torch.equal(y, y2)
    assert (yf - ref).abs().max().item() < 1e-2 * math.sqrt(k / 64)


def test_gemm_strided_input_and_batch_invariance():
    torch.manual_seed(0)
    k, m = 1024, 768
    big = (torch.randn(96, 2 * k, device=DEV) * 0.3).bfloat16()
    x = big[:, :k]  # row stride 2k
    w = (torch.randn(m, k, device=DEV) * 0.05).bfloat16()
    y = cu().linear(x, w, force_splits=2)
    ref = x.float() @ w.float().t()
    bf16_close(y, ref, rel=2 ** -6, abs_=3e-2)
    # a row's result must not depend on how many other rows ride along
    y1 = cu().linear(x[5:6], w, force_splits=2)
    y40 = cu().linear(x[:40], w, force_splits=2)
    assert torch.equal(y1[0], y[5]) and torch.equal(y40[5], y[5])
    status_clean()


@pytest.mark.parametrize("width", [256, 2048, 4096, 5120, 7168])
@pytest.mark.parametrize("offset", [False, True])
def test_rms_norm_and_fused_add(width, offset):
    torch.manual_seed(width)
    x = torch.randn(37, width, device=DEV).bfloat16()
    res = torch.randn(37, width, device=DEV).bfloat16()
    w = (torch.randn(width, device=DEV) * 0.2 + (0 if offset else 1)).bfloat16()
    bf16_close(cu().rms_norm(x, w, 1e-6, offset), R.rms_norm(x, w, 1e-6, offset), rel=2 ** -7)
    for rb in (True, False):
        r1, r2 = res.clone(), res.clone()
        y1 = cu().add_rms_norm(x, r1, w, 1e-6, offset, rb)
        y2 = R.add_rms_norm(x, r2, w, 1e-6, offset, rb)
        assert torch.equal(r1, r2)
        bf16_close(y1, y2, rel=2 ** -7)


def test_swiglu_gather_gated_norm():
    torch.manual_seed(3)
    gu = torch.randn(50, 2 * 1408, device=DEV).bfloat16() * 2
    bf16_close(cu().swiglu(gu), R.swiglu(gu), rel=2 ** -7)
    table = torch.randn(1000, 512, device=DEV).bfloat16()
    ids = torch.randint(0, 1000, (77,), device=DEV, dtype=torch.int32)
    assert torch.equal(cu().gather_rows(table, ids), table[ids.long()])
    x = torch.randn(9, 6, 128, device=DEV).bfloat16()
    g = torch.randn(9, 6, 128, device=DEV).bfloat16()
    w = torch.rand(128, device=DEV) + 0.5
    bf16_close(cu().gated_rms_norm(x, g, w, 1e-6), R.gated_rms_norm(x, g, w, 1e-6), rel=2 ** -6)
    status_clean()


def make_batch(q_lens, kv_lens, page_size, hkv, d, extra_pages=3, pad=0):
    """Random paged KV + metadata for sequences with the given query / KV lengths."""
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    n_pages = sum((l + page_size - 1) // page_size for l in kv_lens) + extra_pages + 1
    perm = (torch.randperm(n_pages - 1) + 1).tolist()
    seqs, p = [], 0
    for ql, kl in zip(q_lens, kv_lens):
        npg = (kl + page_size - 1) // page_size
        pages = perm[p : p + npg]
        p += npg
        seqs.append(SeqStep(rid=len(seqs), input_tokens=[0] * ql, start_pos=kl - ql, view=KvView(pages, kl, page_size)))
    kv = torch.randn(n_pages, 2, page_size, hkv, d, device=DEV).bfloat16()
    _, meta = build_meta(seqs, page_size, DEV, pad_to=len(seqs) + pad)
    return kv, meta


@pytest.mark.parametrize("hq,hkv,page", [(8, 2, 16), (8, 1, 64), (4, 4, 16)])
def test_wide_head_attention_hd512(hq, hkv, page):
    """Head dim 512 (the global layers of the Gemma 4 line): prefill chunks, decode rows and padding rows through the
    one-block-per-(row, KV head) kernel, with scale 1 on normalised rows and with a sliding window."""
    torch.manual_seed(hq)
    d = 512
    q_lens = [1, 64, 65, 130, 1, 17]
    kv_lens = [40, 64, 200, 130, 1, 300]
    kv, meta = make_batch(q_lens, kv_lens, page, hkv, d, pad=2)
    kv = (kv.float() * 0.05).bfloat16()
    q = (torch.randn(meta.num_tokens, hq, d, device=DEV) * 0.5).bfloat16()
    for scale, window in ((None, 0), (1.0, 0), (None, 48)):
        ref = R.paged_attention(q, kv, meta, scale, window)
        out = cu().paged_attention(q, kv, meta, scale, window)
        bf16_close(out, ref, rel=2 ** -6, abs_=6e-3)
    # a decode step of few sequences: the keys of a sequence are split over several blocks and merged
    kv_lens = [1, 15, 300, 1025, 2000]
    kv, meta = make_batch([1] * len(kv_lens), kv_lens, page, hkv, d, pad=2)
    kv = (kv.float() * 0.05).bfloat16()
    q = (torch.randn(meta.num_tokens, hq, d, device=DEV) * 0.5).bfloat16()
    assert meta.decode_only
    for window in (0, 200):
        ref = R.paged_attention(q, kv, meta, None, window)
        before = cu().launch_count(DEV)
        out = cu().paged_attention(q, kv, meta, None, window)
        assert cu().launch_count(DEV) - before == 2  # split kernel + merge
        bf16_close(out, ref, rel=2 ** -6, abs_=6e-3)
        assert out[len(kv_lens):].abs().max().item() == 0  # padding rows are inert
    status_clean()


def test_geglu_softcap_and_value_norm_kernels():
    K = cu()
    g = torch.Generator(device=DEV).manual_seed(5)
    gu = (torch.randn(70, 2 * 1024, device=DEV, generator=g) * 2).bfloat16()
    bf16_close(K.geglu(gu), R.geglu(gu), rel=2 ** -6, abs_=4e-3)
    lg = (torch.randn(9, 4096, device=DEV, generator=g) * 40).bfloat16()
    bf16_close(K.softcap(lg, 30.0), R.softcap(lg, 30.0), rel=2 ** -6, abs_=4e-3)
    # weightless RMSNorm of the value rows inside the fused norm + RoPE + append kernels (vector and scalar variants)
    for d, rot in ((256, 256), (512, 512), (96, 48)):
        hq, hkv, page = 4, 2, 16
        kv, meta = make_batch([5, 1, 20], [21, 33, 20], page, hkv, d)
        kv2 = kv.clone()
        qkv = torch.randn(meta.num_tokens, (hq + 2 * hkv) * d, device=DEV, generator=g).bfloat16()
        w = (torch.randn(d, device=DEV, generator=g) * 0.1 + 1).bfloat16()
        cos, sin = R.rope_tables(512, rot, 1e4, torch.bfloat16, DEV)
        a = K.qk_norm_rope_append(qkv, w, w, cos, sin, meta, kv, hq, hkv, d, 1e-6, False, False, True)
        b = R.qk_norm_rope_append(qkv, w, w, cos, sin, meta, kv2, hq, hkv, d, 1e-6, False, False, True)
        bf16_close(a, b, rel=2 ** -7, abs_=2e-3)
        bf16_close(kv, kv2, rel=2 ** -7, abs_=2e-3)
    status_clean()


@pytest.mark.parametrize("d,hq,hkv,page", [(128, 32, 8, 16), (64, 4, 2, 16), (256, 24, 4, 64), (128, 8, 8, 32), (128, 6, 1, 16)])
def test_decode_attention(d, hq, hkv, page):
    torch.manual_seed(d + hq)
    kv_lens = [1, 15, 16, 17, 200, 1025, 333]
    kv, meta = make_batch([1] * len(kv_lens), kv_lens, page, hkv, d, pad=2)
    q = torch.randn(meta.num_tokens, hq, d, device=DEV).bfloat16()
    ref = R.paged_attention(q, kv, meta)
    for splits in (1, 3, None):
        meta.plan = splits
        out = cu().paged_attention(q, kv, meta)
        bf16_close(out, ref, rel=2 ** -6, abs_=6e-3)
        assert out[len(kv_lens):].abs().max().item() == 0  # padding rows are inert
    # sliding window: the decode kernel walks only the last `window` keys (split over the same partial buffers)
    for window in (48, 200):
        refw = R.paged_attention(q, kv, meta, None, window)
        for splits in (1, 3, None):
            meta.plan = splits
            bf16_close(cu().paged_attention(q, kv, meta, None, window), refw, rel=2 ** -6, abs_=6e-3)
    status_clean()


@pytest.mark.parametrize("d,hq,hkv,page", [(128, 32, 8, 16), (64, 4, 2, 16), (256, 12, 2, 64)])
def test_prefill_attention_ragged_and_mixed(d, hq, hkv, page):
    torch.manual_seed(d)
    q_lens = [1, 64, 65, 130, 1, 17]
    kv_lens = [40, 64, 200, 130, 1, 300]
    kv, meta = make_batch(q_lens, kv_lens, page, hkv, d)
    q = torch.randn(meta.num_tokens, hq, d, device=DEV).bfloat16()
    ref = R.paged_attention(q, kv, meta)
    out = cu().paged_attention(q, kv, meta)
    bf16_close(out, ref, rel=2 ** -6, abs_=6e-3)
    refw = R.paged_attention(q, kv, meta, window=48)
    outw = cu().paged_attention(q, kv, meta, window=48)
    bf16_close(outw, refw, rel=2 ** -6, abs_=6e-3)
    status_clean()


@pytest.mark.parametrize("d,hq,hkv,page", [(128, 32, 8, 16), (256, 24, 4, 64)])
def test_unified_step_attention_splits_chunks_and_decode_rows(d, hq, hkv, page):
    """A unified step (prompt chunks first, decode rows last): the trailing single-row sequences take
    the decode kernel, the chunks the prefill kernel, and together they match the reference; with
    fewer than four decode rows everything stays in the prefill kernel."""
    torch.manual_seed(d + 1)
    for q_lens, kv_lens in (([130, 64, 1, 1, 1, 1, 1, 1], [130, 300, 40, 1025, 1, 333, 16, 17]), ([70, 1, 1], [200, 90, 5]), ([1, 1, 1, 1, 1, 90], [9, 8, 7, 6, 5, 90])):
        kv, meta = make_batch(q_lens, kv_lens, page, hkv, d)
        q = torch.randn(meta.num_tokens, hq, d, device=DEV).bfloat16()
        ref = R.paged_attention(q, kv, meta)
        before = cu().launch_count(DEV)
        out = cu().paged_attention(q, kv, meta)
        launches = cu().launch_count(DEV) - before
        bf16_close(out, ref, rel=2 ** -6, abs_=6e-3)
        trailing = 0
        while trailing < len(q_lens) and q_lens[len(q_lens) - 1 - trailing] == 1:
            trailing += 1
        assert (launches >= 2) == (trailing >= 4), (q_lens, launches)
        # the same step under a sliding window: chunks through the windowed prefill kernel, decode rows through the
        # windowed decode kernel
        refw = R.paged_attention(q, kv, meta, None, 100)
        bf16_close(cu().paged_attention(q, kv, meta, None, 100), refw, rel=2 ** -6, abs_=6e-3)
    status_clean()


@pytest.mark.parametrize("d,rot,gated,offset", [(128, 128, False, False), (64, 64, False, False), (256, 64, True, True), (256, 256, False, False), (128, 32, False, True), (96, 48, False, False)])
def test_qk_norm_rope_append(d, rot, gated, offset):
    torch.manual_seed(rot)
    hq, hkv, page = 8, 2, 16
    q_lens, kv_lens = [5, 1, 20], [21, 33, 20]
    kv, meta = make_batch(q_lens, kv_lens, page, hkv, d)
    kv2 = kv.clone()
    t = meta.num_tokens
    qkv = torch.randn(t, hq * d * (2 if gated else 1) + 2 * hkv * d, device=DEV).bfloat16()
    qw = (torch.randn(d, device=DEV) * 0.1 + (0 if offset else 1)).bfloat16()
    kw = (torch.randn(d, device=DEV) * 0.1 + (0 if offset else 1)).bfloat16()
    cos, sin = R.rope_tables(512, rot, 1e6, torch.bfloat16, DEV)
    a = cu().qk_norm_rope_append(qkv, qw, kw, cos, sin, meta, kv, hq, hkv, d, 1e-6, offset, gated)
    b = R.qk_norm_rope_append(qkv, qw, kw, cos, sin, meta, kv2, hq, hkv, d, 1e-6, offset, gated)
    if gated:
        assert torch.equal(a[1], b[1])
        a, b = a[0], b[0]
    bf16_close(a, b, rel=2 ** -7, abs_=2e-3)
    bf16_close(kv, kv2, rel=2 ** -7, abs_=2e-3)
    status_clean()


def test_position_out_of_range_sets_status_not_trap():
    hq, hkv, d, page = 4, 2, 64, 16
    kv, meta = make_batch([2], [2], page, hkv, d)
    meta.positions = torch.tensor([0, 9999], dtype=torch.int32, device=DEV)
    qkv = torch.randn(2, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    w = torch.ones(d, device=DEV).bfloat16()
    cos, sin = R.rope_tables(128, d, 1e6, torch.bfloat16, DEV)
    cu().qk_norm_rope_append(qkv, w, w, cos, sin, meta, kv, hq, hkv, d, 1e-6)
    torch.cuda.synchronize()
    st = cu().read_status(DEV)
    assert st & 0xFF == 2
    cu().clear_status(DEV)
    status_clean()


@pytest.mark.parametrize("vocab", [1024, 40000, 151936, 248320])  # one CTA, and clusters of 2, 8 and 8 CTAs per row
def test_argmax_sample_logprobs(vocab):
    torch.manual_seed(vocab)
    rows = 9
    logits = (torch.randn(rows, vocab, device=DEV) * 3).bfloat16()
    logits[0, 5] = logits[0, 77] = 50.0  # tie -> lowest index
    am = cu().argmax(logits)
    assert torch.equal(am, R.argmax(logits)) and am[0].item() == 5
    temp = torch.tensor([0.7, 1.0, 1.3, 1.0, 0.5, 1.0, 2.0, 1.0, 1.0], device=DEV)
    top_k = torch.tensor([0, 50, 0, 5, 1000, 0, 40, 1, 0], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.5, 0.95, 1.0, 0.8, 1.0, 0.3], device=DEV)
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.05, 0.02, 0.0, 0.0], device=DEV)
    agree = total = 0
    for trial in range(6):
        u = torch.rand(rows, device=DEV)
        got = cu().sample(logits, temp, top_k, top_p, min_p, u)
        ref = R.sample(logits, temp, top_k, top_p, min_p, u)
        probs = R.filtered_probs(logits, temp, top_k, top_p, min_p)
        # every drawn token must be inside the reference keep-set
        assert (probs.gather(-1, got.long().unsqueeze(-1)) > 0).all()
        assert torch.equal(got, cu().sample(logits, temp, top_k, top_p, min_p, u))  # replay is exact
        agree += (got == ref).sum().item()
        total += rows
    assert agree >= total - 3, f"only {agree}/{total} draws match the fp64 inverse-CDF reference"
    assert cu().sample(logits, temp, top_k, top_p, min_p, torch.rand(rows, device=DEV))[7].item() == R.argmax(logits)[7].item()
    picked = R.argmax(logits)
    c1, tv1, ti1 = cu().logprobs_topk(logits, picked, 5)
    c2, tv2, ti2 = R.logprobs_topk(logits, picked, 5)
    assert (c1 - c2).abs().max().item() < 1e-3 and (tv1 - tv2).abs().max().item() < 1e-3
    # same best alternative, up to ties between equal bf16 logits (a large vocabulary has many)
    lf = logits.float()
    assert torch.equal(lf[1:].gather(-1, ti1[1:, :1].long()), lf[1:].gather(-1, ti2[1:, :1]))
    status_clean()


def test_bounded_wait_times_out_with_status_and_context_survives():
    """A delivery flag that nothing sets: the wait gives up after its limit, reports
    through the status word, and the device stays usable."""
    import ctypes

    from pegainfer_b200 import _native

    lib = _native.load()
    flags = torch.zeros(32, dtype=torch.int32, device=DEV)
    flags[16] = 5  # epoch says "5 deliveries expected", nobody delivered
    torch.cuda.synchronize()
    c = cu().ctx(DEV)
    rc = lib.pg_tp_wait(ctypes.c_void_p(flags.data_ptr()), ctypes.c_int(2), ctypes.c_ulonglong(200_000_000), ctypes.c_void_p(c.status.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    st = cu().read_status(DEV)
    assert st & 0xFF == 1 and (st >> 8) & 0xFF == 4, hex(st)
    cu().clear_status(DEV)
    x = torch.ones(4, device=DEV)
    assert (x + x).sum().item() == 8.0
    status_clean()


def _state_meta(q_lens, slots):
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    seqs = [SeqStep(rid=i, input_tokens=[0] * n, start_pos=0, view=KvView([1], n, 1 << 20)) for i, n in enumerate(q_lens)]
    _, meta = build_meta(seqs, 1 << 20, DEV)
    meta.h_state_slots = list(slots)
    meta.state_slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
    return meta


@pytest.mark.parametrize("q_lens", [[1, 19, 5, 1], [1, 3, 1, 4], [1, 1, 1, 1]])  # pipelined prompt path; row-coalesced mapping of short steps; decode
@pytest.mark.parametrize("dk,hk,hv", [(128, 2, 6), (32, 2, 4)])
def test_gated_delta_net_kernels(dk, hk, hv, q_lens):
    torch.manual_seed(dk)
    dv = dk
    slots = [3, 1, 4, 2]
    meta = _state_meta(q_lens, slots)
    t = meta.num_tokens
    ch = 2 * hk * dk + hv * dv
    x = torch.randn(t, ch, device=DEV).bfloat16()
    conv_w = (torch.randn(ch, 4, device=DEV) * 0.5).bfloat16()
    st1 = torch.randn(6, ch, 3, device=DEV).bfloat16()
    st2 = st1.clone()
    y1 = cu().gdn_conv1d(x, conv_w, st1, meta)
    y2 = R.gdn_conv1d(x, conv_w, st2, meta)
    bf16_close(y1, y2, rel=2 ** -6, abs_=4e-3)
    assert torch.equal(st1, st2)
    a = torch.randn(t, hv, device=DEV).bfloat16()
    b = torch.randn(t, hv, device=DEV).bfloat16()
    a_log = torch.randn(hv, device=DEV) * 0.5
    dt_bias = torch.randn(hv, device=DEV) * 0.5
    g1, b1 = cu().gdn_gates(a, b, a_log, dt_bias)
    g2, b2 = R.gdn_gates(a, b, a_log, dt_bias)
    assert (g1 - g2).abs().max().item() < 1e-4 and (b1 - b2).abs().max().item() < 1e-5
    q = y2[:, : hk * dk].reshape(t, hk, dk)
    k = y2[:, hk * dk : 2 * hk * dk].reshape(t, hk, dk)
    v = y2[:, 2 * hk * dk :].reshape(t, hv, dv)
    s1 = torch.randn(6, hv, dk, dv, device=DEV) * 0.1
    s2 = s1.clone()
    o1 = cu().gdn_recurrent(q, k, v, g2, b2, s1, meta)
    o2 = R.gdn_recurrent(q, k, v, g2, b2, s2, meta)
    bf16_close(o1, o2, rel=2 ** -6, abs_=4e-3)
    assert (s1 - s2).abs().max().item() < 2e-3
    status_clean()


@pytest.mark.parametrize("q_lens", [[1, 19, 5, 1, 40], [1, 3, 1, 4, 2]])
@pytest.mark.parametrize("dk,heads", [(128, 5), (32, 4)])
def test_kda_channel_decay_recurrence(dk, heads, q_lens):
    """Delta rule with one decay per key channel (the gate arithmetic runs in the kernel): ragged step of decode rows and
    prompt chunks (the shuffle mapping) and a step of at most four tokens per sequence (the row-coalesced mapping of decode
    and verify steps), q / k / v as strided slices of one buffer, against the PyTorch recurrence."""
    torch.manual_seed(dk + heads)
    slots = [3, 1, 4, 2, 5]
    meta = _state_meta(q_lens, slots)
    t, inner = meta.num_tokens, heads * dk
    qkv = torch.randn(t, 3 * inner, device=DEV).bfloat16()
    q, k, v = (qkv[:, j * inner : (j + 1) * inner].view(t, heads, dk) for j in range(3))
    f = (torch.randn(t, inner, device=DEV) * 2).bfloat16()
    small = torch.randn(t, heads + 11, device=DEV).bfloat16()
    b = small[:, :heads]
    a_log, dt_bias = torch.randn(heads, device=DEV) * 0.5, torch.randn(inner, device=DEV) * 0.5
    s1 = torch.randn(7, heads, dk, dk, device=DEV) * 0.1
    s2 = s1.clone()
    o1 = cu().kda_recurrent(q, k, v, f, b, a_log, dt_bias, -5.0, s1, meta)
    o2 = R.kda_recurrent(q, k, v, f, b, a_log, dt_bias, -5.0, s2, meta)
    bf16_close(o1, o2, rel=2 ** -6, abs_=4e-3)
    assert (s1 - s2).abs().max().item() < 2e-3 and torch.equal(s1[0], s2[0]) and torch.equal(s1[6], s2[6])  # unused slots untouched
    status_clean()


def test_attnres_mix_situ_and_sigmoid_gated_norm_kernels():
    torch.manual_seed(5)
    t, cap, h = 37, 8, 1024
    cur, snaps = torch.randn(t, h, device=DEV).bfloat16(), torch.randn(t, cap, h, device=DEV).bfloat16()
    sw = torch.randn(h, device=DEV) * 0.2
    for nb in (0, 1, 5, 8):
        bf16_close(cu().attnres_mix(cur, snaps, nb, sw, 1e-5), R.attnres_mix(cur, snaps, nb, sw, 1e-5), rel=2 ** -6, abs_=4e-3)
    gu = (torch.randn(19, 512, device=DEV) * 6).bfloat16()
    bf16_close(cu().situ(gu), R.situ(gu), rel=2 ** -6, abs_=4e-3)
    x, gate = torch.randn(23, 4, 128, device=DEV).bfloat16(), torch.randn(23, 4, 128, device=DEV).bfloat16()
    w = torch.rand(128, device=DEV) + 0.5
    bf16_close(cu().gated_rms_norm(x, gate, w, 1e-5, act="sigmoid"), R.gated_rms_norm(x, gate, w, 1e-5, act="sigmoid"), rel=2 ** -6, abs_=4e-3)
    bf16_close(cu().gated_rms_norm(x, gate, w, 1e-5), R.gated_rms_norm(x, gate, w, 1e-5), rel=2 ** -6, abs_=4e-3)
    status_clean()


def test_moe_experts_with_the_saturating_activation():
    torch.manual_seed(6)
    t, h, inter, e, k = 40, 256, 128, 8, 3
    x = torch.randn(t, h, device=DEV).bfloat16()
    w13 = (torch.randn(e, 2 * inter, h, device=DEV) * 0.2).bfloat16()
    w2 = (torch.randn(e, h, inter, device=DEV) * 0.1).bfloat16()
    ids = torch.stack([torch.randperm(e, device=DEV)[:k] for _ in range(t)]).to(torch.int32)
    wts = torch.rand(t, k, device=DEV)
    a = cu().moe_experts(x, ids, wts, w13, w2, 0, act="situ")
    b = R.moe_experts(x, ids, wts, w13, w2, 0, act="situ")
    assert (a - b).abs().max().item() < 3e-2 * b.abs().max().item() and not torch.allclose(b, R.moe_experts(x, ids, wts, w13, w2, 0), atol=1e-3)
    status_clean()


@pytest.mark.parametrize("q_lens", [[200, 64, 1, 33, 130, 31], [2048], [65, 127]])
def test_gated_delta_chunk_scan_matches_recurrence(q_lens):
    """The 64-token chunk-wise tensor-core scan against the token-by-token rule (fp32 PyTorch
    restatement and the recurrence kernel): ragged lengths, a partial last chunk, a decode row and
    a short chunk in the same step (those two stay on the recurrence kernel), non-zero start state."""
    torch.manual_seed(len(q_lens) * 31 + q_lens[0])
    dk = dv = 128
    hk, hv = 2, 4
    slots = list(range(1, len(q_lens) + 1))
    meta = _state_meta(q_lens, slots)
    t = meta.num_tokens
    q = torch.randn(t, hk, dk, device=DEV).bfloat16()
    k = torch.randn(t, hk, dk, device=DEV).bfloat16()
    v = torch.randn(t, hv, dv, device=DEV).bfloat16()
    a = torch.randn(t, hv, device=DEV).bfloat16()
    b = torch.randn(t, hv, device=DEV).bfloat16()
    g, beta = R.gdn_gates(a, b, torch.randn(hv, device=DEV) * 0.5, torch.randn(hv, device=DEV) * 0.5)
    s0 = torch.randn(len(q_lens) + 2, hv, dk, dv, device=DEV) * 0.1
    s_ref, s_rec, s_chk = s0.clone(), s0.clone(), s0.clone()
    o_ref = R.gdn_recurrent(q, k, v, g, beta, s_ref, meta)
    o_rec = cu().gdn_recurrent(q, k, v, g, beta, s_rec, meta, chunked=False)
    o_chk = cu().gdn_recurrent(q, k, v, g, beta, s_chk, meta, chunked=True)
    torch.cuda.synchronize()
    status_clean()
    scale = o_ref.float().abs().max().item()
    e_rec = (o_rec.float() - o_ref.float()).abs().max().item()
    e_chk = (o_chk.float() - o_ref.float()).abs().max().item()
    es_chk = (s_chk - s_ref).abs().max().item()
    es_rec = (s_rec - s_ref).abs().max().item()
    # bf16 operands (keys, corrections, the state as an operand) against the all-f32 rule
    assert e_chk < 0.03 * scale + 2e-3, f"chunk scan out err {e_chk} (recurrence kernel {e_rec}, scale {scale})"
    assert es_chk < 0.03 * s_ref.abs().max().item(), f"chunk scan state err {es_chk} (recurrence kernel {es_rec})"
    assert torch.equal(s_chk[0], s0[0]) and torch.equal(s_chk[-1], s0[-1]), "slots of other requests are untouched"
    # rows of the short sequences took the recurrence kernel in both runs
    for i, n in enumerate(q_lens):
        if n < 32:
            lo = sum(q_lens[:i])
            assert torch.equal(o_chk[lo : lo + n], o_rec[lo : lo + n])


@pytest.mark.parametrize("scoring,e,k,ng,tg,norm", [("softmax", 64, 6, 1, 1, False), ("sigmoid", 384, 8, 1, 1, True), ("sigmoid", 64, 4, 8, 3, True), ("softmax", 16, 2, 4, 2, False)])
def test_router_topk(scoring, e, k, ng, tg, norm):
    torch.manual_seed(e + k)
    logits = torch.randn(50, e, device=DEV) * 2
    bias = torch.randn(e, device=DEV) * 0.1 if scoring == "sigmoid" else None
    i1, w1 = cu().router_topk(logits, k, scoring, bias, ng, tg, norm, 2.5)
    i2, w2 = R.router_topk(logits, k, scoring, bias, ng, tg, norm, 2.5)
    assert torch.equal(i1, i2)
    assert (w1 - w2).abs().max().item() < 1e-5 * 2.5 + 1e-6
    status_clean()


@pytest.mark.parametrize("t,h,inter,e,k,int4", [(5, 256, 128, 8, 2, False), (64, 2048, 1408, 16, 6, False), (3, 512, 256, 8, 3, True), (130, 1024, 512, 12, 4, True), (700, 512, 256, 4, 2, False)])
def test_moe_pipeline_matches_per_expert_reference(t, h, inter, e, k, int4):
    torch.manual_seed(t + h)
    x = (torch.randn(t, h, device=DEV) * 0.5).bfloat16()
    logits = torch.randn(t, e + 4, device=DEV)
    ids, w = R.router_topk(logits, k, "softmax")
    off = 2  # local experts are [2, 2 + e): some routes fall outside
    if int4:
        p13 = torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, 2 * inter, h // 8), dtype=torch.int32, device=DEV)
        s13 = (torch.rand(e, 2 * inter, h // 32, device=DEV) * 0.004 + 0.002).bfloat16()
        p2 = torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, h, inter // 8), dtype=torch.int32, device=DEV)
        s2 = (torch.rand(e, h, inter // 32, device=DEV) * 0.004 + 0.002).bfloat16()
        got = cu().moe_experts_int4(x, ids, w, p13, s13, p2, s2, off)
        ref = R.moe_experts_int4(x, ids, w, p13, s13, p2, s2, off)
    else:
        w13 = (torch.randn(e, 2 * inter, h, device=DEV) * 0.03).bfloat16()
        w2 = (torch.randn(e, h, inter, device=DEV) * 0.03).bfloat16()
        got = cu().moe_experts(x, ids, w, w13, w2, off)
        ref = R.moe_experts(x, ids, w, w13, w2, off)
    torch.cuda.synchronize()
    status_clean()
    err = (got - ref).abs()
    assert err.max().item() < 2e-2 * max(1.0, ref.abs().max().item()), (err.max().item(), ref.abs().max().item())
    assert torch.equal(got, cu().moe_experts_int4(x, ids, w, p13, s13, p2, s2, off) if int4 else cu().moe_experts(x, ids, w, w13, w2, off))


@pytest.mark.parametrize("t,h,inter,e,k", [(3, 512, 256, 8, 3), (130, 1024, 512, 12, 4), (64, 2048, 1408, 16, 6)])
def test_moe_pipeline_fp8_block_scaled_experts(t, h, inter, e, k):
    """FP8 e4m3 experts with 128x128 scale blocks, dequantised inside the grouped GEMM."""
    torch.manual_seed(t + h + 1)
    x = (torch.randn(t, h, device=DEV) * 0.5).bfloat16()
    ids, w = R.router_topk(torch.randn(t, e + 4, device=DEV), k, "softmax")
    off = 2
    q13, s13 = zip(*[R.quant_fp8_block(torch.randn(2 * inter, h, device=DEV) * 0.03) for _ in range(e)])
    q2, s2 = zip(*[R.quant_fp8_block(torch.randn(h, inter, device=DEV) * 0.03) for _ in range(e)])
    q13, s13, q2, s2 = torch.stack(q13), torch.stack(s13).contiguous(), torch.stack(q2), torch.stack(s2).contiguous()
    got = cu().moe_experts_fp8(x, ids, w, q13, s13, q2, s2, off)
    ref = R.moe_experts_fp8(x, ids, w, q13, s13, q2, s2, off)
    torch.cuda.synchronize()
    status_clean()
    err = (got - ref).abs()
    # the tensor-core path quantises the activations to e4m3 per token and 128-wide k group (3 mantissa bits); the
    # reference keeps them in bf16: single elements may be off by a few percent of the largest value, the mean far less
    assert err.max().item() < 4e-2 * max(1.0, ref.abs().max().item()), (err.max().item(), ref.abs().max().item())
    assert err.mean().item() < 4e-3 * max(1.0, ref.abs().max().item()), err.mean().item()
    assert torch.equal(got, cu().moe_experts_fp8(x, ids, w, q13, s13, q2, s2, off))
    # one-hot rows read single weights back: the in-kernel dequantisation is exact
    m, kk = 256, 256
    q, sc = R.quant_fp8_block(torch.randn(m, kk, device=DEV) * 0.05)
    xs = torch.zeros(32, kk, device=DEV).bfloat16()
    for r in range(32):
        xs[r, (r * 37) % kk] = 1.0
    y = cu().grouped_gemm(xs, torch.tensor([0, 32], dtype=torch.int32, device=DEV), q[None], sc[None].contiguous(), 32)
    wd = R.dequant_fp8_block(q, sc)
    assert torch.equal(y.float(), (xs.float() @ wd.float().t()).bfloat16().float())
    status_clean()


def test_int4_dequant_inside_grouped_gemm_is_exact_on_one_hot_inputs():
    torch.manual_seed(0)
    e, m, k = 3, 256, 128
    packed = torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, m, k // 8), dtype=torch.int32, device=DEV)
    scales = (torch.rand(e, m, k // 32, device=DEV) * 0.01 + 0.001).bfloat16()
    xs = torch.zeros(3 * 16, k, device=DEV).bfloat16()
    for r in range(48):
        xs[r, (r * 5) % k] = 1.0
    offsets = torch.tensor([0, 16, 32, 48], dtype=torch.int32, device=DEV)
    y = cu().grouped_gemm(xs, offsets, packed, scales, 16)
    for ex in range(e):
        wd = R.dequant_int4_g32(packed[ex], scales[ex])
        ref = xs[ex * 16 : (ex + 1) * 16].float() @ wd.float().t()
        assert torch.equal(y[ex * 16 : (ex + 1) * 16].float(), ref.bfloat16().float())
    status_clean()


def _mla_setup(q_lens, kv_lens, heads, page=16, seed=0):
    torch.manual_seed(seed)
    c, rope, nope, v = 512, 64, 128, 128
    kv, meta = make_batch(q_lens, kv_lens, page, 1, 8)  # reuse the page-table builder
    n_pages = kv.shape[0]
    latent = (torch.randn(n_pages, page, c + rope, device=DEV) * 0.5).bfloat16()
    t = meta.num_tokens
    q = (torch.randn(t, heads, nope + rope, device=DEV) * 0.5).bfloat16()
    w_uk = (torch.randn(heads, nope, c, device=DEV) * 0.05).bfloat16()
    w_uv = (torch.randn(heads, v, c, device=DEV) * 0.05).bfloat16()
    cos, sin = R.rope_tables(4096, rope, 10000.0, torch.bfloat16, DEV)
    return meta, latent, q, w_uk, w_uv, cos, sin, c, nope


@pytest.mark.parametrize("heads", [16, 64])
def test_mla_decode_and_prefill_match_reference(heads):
    for q_lens, kv_lens in (([1, 1, 1, 1], [1, 31, 32, 700]), ([5, 40, 1], [5, 90, 33])):
        meta, latent, q, w_uk, w_uv, cos, sin, c, nope = _mla_setup(q_lens, kv_lens, heads, seed=heads)
        scale = 0.1
        q_ref = R.mla_rope_q(q, cos, sin, meta, nope)
        ref = R.mla_attention(q_ref, w_uk, w_uv, latent, meta, scale, c)
        q_cu = cu().mla_rope_q(q, cos, sin, meta, nope)
        got = cu().mla_attention(q_cu, w_uk, w_uv, latent, meta, scale, c)
        torch.cuda.synchronize()
        status_clean()
        err = (got.float() - ref.float()).abs()
        assert err.max().item() < 3e-2 * max(1.0, ref.float().abs().max().item()), (q_lens, err.max().item(), ref.float().abs().max().item())


@pytest.mark.parametrize("heads", [16, 64])
def test_mla_prefill_expanded_tcgen05_matches_reference(heads):
    """Prefill chunks (whole prompts, a chunk behind a cached prefix, ragged tails) through the expanded-form tcgen05
    kernel: gather of the latent rows, K / V expansion, 192 / 128 attention."""
    K = cu()
    # prefill chunks only, then a unified step: chunks in front (expanded form), single-row decodes behind (absorbed kernel)
    for q_lens, kv_lens, n_expanded in (([300, 257, 130, 70], [300, 700, 1000, 90], 4), ([300, 257, 1, 1, 1], [300, 700, 90, 1000, 33], 2)):
        meta, latent, q, w_uk, w_uv, cos, sin, c, nope = _mla_setup(q_lens, kv_lens, heads, seed=heads + 1)
        scale = 0.1
        q_ref = R.mla_rope_q(q, cos, sin, meta, nope)
        ref = R.mla_attention(q_ref, w_uk, w_uv, latent, meta, scale, c)
        q_cu = K.mla_rope_q(q, cos, sin, meta, nope)
        prev = K.set_prefill_tc(0)
        try:
            assert K._mla_expanded_seqs(q_cu, w_uk, w_uv, meta, c) == n_expanded
            got = K.mla_attention(q_cu, w_uk, w_uv, latent, meta, scale, c)
            torch.cuda.synchronize()
        finally:
            K.set_prefill_tc(prev)
        status_clean()
        err = (got.float() - ref.float()).abs()
        assert err.max().item() < 3e-2 * max(1.0, ref.float().abs().max().item()), (q_lens, err.max().item(), ref.float().abs().max().item())


def test_mla_append_matches_reference():
    meta, latent, q, w_uk, w_uv, cos, sin, c, nope = _mla_setup([3, 1, 20], [19, 40, 20], 16, seed=3)
    t = meta.num_tokens
    kv_a = torch.randn(t, c + 64, device=DEV).bfloat16()
    w = (torch.rand(c, device=DEV) + 0.5).bfloat16()
    l1, l2 = latent.clone(), latent.clone()
    cu().mla_append(kv_a, w, cos, sin, meta, l1, c, 1e-6)
    R.mla_append(kv_a, w, cos, sin, meta, l2, c, 1e-6)
    bf16_close(l1, l2, rel=2 ** -7, abs_=4e-3)
    status_clean()


@pytest.mark.parametrize("int4", [False, True])
def test_fused_ep_single_rank_self_dispatch_matches_local_pipeline(int4):
    """World of one: the dispatch / return / combine kernels talk to this GPU's own
    buffers, which exercises slots, epochs and the scatter epilogue without a peer."""
    from types import SimpleNamespace

    from pegainfer_b200.parallel.fused_ep import FusedEP

    torch.manual_seed(5)
    t, h, inter, e, k = 24, 512, 256, 8, 3
    ep = FusedEP(0, 1, DEV, h, k, max_tokens=32, wait_s=1.0)
    x = (torch.randn(t, h, device=DEV) * 0.5).bfloat16()
    ids, w = R.router_topk(torch.randn(t, e, device=DEV), k, "softmax")
    if int4:
        ex = dict(w13_packed=torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, 2 * inter, h // 8), dtype=torch.int32, device=DEV), w13_scale=(torch.rand(e, 2 * inter, h // 32, device=DEV) * 0.004 + 0.002).bfloat16(),
                  w2_packed=torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, h, inter // 8), dtype=torch.int32, device=DEV), w2_scale=(torch.rand(e, h, inter // 32, device=DEV) * 0.004 + 0.002).bfloat16(), offset=0)
        ref = cu().moe_experts_int4(x, ids, w, ex["w13_packed"], ex["w13_scale"], ex["w2_packed"], ex["w2_scale"], 0)
    else:
        ex = dict(w13=(torch.randn(e, 2 * inter, h, device=DEV) * 0.03).bfloat16(), w2=(torch.randn(e, h, inter, device=DEV) * 0.03).bfloat16(), offset=0)
        ref = cu().moe_experts(x, ids, w, ex["w13"], ex["w2"], 0)
    cfg = SimpleNamespace(quant_group_size=32)
    for step in range(3):  # epochs advance; a smaller step after a larger one must ignore stale slots
        n = t if step != 1 else 5
        ep.begin_step()
        got = ep.moe(x[:n], ids[:n], w[:n], ex, cfg)
        got2 = ep.moe(x[:n], ids[:n], w[:n], ex, cfg)  # second site in the same step
        torch.cuda.synchronize()
        status_clean()
        assert torch.equal(got, got2)
        assert (got - ref[:n]).abs().max().item() < 1e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("t,k,m,r,slots_n", [(9, 1024, 2048, 16, 3), (64, 4096, 1024, 64, 4), (1, 512, 512, 8, 2)])
def test_lora_delta_kernel_mixed_slots(t, k, m, r, slots_n):
    """Per-token adapter delta y += scale[s] * B[s] (A[s] x) with a mixed batch (some rows without adapter),
    also on a column slice of a wider output (fused qkv)."""
    torch.manual_seed(t + r)
    x = (torch.randn(t, k, device=DEV) * 0.5).bfloat16()
    A = (torch.randn(slots_n, r, k, device=DEV) * 0.05).bfloat16()
    B = (torch.randn(slots_n, m, r, device=DEV) * 0.05).bfloat16()
    scale = torch.rand(slots_n, device=DEV) * 2
    slots = torch.randint(-1, slots_n, (t,), dtype=torch.int32, device=DEV)
    wide = (torch.randn(t, m + 256, device=DEV) * 0.3).bfloat16()
    y1, y2 = wide.clone(), wide.clone()
    cu().lora_delta_(y1[:, 128 : 128 + m], x, A, B, scale, slots)
    R.lora_delta_(y2[:, 128 : 128 + m], x, A, B, scale, slots)
    torch.cuda.synchronize()
    bf16_close(y1, y2, rel=2 ** -6, abs_=2e-2)
    untouched = slots < 0
    assert torch.equal(y1[untouched], wide[untouched])
    assert torch.equal(y1[:, :128], wide[:, :128]) and torch.equal(y1[:, 128 + m :], wide[:, 128 + m :])
    status_clean()


@pytest.mark.parametrize("t", [1, 7, 64])
def test_fused_decode_chain_matches_separate_kernels(t):
    K = cu()
    """o_proj with the residual add and the norm-weight product in its epilogue, a consumer GEMM that
    completes the RMSNorm with the per-token scale (and applies SwiGLU over interleaved gate/up rows),
    against GEMM -> add + RMSNorm -> GEMM -> SwiGLU as separate kernels."""
    torch.manual_seed(t)
    h, kq, inter = 1024, 1024, 1536
    eps = 1e-6
    a = (torch.randn(t, kq, device=DEV) * 0.5).bfloat16()
    wo = (torch.randn(h, kq, device=DEV) * 0.03).bfloat16()
    res0 = torch.randn(t, h, device=DEV).bfloat16()
    nw = (1.0 + 0.1 * torch.randn(h, device=DEV)).bfloat16()
    wg = (torch.randn(inter, h, device=DEV) * 0.03).bfloat16()
    wu = (torch.randn(inter, h, device=DEV) * 0.03).bfloat16()
    w_il = torch.stack((wg, wu), 1).reshape(2 * inter, h).contiguous()
    if not K.fused_plan_ok(t, h, kq) or not K.fused_plan_ok(t, 2 * inter, h):
        pytest.skip("this shape does not plan onto the on-chip split-K path")
    # separate kernels
    res_ref = res0.clone()
    x_ref = K.add_rms_norm(K.linear(a, wo), res_ref, nw, eps)
    act_ref = K.swiglu(K.linear(x_ref, torch.cat((wg, wu), 0)))
    plain_ref = K.linear(x_ref, wg)
    # fused chain
    res = res0.clone()
    dn = K.linear_fused(a, wo, K.EPI_RESID_NORMW, residual=res, norm_w=nw, eps=eps)
    act = K.linear_fused(dn, w_il, K.EPI_SWIGLU)
    plain = K.linear_fused(dn, wg)
    torch.cuda.synchronize()
    # the fused epilogue adds the residual to the f32 accumulator; the separate kernels round the
    # projection to bf16 first: at most one bf16 step apart, and the fused one is the closer of the two
    exact = res0.float() + a.float() @ wo.float().t()
    assert (res.float() - res_ref.float()).abs().max() <= 2 ** -7 * exact.abs().max()
    assert (res.float() - exact).abs().max() <= (res_ref.float() - exact).abs().max() + 1e-6
    # the normalised activations differ only by where the bf16 rounding sits (before or after the scale)
    inv = torch.rsqrt(res.float().pow(2).mean(-1, keepdim=True) + eps)
    assert torch.allclose(dn.ssp[:, : dn.parts].sum(1), res.float().pow(2).sum(-1), rtol=1e-4)
    x_exact = res.float() * inv * nw.float()
    assert (dn.xw.float() * inv - x_exact).abs().max() <= 2 ** -7 * x_exact.abs().max()
    for got, ref in ((plain, plain_ref), (act, act_ref)):
        err = (got.float() - ref.float()).abs().max().item()
        assert err <= 2e-2 * max(1.0, ref.float().abs().max().item()), err
    # bit-reproducible
    res2 = res0.clone()
    dn2 = K.linear_fused(a, wo, K.EPI_RESID_NORMW, residual=res2, norm_w=nw, eps=eps)
    assert torch.equal(K.linear_fused(dn2, w_il, K.EPI_SWIGLU), act) and torch.equal(dn2.ssp[:, : dn.parts], dn.ssp[:, : dn.parts])
    # a row's result does not depend on how many padding rows ride along in the same token tile
    if t < 16:
        pad = 16 - t
        a_p = torch.cat((a, torch.zeros(pad, kq, device=DEV, dtype=a.dtype)), 0)
        res_p = torch.cat((res0, torch.zeros(pad, h, device=DEV, dtype=a.dtype)), 0)
        dn_p = K.linear_fused(a_p, wo, K.EPI_RESID_NORMW, residual=res_p, norm_w=nw, eps=eps)
        act_p = K.linear_fused(dn_p, w_il, K.EPI_SWIGLU)
        assert torch.equal(res_p[:t], res) and torch.equal(act_p[:t], act)
    assert K.read_status(DEV) == 0


def test_swiglu_interleaved_layout():
    K = cu()
    torch.manual_seed(5)
    g = torch.randn(33, 256, device=DEV).bfloat16()
    u = torch.randn(33, 256, device=DEV).bfloat16()
    halves = torch.cat((g, u), 1)
    il = torch.stack((g, u), 2).reshape(33, 512).contiguous()
    assert torch.equal(K.swiglu(il, True), K.swiglu(halves))
    assert torch.equal(K.swiglu(il, True), R.swiglu(il, True))


@pytest.mark.parametrize("t,h,kq,inter,qkv", [(64, 1024, 1024, 1536, 1536), (5, 1024, 1024, 1536, 1536), (64, 4096, 4096, 12288, 6144), (1, 2048, 2048, 5504, 2560), (33, 1024, 2048, 19200, 1024)])
def test_decode_chain_matches_separate_kernels(t, h, kq, inter, qkv):
    """o_proj -> +residual, RMSNorm -> gate_up + SwiGLU -> down -> +residual, RMSNorm -> qkv in one
    persistent kernel (stream-K split, grid barriers) against the same chain as separate kernels."""
    K = cu()
    torch.manual_seed(t + h)
    eps = 1e-6
    a = (torch.randn(t, kq, device=DEV) * 0.5).bfloat16()
    wo = (torch.randn(h, kq, device=DEV) * 0.03).bfloat16()
    wg = (torch.randn(inter, h, device=DEV) * 0.03).bfloat16()
    wu = (torch.randn(inter, h, device=DEV) * 0.03).bfloat16()
    wd = (torch.randn(h, inter, device=DEV) * 0.02).bfloat16()
    wq = (torch.randn(qkv, h, device=DEV) * 0.03).bfloat16()
    n1 = (1.0 + 0.1 * torch.randn(h, device=DEV)).bfloat16()
    n2 = (1.0 + 0.1 * torch.randn(h, device=DEV)).bfloat16()
    res0 = torch.randn(t, h, device=DEV).bfloat16()
    w_il = torch.stack((wg, wu), 1).reshape(2 * inter, h).contiguous()
    # separate kernels
    res_ref = res0.clone()
    x1 = K.add_rms_norm(K.linear(a, wo), res_ref, n1, eps)
    act = K.swiglu(K.linear(x1, torch.cat((wg, wu), 0)))
    x2 = K.add_rms_norm(K.linear(act, wd), res_ref, n2, eps)
    q_ref = K.linear(x2, wq)
    # one kernel
    chain = [(wo, K.CH_RESID_NORM, n1, False), (w_il, K.CH_SWIGLU, None, False), (wd, K.CH_RESID_NORM, n2, False), (wq, K.CH_PLAIN, None, False)]
    res = res0.clone()
    outs = K.decode_chain(a, chain, residual=res, eps=eps)
    torch.cuda.synchronize()
    assert K.read_status(DEV) == 0
    scale = lambda r: max(1.0, r.float().abs().max().item())

    def normed(dn):  # complete the deferred RMSNorm on the host side of the test
        inv = torch.rsqrt(dn.ssp[:, : dn.parts].sum(1) / dn.width + dn.eps)
        return dn.xw.float() * inv[:, None]

    for name, got, ref, tol in (("x1", normed(outs[0]), x1, 2e-2), ("act", outs[1], act, 3e-2), ("x2", normed(outs[2]), x2, 3e-2), ("qkv", outs[3], q_ref, 4e-2), ("residual", res, res_ref, 3e-2)):
        err = (got.float() - ref.float()).abs().max().item()
        assert err <= tol * scale(ref), f"{name}: max err {err}"
    # bit-reproducible, and the counters were left re-armed: run it twice more
    for _ in range(2):
        res2 = res0.clone()
        outs2 = K.decode_chain(a, chain, residual=res2, eps=eps)
        same = lambda x, y: torch.equal(x.xw, y.xw) and torch.equal(x.ssp[:, : x.parts], y.ssp[:, : y.parts]) if isinstance(x, K.DeferredNorm) else torch.equal(x, y)
        assert all(same(x, y) for x, y in zip(outs, outs2)) and torch.equal(res, res2)
    # a chain that starts from rows whose norm is still owed, and a single-phase chain on finished rows
    one = K.decode_chain(outs[2], [(wq, K.CH_PLAIN, None, False)])[0]  # the scale's epsilon travels with the rows
    assert torch.equal(one, outs[3])
    plain = K.decode_chain(x2, [(wq, K.CH_PLAIN, None, False)])[0]
    assert (plain.float() - q_ref.float()).abs().max().item() <= 2e-2 * scale(q_ref)
    # the separate GEMM kernel completes a deferred norm the same way (lm_head after the last layer)
    lf = K.linear_fused(outs[2], wq)
    assert (lf.float() - q_ref.float()).abs().max().item() <= 4e-2 * scale(q_ref)
    assert K.read_status(DEV) == 0


@pytest.mark.parametrize("t,hq,hkv,page", [(64, 8, 2, 16), (7, 4, 4, 32)])
def test_decode_chain_qkv_rope_append_epilogue(t, hq, hkv, page):
    """The qkv phase with per-head QK RMSNorm, RoPE and the paged KV append in its epilogue, against the
    GEMM followed by the separate norm / rope / append kernel."""
    K = cu()
    torch.manual_seed(hq * 100 + t)
    d, hidden, eps = 128, 1024, 1e-6
    x = (torch.randn(t, hidden, device=DEV) * 0.5).bfloat16()
    wqkv = (torch.randn((hq + 2 * hkv) * d, hidden, device=DEV) * 0.03).bfloat16()
    qn = (1.0 + 0.1 * torch.randn(d, device=DEV)).bfloat16()
    kn = (1.0 + 0.1 * torch.randn(d, device=DEV)).bfloat16()
    cos, sin = R.rope_tables(512, d, 1e6, torch.bfloat16, DEV)
    pages = 40
    positions = torch.randint(0, 500, (t,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * page, device=DEV)[:t].to(torch.int32)
    meta = R.AttnMeta(q_indptr=torch.arange(t + 1, dtype=torch.int32, device=DEV), kv_lens=positions + 1, block_table=torch.zeros((t, 1), dtype=torch.int32, device=DEV), slot_mapping=slots,
                      positions=positions, page_size=page, num_seqs=t, num_tokens=t, max_q_len=1, max_kv_len=512, decode_only=True)
    kv_ref = torch.zeros((pages, 2, page, hkv, d), dtype=torch.bfloat16, device=DEV)
    kv_got = torch.zeros_like(kv_ref)
    q_ref = K.qk_norm_rope_append(K.linear(x, wqkv), qn, kn, cos, sin, meta, kv_ref, hq, hkv, d, eps)
    spec = dict(q_norm=qn, k_norm=kn, cos=cos, sin=sin, meta=meta, kv_layer=kv_got, hq=hq, hkv=hkv, eps=eps)
    q_got = K.decode_chain(x, [(wqkv, K.CH_QKV_ROPE, spec, False)])[0]
    torch.cuda.synchronize()
    assert K.read_status(DEV) == 0
    assert (q_got.float() - q_ref.float().view(t, hq, d)).abs().max().item() <= 3e-2 * max(1.0, q_ref.float().abs().max().item())
    assert (kv_got.float() - kv_ref.float()).abs().max().item() <= 3e-2 * max(1.0, kv_ref.float().abs().max().item())
    assert torch.equal(kv_got != 0, kv_ref != 0)  # exactly the same slots were written


def test_dsa_indexer_kernels_match_reference():
    """Index-key append (LayerNorm + rotary), query rotary, tcgen05 index scores, radix top-k and the gathered
    sparse latent attention against their PyTorch restatements on one ragged step."""
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.ops.reference import rope_tables
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    K = cu()
    dev, page, heads, d, rope, topk = "cuda:0", 16, 32, 128, 64, 128
    g = torch.Generator(device=dev).manual_seed(5)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)  # noqa: E731
    kv_q = [(300, 1), (40, 40), (517, 5)]
    seqs, nxt = [], 1
    for i, (kl, nq) in enumerate(kv_q):
        npg = (kl + page - 1) // page
        seqs.append(SeqStep(rid=i, input_tokens=[0] * nq, start_pos=kl - nq, view=KvView(list(range(nxt, nxt + npg)), kl, page)))
        nxt += npg
    _, meta = build_meta(seqs, page, dev)
    t = meta.num_tokens
    cos, sin = rope_tables(1024, rope, 10000.0, torch.bfloat16, dev)
    cache_k = (rnd(nxt, page, d) * 0.5).to(torch.bfloat16)
    cache_r = cache_k.clone()
    k_rows, nw, nb = rnd(t, d).to(torch.bfloat16), 1 + 0.1 * rnd(d), 0.1 * rnd(d)
    K.dsa_index_append(k_rows, nw, nb, cos, sin, meta, cache_k)
    R.dsa_index_append(k_rows, nw, nb, cos, sin, meta, cache_r)
    torch.cuda.synchronize()
    assert (cache_k.float() - cache_r.float()).abs().max().item() < 0.05
    q = (rnd(t, heads, d) * 0.3).to(torch.bfloat16)
    qk, qr = K.dsa_rope_q(q.clone(), cos, sin, meta), R.dsa_rope_q(q, cos, sin, meta)
    assert (qk.float() - qr.float()).abs().max().item() < 0.02
    w = (rnd(t, heads) * 0.2).float().contiguous()
    sk, sr = K.dsa_index_scores(qr.contiguous(), w, cache_r, meta), R.dsa_index_scores(qr, w, cache_r, meta)
    torch.cuda.synchronize()
    width = sr.shape[1]
    assert torch.equal(torch.isfinite(sk[:, :width]), torch.isfinite(sr)) and not torch.isfinite(sk[:, width:]).any()
    fin = torch.isfinite(sr)
    assert (sk[:, :width][fin] - sr[fin]).abs().max().item() < 2e-2 * max(1.0, sr[fin].abs().max().item())
    sel = K.dsa_topk(sk, topk)
    ref = R.dsa_topk(sk, topk)
    torch.cuda.synchronize()
    for i in range(t):
        a, b = sel[i][sel[i] >= 0].tolist(), sorted(ref[i][ref[i] >= 0].tolist())
        assert a == b and int(sel._pg_counts[i]) == len(b), i  # position order, same set, ties to the earlier key
    # sparse latent attention over the picked keys
    H, nope, vdim, c = 16, 128, 128, 512
    latent = (rnd(nxt, page, c + rope) * 0.3).to(torch.bfloat16)
    qm = (rnd(t, H, nope + rope) * 0.3).to(torch.bfloat16)
    w_uk, w_uv = (rnd(H, nope, c) * 0.05).to(torch.bfloat16), (rnd(H, vdim, c) * 0.05).to(torch.bfloat16)
    scale = (nope + rope) ** -0.5
    out_k = K.mla_attention_sparse(K.mla_rope_q(qm, cos, sin, meta, nope), w_uk, w_uv, latent, meta, scale, c, sel)
    out_r = R.mla_attention_sparse(R.mla_rope_q(qm, cos, sin, meta, nope), w_uk, w_uv, latent, meta, scale, c, sel)
    torch.cuda.synchronize()
    err = (out_k.float() - out_r.float()).abs()
    assert err.max().item() < 0.03 and err.mean().item() < 0.003, (err.max().item(), err.mean().item())
    assert K.read_status(dev) == 0


def test_swiglu_quant_fp8_equals_swiglu_then_quant():
    """The fused SwiGLU + e4m3 quantiser writes the same bytes and scales as the two kernels one after the other."""
    K = cu()
    g = torch.Generator(device=DEV).manual_seed(11)
    for t, k in ((5, 256), (130, 1408 // 128 * 128), (64, 2048)):
        gu = (torch.randn(t, 2 * k, device=DEV, generator=g) * 2).bfloat16()
        q1, s1 = K.quant_fp8_1x128(K.swiglu(gu))
        q2, s2 = K.swiglu_quant_fp8_1x128(gu)
        torch.cuda.synchronize()
        assert torch.equal(q1.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s1, s2)
    status_clean()


@pytest.mark.parametrize("t,m,k", [(1, 256, 512), (7, 1024, 2048), (64, 4096, 4096), (100, 2048, 7168), (16, 12288, 4096)])
def test_fp8_block_scaled_gemm_matches_reference(t, m, k):
    """tcgen05 kind::f8f6f4 GEMM with per-k-group promotion against the dequantised f32 product of the same e4m3 data."""
    K = cu()
    g = torch.Generator(device=DEV).manual_seed(t + m)
    x = (torch.randn(t, k, device=DEV, generator=g) * (1 + torch.rand(t, 1, device=DEV, generator=g) * 3)).to(torch.bfloat16)
    w = torch.randn(m, k, device=DEV, generator=g) * 0.05
    tensors = {"w": w.cpu()}
    from pegainfer_b200.loader.export import quantize_dense_to_fp8

    quantize_dense_to_fp8(tensors, ["w"])
    wq, ws = tensors["w"].to(DEV).contiguous(), tensors["w_scale_inv"].to(DEV).contiguous()
    xq_k, xs_k = K.quant_fp8_1x128(x)
    xq_r, xs_r = R.quant_fp8_1x128(x)
    torch.cuda.synchronize()
    assert torch.equal(xs_k[:, :t], xs_r) or (xs_k[:, :t] - xs_r).abs().max().item() < 1e-6 * xs_r.abs().max().item()
    assert (xq_k.float() - xq_r.float()).abs().max().item() <= 32.0  # at most one e4m3 step at the top of the range
    y = K.linear_fp8_block(x, wq, ws, xq_k, xs_k)
    ref = R.linear_fp8_block(x, wq, ws, xq_k, xs_k)
    torch.cuda.synchronize()
    bf16_close(y, ref, rel=2 ** -6, abs_=2e-2)
    # and the quantised product stays close to the bf16 one
    full = (x.float() @ R.dequant_fp8_block(wq, ws).float().t())
    rel = (y.float() - full).norm() / full.norm()
    assert rel.item() < 0.05, rel.item()
    status_clean()


@pytest.mark.parametrize("page,d", [(16, 128), (64, 128), (16, 256), (64, 256), (32, 256)])
def test_tcgen05_prefill_attention_matches_reference(page, d):
    """Ragged prefill (whole prompts, a chunk behind a cached prefix, a short tail) through the tcgen05 kernels
    (head dim 128: two query tiles per CTA; head dim 256: one query tile, double-buffered scores)."""
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    K = cu()
    hq, hkv = 8, 2
    g = torch.Generator(device=DEV).manual_seed(3)
    cases = [(300, 300), (700, 257), (128, 128), (1000, 130), (90, 70)]  # (kv_len, query rows)
    seqs, nxt = [], 1
    for i, (kl, nq) in enumerate(cases):
        npg = (kl + page - 1) // page
        seqs.append(SeqStep(rid=i, input_tokens=[0] * nq, start_pos=kl - nq, view=KvView(list(range(nxt, nxt + npg)), kl, page)))
        nxt += npg
    _, meta = build_meta(seqs, page, DEV)
    t = meta.num_tokens
    kv = (torch.randn(nxt, 2, page, hkv, d, device=DEV, generator=g) * 0.8).to(torch.bfloat16)
    q = (torch.randn(t, hq, d, device=DEV, generator=g) * 0.8).to(torch.bfloat16)
    ref = R.paged_attention(q, kv, meta).float()
    import ctypes

    from pegainfer_b200 import _native

    errs = {}
    prev = K.set_prefill_tc(0)  # every length through the tcgen05 kernel
    try:
        before = K.launch_count(DEV)
        for variant in (1, 0):
            _native.load().pg_prefill_attention_tc_variant(ctypes.c_int(variant))
            out = K.paged_attention(q, kv, meta).float()
            torch.cuda.synchronize()
            errs[variant] = (out - ref).abs().max().item()
    finally:
        K.set_prefill_tc(prev)
        _native.load().pg_prefill_attention_tc_variant(ctypes.c_int(-1))
    assert errs[1] < 0.03, errs
    if d == 256:  # sliding window on the head-dim-256 kernel: tiles in front of the window are skipped, the edge tiles masked
        prev = K.set_prefill_tc(0)
        try:
            calls = K.PREFILL_TC_CALLS["hd256"]
            for window in (100, 64, 300):
                outw = K.paged_attention(q, kv, meta, None, window).float()
                refw = R.paged_attention(q, kv, meta, None, window).float()
                torch.cuda.synchronize()
                assert (outw - refw).abs().max().item() < 0.03, window
            assert K.PREFILL_TC_CALLS["hd256"] == calls + 3
        finally:
            K.set_prefill_tc(prev)
    status_clean()


def test_int4_repack_kernel_matches_reference_nibble_order():
    K = cu()
    g = torch.Generator(device=DEV).manual_seed(2)
    for shape in ((3, 256, 64), (5, 7), (1, 1, 1030)):
        w = torch.randint(-(2 ** 31), 2 ** 31 - 1, shape, dtype=torch.int32, device=DEV, generator=g)
        got = K.repack_int4_pairs(w)
        want = R.repack_int4_pairs(w)
        torch.cuda.synchronize()
        assert torch.equal(got, want) and got._pg_nibbles == "paired"
        assert torch.equal(R.unrepack_int4_pairs(got), w)


@pytest.mark.parametrize("counts,m,k,bn", [([3, 0, 17, 1, 64, 9], 512, 1024, 16), ([70, 5, 0, 130], 256, 2048, 64), ([1] * 24, 1024, 512, 32)])
def test_grouped_fp8_gemm_matches_dequantised_reference(counts, m, k, bn):
    """Per-expert block-scaled FP8 GEMM on kind::f8f6f4: e4m3 activations (per row and k group) times e4m3 expert weights."""
    from pegainfer_b200.loader.export import quantize_dense_to_fp8

    K = cu()
    g = torch.Generator(device=DEV).manual_seed(len(counts) + m)
    e, rows = len(counts), sum(counts)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    x = (torch.randn(rows, k, device=DEV, generator=g) * 2).to(torch.bfloat16)
    wq, ws = [], []
    for i in range(e):
        d = {"w": torch.randn(m, k, generator=torch.Generator().manual_seed(i)) * 0.05}
        quantize_dense_to_fp8(d, ["w"])
        wq.append(d["w"])
        ws.append(d["w_scale_inv"])
    wq, ws = torch.stack(wq).to(DEV).contiguous(), torch.stack(ws).to(DEV).contiguous()
    xq, xs = K.quant_fp8_1x128(x)
    y = K.grouped_gemm_fp8(xq, xs, offsets, wq, ws, bn)
    torch.cuda.synchronize()
    xf = xq.float().view(rows, k // 128, 128) * xs[:, :rows].t().unsqueeze(-1)
    ref = torch.empty(rows, m, device=DEV)
    for i in range(e):
        r0, r1 = int(offsets[i]), int(offsets[i + 1])
        wf = wq[i].float() * ws[i].repeat_interleave(128, 0)[:m].repeat_interleave(128, 1)[:, :k]
        ref[r0:r1] = xf[r0:r1].view(r1 - r0, k) @ wf.t()
    bf16_close(y, ref, rel=2 ** -6, abs_=2e-2)
    status_clean()


@pytest.mark.parametrize("t,m,k", [(4096, 24576, 4096), (1000, 2048, 1024), (8192, 6144, 2048)])
def test_two_sm_gemm_swiglu_epilogue_equals_gemm_then_swiglu(t, m, k):
    """SwiGLU in the epilogue of the two-SM GEMM (interleaved gate / up rows) writes the bytes of the GEMM followed by the
    SwiGLU kernel."""
    K = cu()
    g = torch.Generator(device=DEV).manual_seed(t + m)
    x = (torch.randn(t, k, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(m, k, device=DEV, generator=g) * 0.05).bfloat16()
    fused = K.linear_swiglu_2sm(x, w)
    if fused is None:  # the two-SM kernel leaves small problems to the other GEMM
        assert t * m < 4096 * 4096
        return
    ref = K.swiglu(K.linear_2sm(x, w), True)
    torch.cuda.synchronize()
    assert torch.equal(fused, ref)
    status_clean()
