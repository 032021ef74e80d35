"""Model families on CPU (fp32, tiny presets): paged engine path vs dense recomputation."""
import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import SamplingParams


def gen(name, prompts, max_tokens, **kw):
    ecfg = EngineConfig(preset=name, kv_page_size=16, num_kv_blocks=128, cuda_graph=False, **kw)
    eng = build_engine(ecfg, preset(name), device="cpu", dtype=torch.float32)
    try:
        outs = eng.generate(prompts, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=max_tokens, timeout=300)
        eng.pool.check_invariants()
        return [o[0] for o in outs], eng
    finally:
        eng.shutdown()


def prompts_for(n, length, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (length + 3 * i,), generator=g).tolist() for i in range(n)]


def _chunking_invariance(name):
    ps = prompts_for(3, 40)
    a, _ = gen(name, ps, 6, max_prefill_tokens=512)
    b, _ = gen(name, ps, 6, max_prefill_tokens=24)  # chunked prefill + mixed steps
    c = [gen(name, [p], 6, max_prefill_tokens=512)[0][0] for p in ps]  # one at a time
    assert a == b == c


def test_dsv2_shape_chunking_and_batching_invariance():
    _chunking_invariance("tiny-dsv2")


def test_kimi_shape_int4_group_routing_chunking_invariance():
    _chunking_invariance("tiny-kimi")


def test_mtp_speculative_decode_is_lossless_and_counts_acceptance():
    ps = prompts_for(3, 30, seed=4)
    plain, _ = gen("tiny-kimi", ps, 12)
    spec, eng = gen("tiny-kimi", ps, 12, spec_method="mtp", max_prefill_tokens=20)
    assert spec == plain  # greedy speculative decoding must not change the tokens
    c = eng.scheduler._metrics.spec_decode
    assert c.num_drafts > 0 and c.num_draft_tokens == c.num_drafts and 0 <= c.num_accepted_tokens <= c.num_draft_tokens


def test_accept_prefix_match_truth_table():
    from pegainfer_b200.spec.speculative import accept_prefix_match as f

    assert f([5, 6, 7], [5, 6, 7, 8]) == [5, 6, 7, 8]
    assert f([5, 6, 7], [5, 9, 7, 8]) == [5, 9]
    assert f([5], [4, 1]) == [4]
    assert f([], [3]) == [3]


def test_qwen35_hybrid_chunking_and_batching_invariance():
    _chunking_invariance("tiny-qwen35")


def test_qwen35_recurrent_slots_are_recycled():
    ps = prompts_for(4, 20, seed=9)
    _, eng = gen("tiny-qwen35", ps, 4)
    assert eng.model.rec.by_rid == {}


def test_draft_model_speculative_decode_is_lossless():
    """A separate draft model (other random weights) proposes k tokens per round; greedy output must
    equal plain decoding of the target for every draft length."""
    ps = prompts_for(3, 21, seed=5)
    plain, _ = gen("tiny-qwen3", ps, 14)
    same, eng = gen("tiny-qwen3", ps, 14, spec_method="draft", draft_model_path="preset:tiny-qwen3", spec_draft_len=3, seed=-1, max_prefill_tokens=32)
    other, eng2 = gen("tiny-qwen3", ps, 14, spec_method="draft", draft_model_path="preset:tiny-qwen3", spec_draft_len=2, max_prefill_tokens=32)
    plain_m1, _ = gen("tiny-qwen3", ps, 14, seed=-1)
    assert other == plain
    assert same == plain_m1
    c2 = eng2.scheduler._metrics.spec_decode
    assert c2.num_drafts > 0 and c2.num_draft_tokens == 2 * c2.num_drafts
    assert eng2.scheduler.spec.draft_forwards > 0


def test_fp8_block_scaled_experts_run_and_match_dequantised_reference():
    """Block-scaled FP8 e4m3 expert weights (128x128 scale blocks): quantise/dequantise round trip,
    and an engine with FP8 experts decodes the same tokens whether prompts are chunked or not."""
    from pegainfer_b200.ops import reference as R

    w = torch.randn(300, 520) * 0.05
    q, s = R.quant_fp8_block(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (3, 5)
    assert (R.dequant_fp8_block(q, s).float() - w).abs().max().item() < 0.02
    # experts: FP8 path equals the bf16 path on the dequantised weights
    torch.manual_seed(0)
    e, h, i, t, k = 4, 256, 128, 9, 2
    w13 = torch.randn(e, 2 * i, h) * 0.05
    w2 = torch.randn(e, h, i) * 0.05
    q13, s13 = zip(*[R.quant_fp8_block(w13[j]) for j in range(e)])
    q2, s2 = zip(*[R.quant_fp8_block(w2[j]) for j in range(e)])
    q13, s13, q2, s2 = torch.stack(q13), torch.stack(s13), torch.stack(q2), torch.stack(s2)
    x = torch.randn(t, h)
    ids = torch.stack([torch.randperm(e)[:k] for _ in range(t)]).int()
    wts = torch.rand(t, k)
    a = R.moe_experts_fp8(x, ids, wts, q13, s13, q2, s2)
    d13 = torch.stack([R.dequant_fp8_block(q13[j], s13[j]).float() for j in range(e)])
    d2 = torch.stack([R.dequant_fp8_block(q2[j], s2[j]).float() for j in range(e)])
    b = R.moe_experts(x, ids, wts, d13, d2)
    assert (a - b).abs().max().item() < 1e-4
    # whole engine on the tiny DeepSeek-V2 shape with FP8 experts
    ps = prompts_for(2, 30, seed=2)
    mcfg = preset("tiny-dsv2", expert_quant="fp8_block128")

    def run(chunk):
        ecfg = EngineConfig(preset="tiny-dsv2", kv_page_size=16, num_kv_blocks=128, cuda_graph=False, max_prefill_tokens=chunk)
        eng = build_engine(ecfg, mcfg, device="cpu", dtype=torch.float32)
        try:
            return [o[0] for o in eng.generate(ps, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=5, timeout=300)]
        finally:
            eng.shutdown()

    assert run(512) == run(16)


def test_decode_overlap_prefill_lane_keeps_outputs():
    """With decode overlap, prompt chunks of later requests run on the prefill lane while earlier
    requests keep decoding; the generated tokens are the same as without it."""
    ps = prompts_for(4, 30, seed=8)
    plain, _ = gen("tiny-qwen3", ps, 10, max_prefill_tokens=24)
    over, eng = gen("tiny-qwen3", ps, 10, max_prefill_tokens=24, decode_overlap=True)
    assert over == plain
    assert eng.scheduler.overlapped_chunks > 0


def test_seeded_request_draws_a_distinct_random_number_for_every_token():
    """A seeded request keys its random stream by (seed, request-local step).  The token sampled at
    the end of the prompt and every later decode token must each use a different step."""
    from pegainfer_b200.sample import select as sel

    seen = []
    inner = sel.mix_seed

    def spy(seed, step):
        if seed == 777:
            seen.append(step)
        return inner(seed, step)

    sel.mix_seed = spy
    try:
        ecfg = EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=64, cuda_graph=False, max_prefill_tokens=32)
        eng = build_engine(ecfg, preset("tiny-qwen3"), device="cpu", dtype=torch.float32)
        try:
            ps = prompts_for(2, 40, seed=3)  # longer than one prefill chunk: the prompt takes two steps
            out = eng.generate(ps, SamplingParams(temperature=0.9, top_p=0.95, seed=777, ignore_eos=True), max_tokens=6, timeout=120)
            assert all(len(o[0]) == 6 for o in out)
        finally:
            eng.shutdown()
    finally:
        sel.mix_seed = inner
    # two requests x six tokens; per request the steps are 0..5, each exactly once
    assert sorted(seen) == sorted(list(range(6)) * 2), seen


def _spec_lossless(method, path, rounds_attr="rounds"):
    ps = prompts_for(3, 21, seed=6)
    plain, _ = gen("tiny-qwen3", ps, 14)
    spec, eng = gen("tiny-qwen3", ps, 14, spec_method=method, draft_model_path=path, max_prefill_tokens=16)
    assert spec == plain
    c = eng.scheduler._metrics.spec_decode
    assert c.num_drafts > 0 and getattr(eng.scheduler.spec, rounds_attr) > 0
    return eng, c


def test_dflash_block_drafter_is_lossless_anchor_drop_and_anchor_first():
    """A random block drafter proposes garbage: the output must still equal plain greedy decoding, with
    chunked prefill feeding the draft cache and verify rows joining the next round's context."""
    eng, c = _spec_lossless("dflash", "random:layers=2,block=4")
    assert eng.scheduler.spec.draft_len == 3 and c.num_draft_tokens == 3 * c.num_drafts
    eng, c = _spec_lossless("dflash", "random:layers=1,block=3,anchor_first=1")
    assert eng.scheduler.spec.draft_len == 3


def test_dspark_markov_head_is_lossless_and_sequential():
    eng, c = _spec_lossless("dspark", "random:layers=1,block=3,markov=8")
    assert eng.scheduler.spec.kind == "dspark" and eng.scheduler.spec.draft_len == 3


def test_dflash_drafter_that_knows_the_answer_is_accepted():
    """Acceptance accounting: a drafter whose picks are replaced by the target's own continuation gets every
    draft accepted, and the request finishes in about max_tokens / (drafts + 1) verify rounds."""
    ps = prompts_for(2, 19, seed=8)
    plain, _ = gen("tiny-qwen3", ps, 13)
    from pegainfer_b200.spec import dflash

    truth = {tuple(p): o for p, o in zip(ps, plain)}
    orig = dflash.DFlashSpec.propose

    def oracle(self, decoders):
        out = orig(self, decoders)  # still runs the drafter (cache bookkeeping), then overrides its picks
        for r in decoders:
            toks = r.kv.tokens
            for p, o in truth.items():
                if tuple(toks[: len(p)]) == p:
                    done = len(toks) - len(p)
                    want = o[done : done + self.draft_len]
                    out[r.q.id] = want + [0] * (self.draft_len - len(want))
        return out

    dflash.DFlashSpec.propose = oracle
    try:
        spec, eng = gen("tiny-qwen3", ps, 13, spec_method="dflash", draft_model_path="random:layers=1,block=4")
    finally:
        dflash.DFlashSpec.propose = orig
    assert spec == plain
    c = eng.scheduler._metrics.spec_decode
    assert c.num_accepted_tokens >= c.num_draft_tokens - 2 * 3  # all but each request's last, truncated round
    assert eng.scheduler.spec.rounds <= 5


def test_eagle3_chain_drafter_is_lossless():
    import dataclasses

    cfg = dataclasses.replace(preset("tiny-qwen3"), num_layers=8)
    ps = prompts_for(3, 21, seed=7)

    def run(**kw):
        ecfg = EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=128, cuda_graph=False, **kw)
        eng = build_engine(ecfg, cfg, device="cpu", dtype=torch.float32)
        try:
            return [o[0] for o in eng.generate(ps, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=12, timeout=300)], eng
        finally:
            eng.shutdown()

    plain, _ = run()
    spec, eng = run(spec_method="eagle3", draft_model_path="random:draft_vocab=512", max_prefill_tokens=16)
    assert spec == plain
    s = eng.scheduler.spec
    assert s.draft_len == 3 and s.rounds > 0 and s.draft.aux_layers == (1, 3, 4)
    c = eng.scheduler._metrics.spec_decode
    assert c.num_draft_tokens == 3 * c.num_drafts


def test_gemma4_sliding_and_global_layers_chunking_invariance():
    """tiny-gemma4: five sliding-window layers (window 32, head dim 64) and one global layer (head dim 128, one KV head, V
    from the key projection) over prompts past the window; chunked, batched and one-at-a-time generation must agree."""
    _chunking_invariance("tiny-gemma4")
    from pegainfer_b200.models.gemma4 import Gemma4Model, proportional_rope_tables

    m = Gemma4Model(preset("tiny-gemma4"), device="cpu", dtype=torch.float32)
    assert [l.head_dim for l in m.layers] == [64] * 5 + [128] and [l.kv_heads for l in m.layers] == [2] * 5 + [1]
    assert m.kv_geometry() == dict(num_layers=6, kv_heads=1, head_dim=128) and m.supports_prefix_cache  # 2 x 64 == 1 x 128
    assert torch.equal(m.layers[5].qkv[4 * 128 : 5 * 128], m.layers[5].qkv[5 * 128 :])  # V rows are the K rows
    cos, sin = proportional_rope_tables(64, 128, 0.25, 1e6, torch.float32, "cpu")
    assert cos.shape == (64, 64) and torch.all(cos[:, 16:] == 1) and torch.all(sin[:, 16:] == 0) and sin[5, 0] != 0


def test_glm_sparse_indexer_chunking_invariance_and_mtp():
    """tiny-glm keeps 24 keys per query: prompts of 40+ tokens run the indexer and the sparse latent attention.
    Chunked, batched and one-at-a-time generation must agree, and the MTP head must stay lossless."""
    _chunking_invariance("tiny-glm")
    ps = prompts_for(2, 33, seed=12)
    plain, _ = gen("tiny-glm", ps, 10)
    spec, eng = gen("tiny-glm", ps, 10, spec_method="mtp")
    assert spec == plain and eng.scheduler._metrics.spec_decode.num_drafts > 0


def test_glm_fp8_dense_projections_load_as_fp8_and_generate():
    """With FP8 dense weights the projections outside the experts stay e4m3 + block scales and go through the
    quantise-activations + FP8 GEMM path; chunked and whole-prompt generation must still agree."""
    import dataclasses

    from pegainfer_b200 import ops

    cfg = dataclasses.replace(preset("small-glm-fp8"), hidden_size=256, num_q_heads=4, num_kv_heads=4, q_lora_rank=128, kv_lora_rank=128, qk_nope_head_dim=64, qk_rope_head_dim=64,
                              v_head_dim=64, intermediate_size=256, moe_intermediate_size=128, n_routed_experts=8, num_experts_per_tok=2, index_n_heads=4, index_head_dim=128, index_topk=24,
                              vocab_size=1024, max_position=4096, num_mtp_layers=0)
    ps = prompts_for(2, 41, seed=3)

    def run(chunk):
        eng = build_engine(EngineConfig(preset="small-glm-fp8", kv_page_size=16, num_kv_blocks=64, cuda_graph=False, max_prefill_tokens=chunk), cfg, device="cpu", dtype=torch.float32)
        try:
            L = eng.model.layers
            assert isinstance(L[0].q_b, ops.Fp8Weight) and isinstance(L[0].dense_gate_up, ops.Fp8Weight) and isinstance(L[1].shared_down, ops.Fp8Weight) and isinstance(L[1].idx_wq_b, ops.Fp8Weight)
            assert not isinstance(L[0].kv_a, ops.Fp8Weight)  # 128 + 64 output rows: not a whole number of scale blocks
            outs = eng.generate(ps, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=6, timeout=300)
            assert all(o[1].kind == "finished" for o in outs)
            return [o[0] for o in outs]
        finally:
            eng.shutdown()

    assert run(512) == run(24)
