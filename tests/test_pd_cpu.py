"""Prefill / decode disaggregation: two engines joined by one KV store reproduce a single engine's output,
and the decode engine starts from the blocks the prefill engine published."""
import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import Request, SamplingParams
from pegainfer_b200.engine.pd import build_pd_engine


def _ecfg(**kw):
    return EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=96, cuda_graph=False, max_prefill_tokens=48, **kw)


def _prompts(n, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1024, (53 + 17 * i,), generator=g).tolist() for i in range(n)]


def test_pd_pair_matches_single_engine_and_moves_blocks_through_the_store():
    ps = _prompts(3, 1)
    single = build_engine(_ecfg(), preset("tiny-qwen3"), device="cpu", dtype=torch.float32)
    try:
        want = [o[0] for o in single.generate(ps, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=9)]
    finally:
        single.shutdown()
    pd = build_pd_engine(_ecfg(), preset("tiny-qwen3"), prefill_device="cpu", decode_device="cpu", dtype=torch.float32, store_bytes=64 << 20)
    try:
        got = pd.generate(ps, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=9)
        assert [o[0] for o in got] == want
        full_blocks = sum((len(p) - 1) // 16 for p in ps)
        assert pd.handoffs == 3
        assert pd.prefill.host_tier.stats.saves >= full_blocks  # every full prompt block was published before the finish went out
        assert pd.decode.host_tier.stats.host_hits == full_blocks and pd.decode.host_tier.stats.loads == 3
        assert not pd.store.busy
        pd.prefill.pool.check_invariants()
        pd.decode.pool.check_invariants()
        # a second request with the same prompt is a plain prefix hit on the decode engine: nothing is loaded again
        again = pd.generate(ps[:1], SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=9)
        assert again[0][0] == want[0] and pd.decode.host_tier.stats.loads == 3
    finally:
        pd.shutdown()


def test_pd_stream_abort_and_listener():
    pd = build_pd_engine(_ecfg(), preset("tiny-qwen3"), prefill_device="cpu", decode_device="cpu", dtype=torch.float32, store_bytes=16 << 20)
    try:
        seen = []
        s = pd.submit(Request(prompt_tokens=_prompts(1, 2)[0], params=SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=5), listener=seen.append)
        toks, term, _ = s.collect(120)
        assert len(toks) == 5 and term.kind == "finished" and sum(len(u.tokens) for u in seen) == 5 and s.prefill_s is not None
        s2 = pd.submit(Request(prompt_tokens=_prompts(1, 3)[0], params=SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=400))
        s2.abort()
        toks2, term2, _ = s2.collect(120)
        assert term2.kind == "finished" and len(toks2) < 400
    finally:
        pd.shutdown()
