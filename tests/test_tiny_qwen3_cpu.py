"""Plumbing check on CPU: a tiny Qwen3-architecture decoder (2 layers, hidden 256,
4 Q / 2 KV heads, head_dim 64, QK-norm, RoPE theta 1e6, FFN 768, vocab 1024, fp32,
seed 0) decodes 8 prompts of 32 random tokens for 16 greedy tokens through the
scheduler, the paged KV cache (16-token pages) and the sampler; the result must
equal a dense-attention forward that uses no paging and no scheduler."""
import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import FinishReason, Request, SamplingParams
from pegainfer_b200.ops import reference as R


def dense_greedy(model, prompt, n_new):
    """Recompute the full sequence densely for every new token."""
    cfg = model.cfg
    toks = list(prompt)
    for _ in range(n_new):
        ids = torch.tensor(toks)
        x = model.embed[ids]
        res = x.clone()
        h = R.rms_norm(res, model.layers[0].input_norm, cfg.rms_eps)
        pos = torch.arange(len(toks))
        for i, l in enumerate(model.layers):
            qkv = h @ l.qkv.t()
            q, k, v = qkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size], dim=-1)
            q = R.rms_norm(q.view(-1, cfg.num_q_heads, cfg.head_dim), l.q_norm, cfg.rms_eps)
            k = R.rms_norm(k.view(-1, cfg.num_kv_heads, cfg.head_dim), l.k_norm, cfg.rms_eps)
            v = v.view(-1, cfg.num_kv_heads, cfg.head_dim)
            q = R._rope_half(q, model.cos[pos], model.sin[pos])
            k = R._rope_half(k, model.cos[pos], model.sin[pos])
            a = R.dense_causal_attention(q, k, v).reshape(len(toks), -1)
            res = res + a @ l.o.t()
            h = R.rms_norm(res, l.post_norm, cfg.rms_eps)
            act = R.swiglu(h @ l.gate_up.t())
            res = res + act @ l.down.t()
            nxt = model.layers[i + 1].input_norm if i + 1 < len(model.layers) else model.final_norm
            h = R.rms_norm(res, nxt, cfg.rms_eps)
        logits = h[-1] @ model.lm_head.t()
        toks.append(int(R.argmax(logits.unsqueeze(0))[0]))
    return toks[len(prompt):]


def make_engine(**kw):
    ecfg = EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=128, cuda_graph=False, **kw)
    return build_engine(ecfg, preset("tiny-qwen3"), device="cpu", dtype=torch.float32)


def test_tiny_qwen3_paged_matches_dense():
    eng = make_engine(max_prefill_tokens=64)
    try:
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, 1024, (32,), generator=g).tolist() for _ in range(8)]
        outs = eng.generate(prompts, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=16, timeout=120)
        for p, (toks, term, _) in zip(prompts, outs):
            assert term.kind == "finished" and term.finish_reason == FinishReason.LENGTH
            assert len(toks) == 16
            assert toks == dense_greedy(eng.model, p, 16)
        eng.pool.check_invariants()
        assert eng.pool.used() == 0
    finally:
        eng.shutdown()


def test_chunked_prefill_and_prefix_cache_do_not_change_tokens():
    eng = make_engine(max_prefill_tokens=24)
    try:
        g = torch.Generator().manual_seed(1)
        base = torch.randint(0, 1024, (48,), generator=g).tolist()
        p1 = base + [1, 2, 3]
        p2 = base + [4, 5, 6, 7]
        (t1, _, u1), = eng.generate([p1], max_tokens=6)
        (t2, _, u2), = eng.generate([p2], max_tokens=6)
        cached = [u.cached_tokens for u in u2 if u.cached_tokens is not None]
        assert cached == [48]  # three full 16-token pages shared
        assert [u.cached_tokens for u in u1 if u.cached_tokens is not None] == [0]
        assert t1 == dense_greedy(eng.model, p1, 6)
        assert t2 == dense_greedy(eng.model, p2, 6)
    finally:
        eng.shutdown()


def test_stop_token_is_not_emitted_and_max_tokens_one():
    eng = make_engine()
    try:
        prompt = list(range(10, 30))
        ref = dense_greedy(eng.model, prompt, 4)
        s = eng.submit(Request(prompt_tokens=prompt, max_tokens=8, params=SamplingParams(stop_token_ids=(ref[2],))))
        toks, term, _ = s.collect(60)
        assert toks == ref[:2] and term.finish_reason == FinishReason.STOP
        s = eng.submit(Request(prompt_tokens=prompt, max_tokens=8, params=SamplingParams(stop_token_ids=(ref[0],))))
        toks, term, _ = s.collect(60)
        assert toks == [] and term.finish_reason == FinishReason.STOP
        s = eng.submit(Request(prompt_tokens=prompt, max_tokens=1))
        toks, term, _ = s.collect(60)
        assert toks == ref[:1] and term.finish_reason == FinishReason.LENGTH
    finally:
        eng.shutdown()
