"""Drafter forward passes against dense restatements written from the published model definitions."""
import math

import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_model
from pegainfer_b200.kv.request_kv import KvView
from pegainfer_b200.ops.reference import markov_step_argmax
from pegainfer_b200.sched.executor import SeqStep, build_meta
from pegainfer_b200.spec.dflash import DFlashConfig, DFlashDraftModel
from pegainfer_b200.spec.draft_model import _make_kv
from pegainfer_b200.spec.eagle3 import Eagle3Config, Eagle3DraftModel, aux_hidden_state_layers

PAGE = 8


def _target():
    cfg = preset("tiny-qwen3")
    return build_model(cfg, EngineConfig(preset="tiny-qwen3", seed=3), "cpu", torch.float32)


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, cos, sin):
    """x [T, H, D], half-split rotation."""
    c, s = cos[pos].unsqueeze(1), sin[pos].unsqueeze(1)
    h = x.shape[-1] // 2
    a, b = x[..., :h], x[..., h:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def _attend(q, k, v, mask=None):
    """q [Tq, Hq, D], k/v [Tk, Hkv, D]."""
    g = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(q.shape[-1])
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(q.shape[0], -1)


def test_dflash_block_forward_matches_dense_bidirectional_attention():
    tgt = _target()
    cfg = DFlashConfig.for_target(tgt.cfg, num_layers=2, block_size=4)
    d = DFlashDraftModel(cfg, tgt, seed=11)
    kv = _make_kv(d, 16, PAGE)
    g = torch.Generator().manual_seed(0)
    n_ing, n_pend, B = 11, 3, cfg.block_size
    aux = [torch.randn(n_ing + n_pend, cfg.hidden_size, generator=g) for _ in cfg.target_layer_ids]
    ctx = d.project_context(aux)
    view = KvView([3, 1, 2], n_ing + n_pend + B, PAGE)
    _, meta = build_meta([SeqStep(rid=0, input_tokens=[0] * n_ing, start_pos=0, view=view)], PAGE, "cpu")
    d.ingest(ctx[:n_ing], meta, kv)
    cur = 17
    logits = d.block_logits(kv, PAGE, [(view, n_ing, ctx[n_ing:], cur)])
    # dense oracle
    C, eps, hq, hk, D = n_ing + n_pend, cfg.rms_eps, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
    want_ctx = _rms(torch.cat(aux, -1) @ d.fc.t(), d.hidden_norm, eps)
    torch.testing.assert_close(ctx, want_ctx, rtol=1e-5, atol=1e-5)
    toks = torch.tensor([cur] + [cfg.mask_token_id] * (B - 1))
    h = tgt.embed[toks]
    pos_all, pos_blk = torch.arange(C + B), torch.arange(C, C + B)
    for l in d.layers:
        x = _rms(h, l.input_norm, eps)
        tail = torch.cat([want_ctx, x])
        qkv = tail @ l.qkv.t()
        q, k, v = qkv[:, : hq * D], qkv[:, hq * D : (hq + hk) * D], qkv[:, (hq + hk) * D :]
        q = _rope(_rms(q.view(-1, hq, D), l.q_norm, eps), pos_all, d.cos, d.sin)[C:]
        k = _rope(_rms(k.view(-1, hk, D), l.k_norm, eps), pos_all, d.cos, d.sin)
        a = _attend(q, k, v.view(-1, hk, D))  # no mask: the block sees the whole tail
        h = h + a @ l.o.t()
        x = _rms(h, l.post_norm, eps)
        gu = x @ l.gate_up.t()
        half = gu.shape[1] // 2
        h = h + (torch.nn.functional.silu(gu[:, :half]) * gu[:, half:]) @ l.down.t()
    want = _rms(h, d.norm, eps) @ tgt.lm_head.t()
    torch.testing.assert_close(logits, want, rtol=2e-4, atol=2e-4)
    assert d.pick(logits, [cur]) == [want.argmax(-1)[1:].tolist()]
    assert pos_blk[-1] == C + B - 1


def test_dflash_config_reads_nested_and_flat_schemas():
    base = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=100, block_size=16, rms_norm_eps=1e-6, num_target_layers=36)
    a = DFlashConfig.from_hf(dict(base, rope_theta=1e6, dflash_config=dict(mask_token_id=99, target_layer_ids=[1, 9, 17])))
    assert not a.anchor_first and a.num_drafts == 15 and a.context_dim == 192 and a.markov_rank == 0
    b = DFlashConfig.from_hf(dict(base, rope_parameters=dict(rope_theta=5e5), mask_token_id=98, target_layer_ids=[2, 4], num_anchors=1, markov_rank=32))
    assert b.anchor_first and b.num_drafts == 16 and b.rope_theta == 5e5 and b.markov_rank == 32
    assert DFlashConfig.from_hf(a.to_hf()) == a and DFlashConfig.from_hf(b.to_hf()) == b


def test_markov_head_corrects_the_block_left_to_right():
    g = torch.Generator().manual_seed(1)
    rows, B, V, r = 3, 4, 50, 6
    base = torch.randn(rows * B, V, generator=g)
    w1, w2 = torch.randn(V, r, generator=g), torch.randn(V, r, generator=g)
    prev = torch.tensor([4, 9, 30], dtype=torch.int32)
    nxt, drafts = torch.empty_like(prev), torch.zeros(rows * B, dtype=torch.int32)
    p = prev.clone()
    for step in range(B):
        markov_step_argmax(base, w1[p.long()] @ w2.t(), B, step, nxt, drafts)
        p = nxt.clone()
    for i in range(rows):
        t = int(prev[i])
        for step in range(B):
            t = int((base[i * B + step] + w2 @ w1[t]).argmax())
            assert drafts[i * B + step] == t


def test_eagle3_first_step_and_chain_match_dense_layer():
    import dataclasses

    cfg8 = dataclasses.replace(preset("tiny-qwen3"), num_layers=8)
    tgt = build_model(cfg8, EngineConfig(preset="tiny-qwen3", seed=3), "cpu", torch.float32)
    assert aux_hidden_state_layers(36) == (1, 17, 32)
    cfg = Eagle3Config.for_target(tgt.cfg, draft_vocab=300)
    d2t = torch.randint(0, 50, (300,)).cumsum(0) - torch.arange(300) + torch.arange(300)  # increasing offsets
    d2t = torch.clamp(d2t - torch.arange(300), min=0).clamp(max=tgt.cfg.vocab_size - 300)
    d = Eagle3DraftModel(cfg, tgt, seed=5, d2t=d2t)
    kv = _make_kv(d, 16, PAGE)
    g = torch.Generator().manual_seed(2)
    T = 9
    toks = torch.randint(0, 1000, (T,), generator=g).to(torch.int32)
    feat = torch.randn(T, cfg.hidden_size, generator=g)
    view = KvView([2, 5], T + 2, PAGE)
    _, meta = build_meta([SeqStep(rid=0, input_tokens=toks.tolist(), start_pos=0, view=view)], PAGE, "cpu")
    draft, f1 = d.step(toks, feat, meta, kv, torch.tensor([T - 1], dtype=torch.int32))
    eps, hq, hk, D = cfg.rms_eps, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim

    def dense(tok, ft, pos, k_prev=None, v_prev=None):
        x = torch.cat([_rms(tgt.embed[tok.long()], d.input_norm, eps), _rms(ft, d.hidden_norm, eps)], -1)
        qkv = x @ d.qkv.t()
        q = _rope(qkv[:, : hq * D].reshape(-1, hq, D), pos, d.cos, d.sin)
        k = _rope(qkv[:, hq * D : (hq + hk) * D].reshape(-1, hk, D), pos, d.cos, d.sin)
        v = qkv[:, (hq + hk) * D :].reshape(-1, hk, D)
        if k_prev is not None:
            k, v = torch.cat([k_prev, k]), torch.cat([v_prev, v])
        mask = torch.arange(k.shape[0]).view(1, 1, -1) <= pos.view(1, -1, 1)
        h = ft + _attend(q, k, v, mask) @ d.o.t()
        gu = _rms(h, d.post_norm, eps) @ d.gate_up.t()
        half = gu.shape[1] // 2
        h = h + (torch.nn.functional.silu(gu[:, :half]) * gu[:, half:]) @ d.down.t()
        return h, _rms(h, d.norm, eps) @ d.lm_head.t(), k, v

    h, lg, k, v = dense(toks, feat, torch.arange(T))
    torch.testing.assert_close(f1[0], h[-1], rtol=2e-4, atol=2e-4)
    want1 = int(d.d2t[lg[-1].argmax()])
    assert int(draft[0]) == want1
    # second link of the chain: (draft 1, own output) at the next position, attending to everything before
    _, meta2 = build_meta([SeqStep(rid=0, input_tokens=[0], start_pos=T, view=view)], PAGE, "cpu")
    draft2, f2 = d.step(draft.to(torch.int32), f1, meta2, kv, torch.tensor([0], dtype=torch.int32))
    h2, lg2, _, _ = dense(torch.tensor([want1]), h[-1:], torch.tensor([T]), k, v)
    torch.testing.assert_close(f2[0], h2[0], rtol=2e-4, atol=2e-4)
    assert int(draft2[0]) == int(d.d2t[lg2[0].argmax()])
