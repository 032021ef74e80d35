"""Speculative drafters on a GPU: the Markov-step kernel against its PyTorch restatement, and block /
chain drafters through the engine with the verify step replayed as a widened decode graph."""
import pytest
import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine

pytestmark = pytest.mark.gpu


def test_markov_step_argmax_kernel_matches_reference():
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.ops import reference as R

    g = torch.Generator(device="cuda").manual_seed(0)
    for rows, block, vocab, dt in ((5, 4, 40000, torch.bfloat16), (64, 16, 151936, torch.bfloat16), (3, 2, 1000, torch.float32)):
        base = torch.randn(rows * block, vocab, device="cuda", generator=g).to(dt)
        bias = torch.randn(rows, vocab, device="cuda", generator=g).to(dt)
        for step in (0, block - 1):
            nxt, dr = torch.full((rows,), -1, dtype=torch.int32, device="cuda"), torch.full((rows * block,), -1, dtype=torch.int32, device="cuda")
            rn, rd = nxt.clone(), dr.clone()
            K.markov_step_argmax(base, bias, block, step, nxt, dr)
            R.markov_step_argmax(base, bias, block, step, rn, rd)
            torch.cuda.synchronize()
            score = base.view(rows, block, vocab)[:, step].float() + bias.float()
            # ties between equal bf16 sums may resolve to another index: compare the scores of the picks
            assert torch.equal(score.gather(1, nxt.long()[:, None]), score.gather(1, rn.long()[:, None]))
            assert torch.equal(dr.view(rows, block)[:, step], nxt) and (dr.view(rows, block)[:, [s for s in range(block) if s != step]] == -1).all()
    assert K.read_status("cuda:0") == 0


def _engine(layers, **kw):
    mcfg = preset("qwen3-0.6b", num_layers=layers, vocab_size=8192)
    ecfg = EngineConfig(preset="qwen3-0.6b", num_kv_blocks=512, cuda_graph=True, max_decode_batch=8, max_model_len=1024, max_prefill_tokens=128, batch_invariant=True, **kw)
    return build_engine(ecfg, mcfg, device="cuda:0", dtype=torch.bfloat16)


def _prompts(n, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 8192, (40 + 61 * i,), generator=g).tolist() for i in range(n)]


@pytest.mark.parametrize("method,path,layers,drafts", [
    ("dflash", "random:layers=2,block=4", 3, 3),
    ("dspark", "random:layers=1,block=4,markov=32", 3, 4),
    ("eagle3", "random:draft_vocab=4096", 8, 3),
])
def test_drafters_are_lossless_with_the_verify_graph(method, path, layers, drafts):
    """Under the batch-invariant policy a row's result does not depend on the batch it rides in, so the
    verify rows (a decode graph of requests x span rows) must reproduce plain greedy decoding exactly."""
    from pegainfer_b200.ops import cuda as K

    plain, spec = _engine(layers), _engine(layers, spec_method=method, draft_model_path=path)
    try:
        ps = _prompts(3, 5)
        a = plain.generate(ps, max_tokens=24)
        b = spec.generate(ps, max_tokens=24)
        assert [x[0] for x in a] == [x[0] for x in b]
        s = spec.scheduler.spec
        c = spec.scheduler._metrics.spec_decode
        assert s.draft_len == drafts and s.rounds > 0 and c.num_draft_tokens == drafts * c.num_drafts
        g = spec.executor._graphs
        assert g.replays >= s.rounds and g.aux_layers == tuple(s.aux_layers)  # every verify step was a graph replay
        torch.cuda.synchronize()
        assert K.read_status("cuda:0") == 0
    finally:
        plain.shutdown()
        spec.shutdown()


def test_eagle3_chain_graph_gives_the_drafts_of_the_kernel_by_kernel_chain(monkeypatch):
    """The chain steps of an EAGLE-3 round replayed as a CUDA graph propose the same tokens as the eager chain: the two
    engines accept the same number of draft tokens and emit the same text."""
    ps = _prompts(3, 9)
    stats = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("PEGAINFER_DRAFT_GRAPH", mode)
        eng = _engine(8, spec_method="eagle3", draft_model_path="random:draft_vocab=4096")
        try:
            out = eng.generate(ps, max_tokens=24)
            s, c = eng.scheduler.spec, eng.scheduler._metrics.spec_decode
            stats[mode] = ([x[0] for x in out], c.num_drafts, c.num_accepted_tokens)
            if mode == "1":
                assert s._chain is not None and s._chain.replays == s.rounds > 0
            else:
                assert s._chain is None
        finally:
            eng.shutdown()
    assert stats["1"] == stats["0"]
