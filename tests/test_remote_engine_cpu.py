"""The engine in a child process behind the frontend's surface: same tokens, aborts, listener, orderly shutdown."""
import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import Request, SamplingParams
from pegainfer_b200.engine.remote import RemoteEngine


def test_remote_engine_matches_in_process_engine_and_aborts():
    ecfg = EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=96, cuda_graph=False)
    g = torch.Generator().manual_seed(4)
    ps = [torch.randint(0, 1024, (20 + 7 * i,), generator=g).tolist() for i in range(3)]
    sp = SamplingParams(temperature=0.0, ignore_eos=True)
    local = build_engine(ecfg, preset("tiny-qwen3"), device="cpu", dtype=torch.float32)
    try:
        want = [o[0] for o in local.generate(ps, sp, max_tokens=7)]
    finally:
        local.shutdown()
    remote = RemoteEngine(ecfg, preset("tiny-qwen3"), device="cpu", dtype=torch.float32, start_timeout=300)
    try:
        assert remote.info.vocab_size == 1024 and remote.healthy()
        got = remote.generate(ps, sp, max_tokens=7)
        assert [o[0] for o in got] == want and all(o[1].kind == "finished" for o in got)
        seen = []
        s = remote.submit(Request(prompt_tokens=ps[0], params=sp, max_tokens=4), listener=seen.append)
        toks, term, _ = s.collect(120)
        assert toks == want[0][:4] and sum(len(u.tokens) for u in seen) == 4
        s2 = remote.submit(Request(prompt_tokens=ps[1], params=sp, max_tokens=600))
        s2.abort()
        toks2, term2, _ = s2.collect(120)
        assert term2.kind == "finished" and len(toks2) < 600
    finally:
        remote.shutdown()
    assert not remote.healthy()
