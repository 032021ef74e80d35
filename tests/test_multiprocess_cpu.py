"""Multi-process paths on CPU (gloo, two ranks): tensor parallel with replicated
schedulers, data-parallel attention with expert parallelism in lock-step, and host-side
detection of a rank that leaves between steps."""
import json
import os
import subprocess
import sys

import pytest
import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import SamplingParams

HERE = os.path.dirname(os.path.abspath(__file__))


def run_workers(mode, tmp_path, world=2, timeout=240):
    out = tmp_path / f"{mode}.json"
    port = 29700 + (os.getpid() + hash(mode)) % 200
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(HERE, "mp_worker.py"), mode, str(out)]
    env = dict(os.environ, OMP_NUM_THREADS="2", PYTHONPATH=os.path.dirname(HERE))
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert out.exists(), f"workers produced no result (rc={r.returncode})\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    return json.loads(out.read_text())


def single_process_tokens(name, n_tok=6):
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (18 + 5 * i,), generator=g).tolist() for i in range(4)]
    ecfg = EngineConfig(preset=name, kv_page_size=16, num_kv_blocks=128, cuda_graph=False, max_prefill_tokens=32)
    eng = build_engine(ecfg, preset(name), device="cpu", dtype=torch.float32)
    try:
        return [o[0] for o in eng.generate(prompts, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=n_tok, timeout=120)]
    finally:
        eng.shutdown()


def test_tensor_parallel_two_ranks_match_single_process(tmp_path):
    res = run_workers("tp", tmp_path)
    assert res["terminals"] == ["finished"] * 4
    assert res["tokens"] == single_process_tokens("tiny-qwen3")


def test_dp_attention_ep_experts_two_ranks_match_single_process(tmp_path):
    res = run_workers("dp_ep", tmp_path)
    assert res["terminals"] == ["finished"] * 4
    assert res["tokens"] == single_process_tokens("tiny-dsv2")


def test_k3_latent_experts_over_two_expert_parallel_ranks_match_single_process(tmp_path):
    """The Kimi-K3 line with its routed experts split over two ranks (tokens gathered, local experts with the saturating
    activation in the latent, outputs reduced): same tokens as one process that owns every expert."""
    res = run_workers("dp_ep_k3", tmp_path)
    assert res["terminals"] == ["finished"] * 4
    assert res["tokens"] == single_process_tokens("tiny-k3")


def test_lost_rank_fails_open_requests_instead_of_hanging(tmp_path):
    res = run_workers("rank_loss", tmp_path)
    assert all(t == "failed" for t in res["terminals"]), res
    assert all(("engine failure" in m) or ("step failed" in m) for m in res["messages"]), res


def test_abort_from_a_client_thread_keeps_tensor_parallel_ranks_on_identical_batches(tmp_path):
    """A client may set a request's abort flag at any moment.  Tensor-parallel ranks run one
    replicated schedule, so the abort must reach every rank's scheduler in the same iteration:
    each rank's log of executed batches (kind, request ids, positions) has to be identical."""
    res = run_workers("abort", tmp_path)
    other = json.loads((tmp_path / "abort.json.rank1").read_text())
    assert res["terminals"][0] == "finished" and res["terminals"][2] == "finished", res["terminals"]
    assert res["terminals"][1] == "aborted" and res["terminals"][3] == "aborted", res["terminals"]
    assert len(res["batches"]) > 20
    assert res["batches"] == other["batches"]
    # the aborted requests really left the batch early: later batches no longer carry their ids
    last = res["batches"][-1]
    assert {row[0] for row in last[1:]} <= {1, 3}
