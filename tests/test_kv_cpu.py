"""Block pool, request KV lifecycle, host tier and scheduler mechanics (CPU only)."""
import random

import pytest
import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import FinishReason, QueuedRequest, Request, SamplingParams
from pegainfer_b200.engine.ledger import LedgerMisuse, RequestLedger
from pegainfer_b200.kv.block_pool import BlockPool, OutOfBlocks, block_hashes
from pegainfer_b200.kv.request_kv import RequestKv
from pegainfer_b200.sched.executor import ModelExecutor, StepResult
from pegainfer_b200.sched.scheduler import ContinuousScheduler, SchedulerConfig, plan_kind


def test_block_pool_refcounts_lru_and_padding_block():
    pool = BlockPool(6, 4)
    assert pool.usable_blocks == 5 and pool.available() == 5
    a = pool.allocate(3)
    assert 0 not in a
    hs = block_hashes(list(range(12)), 4)
    for b, h in zip(a, hs):
        pool.register(b, h)
    pool.release(a)
    assert pool.num_inactive() == 3 and pool.available() == 5
    assert pool.match_prefix(hs) == a  # revived, in order
    pool.release(a)
    b = pool.allocate(4)  # 2 free + evict 2 LRU inactive (deepest blocks go first)
    assert pool.stats.evictions == 2
    assert pool.match_prefix(hs, acquire=False) == a[:1]
    with pytest.raises(OutOfBlocks):
        pool.allocate(5)
    pool.release(b)
    pool.check_invariants()


def test_request_kv_prefix_leaves_one_token_and_speculative_rollback():
    pool = BlockPool(32, 4)
    p = list(range(100, 116))  # 16 tokens = 4 full blocks
    r1 = RequestKv(pool, p)
    assert r1.match_and_add_prefix() == 0
    r1.schedule_prefill(16)
    assert r1.step_page_indices() == r1.blocks and len(r1.blocks) == 4
    r1.apply_prefill_chunk()
    r1.push_token(7)
    r2 = RequestKv(pool, p)
    assert r2.match_and_add_prefix() == 12  # never the whole prompt: one token must be computed
    assert r2.blocks == r1.blocks[:3]
    # speculative: feed [cur, d1, d2], accept cur + d1
    before = len(r1.blocks)
    r1.schedule_speculative(3)
    assert r1.view().seq_len == 19 and len(r1.blocks) == before + 1
    r1.apply_speculative(2, [8, 9])
    assert r1.committed == 18 and r1.tokens[-2:] == [8, 9] and len(r1.blocks) == 5
    r1.schedule_decode()
    r1.revert_schedule()
    assert r1.scheduled == r1.committed
    r1.release()
    r2.release()
    pool.check_invariants()
    assert pool.used() == 0


def test_block_pool_random_walk_keeps_invariants():
    rng = random.Random(0)
    pool = BlockPool(40, 4)
    live = []
    for step in range(400):
        if live and rng.random() < 0.45:
            live.pop(rng.randrange(len(live))).release()
        else:
            n = rng.randrange(1, 30)
            base = [rng.randrange(3) for _ in range(n)]  # small alphabet -> shared prefixes
            r = RequestKv(pool, base)
            r.match_and_add_prefix()
            need = r.blocks_needed(n - r.committed)
            if need <= pool.available():
                r.schedule_prefill(n - r.committed)
                r.apply_prefill_chunk()
                live.append(r)
            else:
                r.release()
        pool.check_invariants()
    for r in live:
        r.release()
    assert pool.used() == 0


def test_ledger_terminal_exactly_once():
    out = []
    led = RequestLedger(sink=out.append)
    q = QueuedRequest(id=1, request=Request(prompt_tokens=[1]))
    led.register(q)
    led.mark_scheduled(1, 1)
    led.push_tokens(1, [5])
    led.finish(1, FinishReason.LENGTH)
    with pytest.raises(LedgerMisuse):
        led.push_tokens(1, [6])
    with pytest.raises(LedgerMisuse):
        led.finish(1, FinishReason.STOP)
    step = led.commit_step()
    assert len(step.updates) == 1 and step.updates[0].tokens == [5] and step.updates[0].terminal.finish_reason == FinishReason.LENGTH
    assert led.commit_step() is None
    with pytest.raises(LedgerMisuse):
        led.push_tokens(1, [7])  # account retired


def test_plan_truth_table():
    assert plan_kind(True, True, False) == "unified"
    assert plan_kind(True, False, False) == "prefill"
    assert plan_kind(False, True, False) == "decode"
    assert plan_kind(False, True, True) == "spec"
    assert plan_kind(True, True, True) == "unified"
    assert plan_kind(False, False, False) is None


class FakeExecutor(ModelExecutor):
    """Scripted executor: token = (rid * 7 + step) % 97, optional one-shot failure."""

    vocab_size = 1000

    def __init__(self):
        self.fail_next = False
        self.batches = []

    def execute(self, batch):
        self.batches.append((batch.kind, [(s.rid, len(s.input_tokens), s.start_pos) for s in batch.seqs]))
        if self.fail_next:
            self.fail_next = False
            raise RuntimeError("injected decode failure")
        return StepResult(tokens={s.rid: [(s.rid * 7 + s.start_pos) % 97] for s in batch.seqs if s.sample})


def _drive(sched, reqs, steps=200):
    out, done = {}, {}
    led = RequestLedger(sink=lambda so: [out.setdefault(u.id, []).append(u) for u in so.updates])
    for i, r in enumerate(reqs, 1):
        q = QueuedRequest(id=i, request=r)
        led.register(q)
        sched.submit(q)
    for _ in range(steps):
        sched.step(led)
        led.commit_step()
        if not led.open_ids():
            break
    return out


def test_scheduler_chunking_admission_and_failure_containment():
    ex = FakeExecutor()
    pool = BlockPool(20, 4)
    sched = ContinuousScheduler(ex, pool, SchedulerConfig(max_prefill_tokens=6, max_decode_batch=4, max_model_len=64))
    reqs = [Request(prompt_tokens=list(range(10)), max_tokens=3), Request(prompt_tokens=list(range(100, 105)), max_tokens=2), Request(prompt_tokens=[], max_tokens=2), Request(prompt_tokens=list(range(70)), max_tokens=2)]
    out = _drive(sched, reqs)
    # chunk budget 6: first step takes 6 tokens of request 1 only
    assert ex.batches[0] == ("prefill", [(1, 6, 0)])
    # second step: remaining 4 of request 1 plus 2 of request 2 (FIFO within the budget)
    assert ex.batches[1][1][:2] == [(1, 4, 6), (2, 2, 0)]
    assert any(k == "unified" for k, _ in ex.batches)
    t1 = [t for u in out[1] for t in u.tokens]
    assert len(t1) == 3 and out[1][-1].terminal.finish_reason == FinishReason.LENGTH
    assert out[3][-1].terminal.kind == "rejected" and out[4][-1].terminal.kind == "rejected"
    assert pool.used() == 0
    # a failing step fails only the requests in that batch; later requests are served
    ex2 = FakeExecutor()
    sched2 = ContinuousScheduler(ex2, BlockPool(20, 4), SchedulerConfig(max_prefill_tokens=64, max_decode_batch=4, max_model_len=64))
    ex2.fail_next = True
    out2 = _drive(sched2, [Request(prompt_tokens=[1, 2, 3], max_tokens=2)])
    assert out2[1][-1].terminal.kind == "failed"
    out3 = _drive(sched2, [Request(prompt_tokens=[1, 2, 3], max_tokens=2)])
    assert out3[1][-1].terminal.kind == "finished" and sched2.failed_batches == 1


def test_admission_reserves_full_lifetime_blocks():
    ex = FakeExecutor()
    pool = BlockPool(9, 4)  # 8 usable blocks
    sched = ContinuousScheduler(ex, pool, SchedulerConfig(max_prefill_tokens=64, max_decode_batch=8, max_model_len=64))
    led = RequestLedger()
    # each request needs ceil((8 + 8) / 4) = 4 blocks over its lifetime: only two fit
    for i in range(1, 4):
        q = QueuedRequest(id=i, request=Request(prompt_tokens=list(range(8)), max_tokens=8))
        led.register(q)
        sched.submit(q)
    sched.step(led)
    assert len(sched.running) == 2 and len(sched.waiting) == 1
    for _ in range(40):
        sched.step(led)
        led.commit_step()
    assert not led.open_ids() and pool.used() == 0


def test_host_tier_restores_evicted_prefix_and_keeps_tokens():
    mk = lambda **kw: build_engine(EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=64, cuda_graph=False, **kw), preset("tiny-qwen3"), device="cpu", dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    base = torch.randint(0, 1024, (70,), generator=g).tolist()
    plain = mk()
    off = mk(kv_offload=True, kv_offload_host_gib=0.05, kv_offload_l1_disabled=True)
    try:
        a1 = plain.generate([base + [1, 2]], max_tokens=5)[0][0]
        a2 = plain.generate([base + [3, 4, 5]], max_tokens=5)[0][0]
        b1, _, _ = off.generate([base + [1, 2]], max_tokens=5)[0]
        assert off.host_tier.stats.saves >= 4
        b2, _, upd = off.generate([base + [3, 4, 5]], max_tokens=5)[0]
        assert (b1, b2) == (a1, a2)
        cached = [u.cached_tokens for u in upd if u.cached_tokens is not None]
        assert cached == [64] and off.host_tier.stats.loads == 1 and off.host_tier.stats.host_hits == 4
        off.pool.check_invariants()
    finally:
        plain.shutdown()
        off.shutdown()


def test_disk_tier_below_the_host_tier_restores_blocks_evicted_from_host_memory(tmp_path):
    """A host slab of two blocks cannot hold a four-block prefix: the oldest blocks spill to files and
    come back from there when the prefix is asked for again; a second engine finds them on disk too."""
    d = str(tmp_path / "kvdisk")
    cfg = preset("tiny-qwen3")
    probe = build_engine(EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=64, cuda_graph=False, kv_offload=True, kv_offload_host_gib=0.01), cfg, device="cpu", dtype=torch.float32)
    block_bytes = probe.host_tier.block_bytes
    probe.shutdown()
    mk = lambda **kw: build_engine(EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=64, cuda_graph=False, **kw), cfg, device="cpu", dtype=torch.float32)
    host_gib = 2.5 * block_bytes / (1 << 30)  # two slots
    g = torch.Generator().manual_seed(8)
    base = torch.randint(0, 1024, (70,), generator=g).tolist()
    plain = mk()
    off = mk(kv_offload=True, kv_offload_host_gib=host_gib, kv_offload_l1_disabled=True, kv_offload_disk_dir=d, kv_offload_disk_gib=0.05)
    try:
        assert off.host_tier.num_slots == 2 and off.host_tier.disk is not None
        a1 = plain.generate([base + [1, 2]], max_tokens=5)[0][0]
        a2 = plain.generate([base + [3, 4, 5]], max_tokens=5)[0][0]
        b1 = off.generate([base + [1, 2]], max_tokens=5)[0][0]
        off.host_tier.poll()
        off.host_tier.disk.flush()
        assert off.host_tier.stats.evictions >= 2 and off.host_tier.disk.writes >= 2
        b2, _, upd = off.generate([base + [3, 4, 5]], max_tokens=5)[0]
        assert (b1, b2) == (a1, a2)
        cached = [u.cached_tokens for u in upd if u.cached_tokens is not None]
        # the two-slot slab limits one restore to two blocks at a time; what matters: disk blocks were used and tokens match
        assert cached and cached[0] >= 32 and off.host_tier.disk.hits >= 1
        off.pool.check_invariants()
        off.host_tier.disk.flush()
    finally:
        plain.shutdown()
        off.shutdown()
    # content-addressed files survive the process: a fresh engine indexes them at start-up
    again = mk(kv_offload=True, kv_offload_host_gib=host_gib, kv_offload_l1_disabled=True, kv_offload_disk_dir=d, kv_offload_disk_gib=0.05)
    try:
        assert len(again.host_tier.disk.index) >= 2
        c2, _, upd = again.generate([base + [3, 4, 5]], max_tokens=5)[0]
        assert c2 == a2 and again.host_tier.disk.hits >= 1
    finally:
        again.shutdown()


class AheadExecutor(FakeExecutor):
    """The run-ahead protocol as the scheduler sees it: after a decode step flagged ``run_ahead``
    the next position of every non-final request counts as already launched, which needs the
    page of that position in ``table_pages``."""

    supports_run_ahead = True

    def __init__(self, block_size):
        super().__init__()
        self.bs = block_size
        self.pending = {}
        self.claimed = self.wasted = 0

    def execute(self, batch):
        hit = {s.rid for s in batch.seqs if len(s.input_tokens) == 1 and self.pending.get(s.rid) == s.start_pos}
        self.claimed += len(hit)
        self.wasted += len(self.pending) - len(hit)
        self.pending = {}
        res = super().execute(batch)
        if batch.run_ahead:
            assert batch.kind == "decode"
            for s in batch.seqs:
                if not s.final:
                    assert s.table_pages is not None and (s.start_pos + 1) // self.bs < len(s.table_pages), "no page for the position that runs ahead"
                    self.pending[s.rid] = s.start_pos + 1
        return res


def test_run_ahead_lookahead_pages_and_final_marks():
    bs = 4
    reqs = [
        Request(prompt_tokens=list(range(9)), max_tokens=11),
        Request(prompt_tokens=list(range(50, 56)), max_tokens=7, params=SamplingParams(stop_token_ids=(((2 * 7 + 9) % 97),))),  # stops at position 9, unannounced
        Request(prompt_tokens=list(range(20, 23)), max_tokens=1),
        Request(prompt_tokens=list(range(30, 41)), max_tokens=5),
    ]
    # the pool holds exactly the lifetime blocks of all four: look-ahead pages must stay inside the reservation
    need = sum((len(r.prompt_tokens) + r.max_tokens + bs - 1) // bs for r in reqs)
    plain = _drive(ContinuousScheduler(FakeExecutor(), BlockPool(need + 1, bs), SchedulerConfig(max_prefill_tokens=64, max_decode_batch=8, max_model_len=64)), reqs)
    ex = AheadExecutor(bs)
    pool = BlockPool(need + 1, bs)
    sched = ContinuousScheduler(ex, pool, SchedulerConfig(max_prefill_tokens=64, max_decode_batch=8, max_model_len=64, run_ahead=True))
    ahead = _drive(sched, reqs)
    assert sched.failed_batches == 0 and pool.used() == 0
    for rid in plain:
        assert [t for u in plain[rid] for t in u.tokens] == [t for u in ahead[rid] for t in u.tokens]
        assert plain[rid][-1].terminal == ahead[rid][-1].terminal
    assert ahead[2][-1].terminal.finish_reason == FinishReason.STOP
    # every decode row but the first of each request was launched ahead; the only wasted row is the unannounced stop
    assert ex.claimed > 10 and ex.wasted == 1, (ex.claimed, ex.wasted)
    # a request at the context limit is marked final as well
    ex2 = AheadExecutor(bs)
    sched2 = ContinuousScheduler(ex2, BlockPool(8, bs), SchedulerConfig(max_prefill_tokens=64, max_decode_batch=8, max_model_len=12, run_ahead=True))
    out = _drive(sched2, [Request(prompt_tokens=list(range(6)), max_tokens=50)])
    assert out[1][-1].terminal.finish_reason == FinishReason.LENGTH and ex2.wasted == 0 and sched2.failed_batches == 0


def test_thread_binding_and_gc_tuning_are_safe_without_a_gpu():
    """The scheduler thread binds to the executor's GPU when there is one and does nothing on CPU;
    the collector tuning can be applied more than once."""
    import gc

    from pegainfer_b200.engine.driver import _bind_thread_to_device
    from pegainfer_b200.utils.runtime import tune_gc

    class _S:
        ex = FakeExecutor()

    _bind_thread_to_device(_S())  # no device attribute
    _S.ex.device = torch.device("cpu")
    _bind_thread_to_device(_S())
    before = gc.get_threshold()
    try:
        tune_gc()
        tune_gc()
        assert gc.get_threshold()[0] >= 50_000
        assert gc.get_freeze_count() > 0
    finally:
        gc.unfreeze()
        gc.set_threshold(*before)
