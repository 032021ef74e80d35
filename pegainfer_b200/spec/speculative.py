"""Speculative decoding: propose, verify in one target forward, accept a prefix.

``accept_prefix_match`` keeps the longest prefix of the drafts that equals what the
target would have produced, plus the one token the target produced itself.  The KV of
rejected positions is rolled back by ``RequestKv.apply_speculative``.

* ``MtpSpec``: the model's own depth-1 multi-token-prediction head drafts one token
  per round; verification is a 2-row forward per request.
* ``DraftModelSpec``: a smaller model of the same vocabulary drafts ``k`` tokens
  autoregressively (its own paged KV).
* ``DFlashSpec`` (``spec.dflash``): a block drafter over the target's hidden states drafts a whole
  block in one forward pass; with a Markov head (DSpark) the block is corrected left to right.
* ``Eagle3Spec`` (``spec.eagle3``): one decoder layer over (next token, fused target feature) pairs
  drafts a chain of three tokens.

A round runs only when every running request is draft-ready, greedy, and wants no
logprobs (pegainfer-qwen3/src/scheduler/plan.rs:153-164); prefix caching is off while
speculation is on (the draft state is not cached).

Reference parity: pegainfer-qwen3/src/speculative.rs:133-195 (accept_prefix_match,
transaction), src/executor.rs execute_speculative_{draft,verify},
pegainfer-kv-cache/src/pool.rs:457-467 (apply_speculative), engine/metrics.rs:59-94.
"""
from __future__ import annotations

from typing import Sequence


def accept_prefix_match(drafts: Sequence[int], target: Sequence[int]) -> list:
    """``target[i]`` is the target model's token after consuming ``drafts[:i]``.  Returns
    the accepted tokens: matching drafts followed by one target token (length 1..k+1)."""
    assert len(target) == len(drafts) + 1
    out = []
    for i, d in enumerate(drafts):
        if target[i] != d:
            break
        out.append(d)
    out.append(target[len(out)])
    return out


class MtpSpec:
    allows_prefix_cache = False
    draft_len = 1
    kind = "mtp"

    def __init__(self, model, executor):
        if getattr(model, "mtp", None) is None:
            raise ValueError("this model has no MTP head (num_mtp_layers == 0)")
        executor.mtp = model.mtp

    def ready(self, r) -> bool:
        req = r.q.request
        return r.spec_state is not None and req.logprobs == 0 and req.params.temperature < 1e-5 and r.lora_slot < 0


def build_spec(ecfg, model, executor):
    if ecfg.spec_method == "mtp":
        return MtpSpec(model, executor)
    if ecfg.spec_method == "draft":
        from .draft_model import DraftModelSpec

        return DraftModelSpec(ecfg, model, executor)
    if ecfg.spec_method in ("dflash", "dspark"):
        from .dflash import DFlashSpec

        spec = DFlashSpec(ecfg, model, executor)
        if ecfg.spec_method == "dspark" and spec.kind != "dspark":
            raise ValueError("--spec-method dspark needs a drafter with a Markov head (markov_rank > 0)")
        return spec
    if ecfg.spec_method == "eagle3":
        from .eagle3 import Eagle3Spec

        return Eagle3Spec(ecfg, model, executor)
    raise ValueError(f"unknown speculative method {ecfg.spec_method!r}")
