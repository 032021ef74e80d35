"""Token selection for one step's logits rows.

Rows are partitioned by policy: *greedy* rows go through one batched argmax
(ties -> lowest index); *sampling* rows go through one batched
temperature/top-k/top-p/min-p pass; rows with an explicit ``seed`` draw from a
per-request counter-based stream keyed by ``mix_seed(seed, step)`` so a replay with
the same seed reproduces the same tokens whatever else is in the batch.

Reference parity: pegainfer-sample/src/lib.rs:56-116 (effectively_greedy),
:133-267 (select_batch), :273-299 (mix_seed, SplitMix64), :310-330
(token_logprob_from_row).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from .. import ops
from ..engine.contract import SamplingParams, TokenLogprob

_MASK64 = (1 << 64) - 1


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK64
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def mix_seed(seed: int, step: int) -> int:
    """Per-(request, step) seed: two SplitMix64 rounds over seed and step."""
    return splitmix64(splitmix64(seed & _MASK64) ^ (step & _MASK64))


def uniform_from_seed(seed64: int) -> float:
    """Uniform in [0,1) from the top 53 bits of a mixed seed.  Clamped so that the value is still
    below 1 after the kernel's conversion to float32 (a double just under 1 rounds up to 1.0f)."""
    return min((splitmix64(seed64) >> 11) * (1.0 / (1 << 53)), 1.0 - 2.0 ** -24)


def select_batch(
    logits: torch.Tensor,
    params: Sequence[SamplingParams],
    steps: Optional[Sequence[int]] = None,
    generator: Optional[torch.Generator] = None,
    base_seed: int = 0,
) -> torch.Tensor:
    """Pick one token per logits row.  Returns int32 ``[rows]`` on the logits device."""
    rows, vocab = logits.shape
    assert len(params) == rows
    steps = steps if steps is not None else [0] * rows
    greedy = [i for i, p in enumerate(params) if p.effectively_greedy(vocab)]
    if len(greedy) == rows:
        return ops.argmax(logits)
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if greedy:
        gi = torch.tensor(greedy, device=logits.device)
        out[gi] = ops.argmax(logits[gi] if len(greedy) != rows else logits)
    samp = [i for i in range(rows) if i not in set(greedy)]
    si = torch.tensor(samp, device=logits.device)
    dev = logits.device
    temp = torch.tensor([params[i].temperature for i in samp], dtype=torch.float32, device=dev)
    top_k = torch.tensor([params[i].top_k if params[i].top_k > 0 else 0 for i in samp], dtype=torch.int32, device=dev)
    top_p = torch.tensor([params[i].top_p for i in samp], dtype=torch.float32, device=dev)
    min_p = torch.tensor([params[i].min_p for i in samp], dtype=torch.float32, device=dev)
    # one uniform per row: seeded rows get their own reproducible stream
    u = []
    for i in samp:
        if params[i].seed is not None:
            u.append(uniform_from_seed(mix_seed(params[i].seed, steps[i])))
        else:
            u.append(None)
    if any(x is None for x in u):
        if generator is None:
            generator = torch.Generator(device="cpu")
            generator.manual_seed(mix_seed(base_seed, sum(steps) + rows) & 0x7FFFFFFFFFFFFFFF)
        r = torch.rand(len(samp), generator=generator).tolist()
        u = [r[j] if x is None else x for j, x in enumerate(u)]
    uu = torch.tensor(u, dtype=torch.float32, device=dev)
    out[si] = ops.sample(logits[si], temp, top_k, top_p, min_p, uu)
    return out


def token_logprob_from_row(row: torch.Tensor, token: int, top_k: int = 0) -> TokenLogprob:
    """Host log-softmax of one logits row with float64 accumulation."""
    r = row.detach().to("cpu", torch.float64)
    m = r.max()
    lse = m + torch.log(torch.exp(r - m).sum())
    top = []
    if top_k > 0:
        tv, ti = (r - lse).topk(top_k)
        top = [(int(i), float(v)) for v, i in zip(tv, ti)]
    return TokenLogprob(token=int(token), logprob=float(r[token] - lse), top=top)


def batch_logprobs(logits: torch.Tensor, picked: torch.Tensor, top_k: int) -> list:
    chosen, tv, ti = ops.logprobs_topk(logits, picked, top_k)
    chosen = chosen.tolist()
    picked_l = picked.tolist()
    out = []
    if top_k > 0:
        tvl, til = tv.tolist(), ti.tolist()
    for i, tok in enumerate(picked_l):
        top = list(zip(til[i], tvl[i])) if top_k > 0 else []
        out.append(TokenLogprob(token=int(tok), logprob=float(chosen[i]), top=top))
    return out
