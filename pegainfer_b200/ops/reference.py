"""Plain PyTorch restatement of every op (oracle for the CUDA kernels, CPU path,
and the library-backed comparison arm on GPU).

Rounding points are explicit: intermediate results are rounded to the activation
dtype exactly where the CUDA kernels round, so kernel tests can use tight bounds.
All activations are token-major ``[tokens, features]``; weights are ``[out, in]``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------------
# metadata shared by reference and CUDA attention paths
# ----------------------------------------------------------------------------------
@dataclass
class AttnMeta:
    """One step's ragged batch description.

    ``q_indptr[b]..q_indptr[b+1]`` are the query rows of sequence ``b``;
    ``kv_lens[b]`` is its KV length *after* this step's append; its pages are
    ``block_table[b, :ceil(kv_lens[b] / page_size)]``.  ``slot_mapping[t]`` is the
    flat KV slot (``page * page_size + offset``) where row ``t`` is appended.
    Padding sequences (CUDA-graph buckets) have ``kv_lens == 0``: they point at
    page 0, attend to nothing and produce zeros.
    """

    q_indptr: torch.Tensor  # int32 [B+1]
    kv_lens: torch.Tensor  # int32 [B]
    block_table: torch.Tensor  # int32 [B, W]
    slot_mapping: torch.Tensor  # int32 [T]
    positions: torch.Tensor  # int32 [T]
    page_size: int
    num_seqs: int
    num_tokens: int
    max_q_len: int
    max_kv_len: int
    decode_only: bool = False
    # host copies (the reference path and planners read these; no device sync)
    h_q_indptr: Optional[list] = None
    h_kv_lens: Optional[list] = None
    # per-step scratch planned by the CUDA path (split-KV partials etc.)
    plan: Optional[object] = None
    # recurrent-state slot of every sequence (hybrid linear-attention models)
    state_slots: Optional[torch.Tensor] = None  # int32 [B]
    # LoRA adapter slot of every token row (None when no request in the step uses one)
    lora_slots: Optional[torch.Tensor] = None  # int32 [T]
    h_state_slots: Optional[list] = None


# ----------------------------------------------------------------------------------
# elementwise / norms
# ----------------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return table[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, offset: bool = False) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + 1.0 if offset else w.float()
    return (xf * inv * wf).to(x.dtype)


def add_rms_norm(x, residual, w, eps, offset=False, round_before_norm=True):
    """``residual += x`` (in place); returns ``rms_norm(residual)``.

    With ``round_before_norm`` the sum is rounded to the activation dtype before the
    mean-square reduction (what the norm then sees is exactly the stored residual);
    otherwise the reduction uses the unrounded fp32 sum.
    """
    s = x.float() + residual.float()
    residual.copy_(s.to(residual.dtype))
    src = residual.float() if round_before_norm else s
    inv = torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + 1.0 if offset else w.float()
    return (src * inv * wf).to(x.dtype)


def geglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``round(gelu_tanh(gate)) * up`` on a fused ``[T, 2I]`` buffer, gate half first."""
    i = gate_up.shape[-1] // 2
    g = gate_up[..., :i].float()
    u = gate_up[..., i:].float()
    a = torch.nn.functional.gelu(g, approximate="tanh").to(gate_up.dtype).float()
    return (a * u).to(gate_up.dtype)


def softcap(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """``cap * tanh(logits / cap)`` (final-logit soft-capping)."""
    return (torch.tanh(logits.float() / cap) * cap).to(logits.dtype)


def gated_rms_norm(x, gate, w, eps, act: str = "silu"):
    """Per-head ``rms_norm(x, w_f32) * silu(gate)``; x, gate: [T, H, D].  ``act="sigmoid"``: the normalised row is
    rounded to the activation dtype and multiplied by the rounded ``sigmoid(gate)`` (the KDA output gate,
    pegainfer-k3/kernels/tilelang_defs.py:398-410)."""
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    g = gate.float()
    if act == "sigmoid":
        return ((xf * inv * w.float()).to(x.dtype).float() * torch.sigmoid(g).to(x.dtype).float()).to(x.dtype)
    return (xf * inv * w.float() * (g * torch.sigmoid(g))).to(x.dtype)


def situ(gate_up: torch.Tensor) -> torch.Tensor:
    """Saturating gated activation on a fused ``[T, 2I]`` buffer (gate half first):
    ``4 tanh(g / 4) sigmoid(g) * 25 tanh(u / 25)`` in f32, rounded once (pegainfer-k3/kernels/tilelang_defs.py:244-262)."""
    i = gate_up.shape[-1] // 2
    g, u = gate_up[..., :i].float(), gate_up[..., i:].float()
    return (4.0 * torch.tanh(g / 4.0) * torch.sigmoid(g) * (25.0 * torch.tanh(u / 25.0))).to(gate_up.dtype)


def attnres_mix(cur, snaps, nb: int, score_w, eps: float):
    """Attention-residual mix.  ``cur`` [T, H] is each token's current residual row, ``snaps`` [T, cap, H] its snapshot
    rows (the first ``nb`` are live).  Every candidate (snapshots, then the current row) scores
    ``dot(x / rms(x), score_w)``; the result is the softmax-weighted sum of the un-normalised candidates
    (pegainfer-k3/kernels/tilelang_defs.py:67-139)."""
    cand = torch.cat([snaps[:, :nb].float(), cur.float().unsqueeze(1)], 1)  # [T, nb + 1, H]
    inv = torch.rsqrt(cand.pow(2).mean(-1) + eps)
    score = (cand * score_w.float()).sum(-1) * inv
    p = torch.softmax(score, -1)
    return (p.unsqueeze(-1) * cand).sum(1).to(cur.dtype)


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def dequant_mxfp4(packed, scales, dtype=torch.bfloat16):
    """MXFP4 to a dense matrix: ``packed`` uint8 [..., K / 2] holds two e2m1 values per byte (low nibble first),
    ``scales`` uint8 [..., K / 32] one e8m0 exponent per 32 values (value ``2 ** (s - 127)``)."""
    lut = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), dtype=torch.float32, device=packed.device)
    b = packed.to(torch.int64)
    vals = torch.stack([lut[b & 15], lut[(b >> 4) & 15]], -1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    sc = torch.exp2(scales.float() - 127.0).repeat_interleave(32, dim=-1)
    return (vals * sc).to(dtype)


def quant_mxfp4(w):
    """Round a matrix to MXFP4 (the inverse layout of ``dequant_mxfp4``): per 32 values the e8m0 scale is the power of two
    that brings the largest magnitude to at most 6, and every value goes to the nearest e2m1 magnitude."""
    k = w.shape[-1]
    g = w.float().reshape(*w.shape[:-1], k // 32, 32)
    amax = g.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    x = g / torch.exp2(e)
    mags = torch.tensor(_E2M1, dtype=torch.float32, device=w.device)
    idx = (x.abs().unsqueeze(-1) - mags).abs().argmin(-1)
    nib = (idx + 8 * (x < 0)).reshape(*w.shape[:-1], k // 2, 2)
    packed = (nib[..., 0] | (nib[..., 1] << 4)).to(torch.uint8)
    return packed, (e.squeeze(-1) + 127).to(torch.uint8)


def swiglu(gate_up: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """``round(silu(gate)) * up`` on a fused ``[T, 2I]`` buffer: gate half first, or with
    ``interleaved`` the columns alternate (gate_0, up_0, gate_1, up_1, ...)."""
    i = gate_up.shape[-1] // 2
    if interleaved:
        g = gate_up[..., 0::2].float()
        u = gate_up[..., 1::2].float()
    else:
        g = gate_up[..., :i].float()
        u = gate_up[..., i:].float()
    s = (g * torch.sigmoid(g)).to(gate_up.dtype).float()
    return (s * u).to(gate_up.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype=None) -> torch.Tensor:
    if x.device.type == "cpu" and x.dtype == torch.bfloat16:
        y = x.float() @ w.float().t()
    else:
        y = F.linear(x, w)
    return y.to(out_dtype or x.dtype)


def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    return x[idx.long()]


# ----------------------------------------------------------------------------------
# RoPE
# ----------------------------------------------------------------------------------
def rope_tables(max_pos: int, rotary_dim: int, theta: float, dtype=torch.bfloat16, device="cpu", scaling: Optional[dict] = None):
    """cos/sin tables ``[max_pos, rotary_dim/2]`` stored in the activation dtype
    (pegainfer-core/src/rope.rs:46-90 keeps them in bf16)."""
    half = rotary_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / rotary_dim))
    mscale = 1.0
    if scaling and scaling.get("type", scaling.get("rope_type")) == "yarn":
        inv_freq, mscale = _yarn_inv_freq(inv_freq, rotary_dim, theta, scaling)
    t = torch.arange(max_pos, dtype=torch.float64)
    ang = torch.outer(t, inv_freq)
    cos = (ang.cos() * mscale).to(torch.float32).to(dtype).to(device)
    sin = (ang.sin() * mscale).to(torch.float32).to(dtype).to(device)
    return cos, sin


def _yarn_inv_freq(inv_freq, dim, theta, sc):
    from ..config import yarn_get_mscale

    factor = sc["factor"]
    orig = sc.get("original_max_position_embeddings", 4096)
    beta_fast, beta_slow = sc.get("beta_fast", 32), sc.get("beta_slow", 1)

    def corr_dim(rot):
        return (dim * math.log(orig / (rot * 2 * math.pi))) / (2 * math.log(theta))

    low = max(math.floor(corr_dim(beta_fast)), 0)
    high = min(math.ceil(corr_dim(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
    mask = 1.0 - ramp
    inv = inv_freq / factor * (1 - mask) + inv_freq * mask
    mscale = yarn_get_mscale(factor, sc.get("mscale", 1.0)) / yarn_get_mscale(factor, sc.get("mscale_all_dim", 0.0))
    return inv, mscale


def _rope_half(x, cos, sin):
    """Half-split rotation of the first ``2*cos.shape[-1]`` dims of x [T,H,D]."""
    r = cos.shape[-1] * 2
    xr = x[..., :r].float()
    x1, x2 = xr[..., : r // 2], xr[..., r // 2 :]
    c, s = cos.float().unsqueeze(1), sin.float().unsqueeze(1)
    o1 = (x1 * c - x2 * s).to(x.dtype)
    o2 = (x2 * c + x1 * s).to(x.dtype)
    return torch.cat([o1, o2, x[..., r:]], dim=-1)


def _rope_interleaved_in(x, cos, sin):
    """Input pairs ``(x[2i], x[2i+1])``, output half-split (DeepSeek convention)."""
    xf = x.float()
    x1, x2 = xf[..., 0::2], xf[..., 1::2]
    c, s = cos.float().unsqueeze(1), sin.float().unsqueeze(1)
    o1 = (x1 * c - x2 * s).to(x.dtype)
    o2 = (x2 * c + x1 * s).to(x.dtype)
    return torch.cat([o1, o2], dim=-1)


def qk_norm_rope_append(qkv, q_norm_w, k_norm_w, cos, sin, meta: AttnMeta, kv_layer, num_q_heads, num_kv_heads, head_dim, eps, offset=False, gated=False, v_norm=False):
    """Split fused qkv rows, per-head RMSNorm on q/k (optional), rotate, append k/v
    to the paged cache (``v_norm``: the value rows get a weightless per-head RMSNorm first).  Returns ``q [T, Hq, D]`` (and ``gate [T, Hq, D]`` if gated:
    q_proj rows are then per-head ``[q(D), gate(D)]``)."""
    t = qkv.shape[0]
    qw = num_q_heads * head_dim * (2 if gated else 1)
    q = qkv[:, :qw]
    k = qkv[:, qw : qw + num_kv_heads * head_dim].reshape(t, num_kv_heads, head_dim)
    v = qkv[:, qw + num_kv_heads * head_dim :].reshape(t, num_kv_heads, head_dim)
    gate = None
    if gated:
        qg = q.reshape(t, num_q_heads, 2, head_dim)
        q, gate = qg[:, :, 0], qg[:, :, 1].contiguous()
    else:
        q = q.reshape(t, num_q_heads, head_dim)
    if q_norm_w is not None:
        q = rms_norm(q, q_norm_w, eps, offset)
        k = rms_norm(k, k_norm_w, eps, offset)
    pos = meta.positions.long()
    c, s = cos[pos], sin[pos]
    q = _rope_half(q, c, s)
    k = _rope_half(k, c, s)
    if v_norm:
        vf = v.float()
        v = (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + eps)).to(v.dtype)
    ps = meta.page_size
    slots = meta.slot_mapping.long()
    kv_layer[slots // ps, 0, slots % ps] = k
    kv_layer[slots // ps, 1, slots % ps] = v
    return (q.contiguous(), gate) if gated else q.contiguous()


# ----------------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------------
def _gather_kv(kv_layer, pages, kv_len, page_size):
    k = kv_layer[pages, 0].reshape(-1, kv_layer.shape[-2], kv_layer.shape[-1])[:kv_len]
    v = kv_layer[pages, 1].reshape(-1, kv_layer.shape[-2], kv_layer.shape[-1])[:kv_len]
    return k, v


def paged_attention(q, kv_layer, meta: AttnMeta, scale: Optional[float] = None, window: int = 0):
    """Causal GQA attention of ragged query rows over paged KV.  q: [T, Hq, D]."""
    t, hq, d = q.shape
    hkv = kv_layer.shape[-2]
    group = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    kl = meta.h_kv_lens if meta.h_kv_lens is not None else meta.kv_lens.tolist()
    ps = meta.page_size
    for b in range(meta.num_seqs):
        q0, q1 = qi[b], qi[b + 1]
        if q1 == q0:
            continue
        if kl[b] == 0:
            out[q0:q1] = 0
            continue
        pages = meta.block_table[b, : (kl[b] + ps - 1) // ps].long()
        k, v = _gather_kv(kv_layer, pages, kl[b], meta.page_size)
        qb = q[q0:q1].float()  # [n, Hq, D]
        kf = k.float().repeat_interleave(group, dim=1)
        vf = v.float().repeat_interleave(group, dim=1)
        s = torch.einsum("qhd,khd->hqk", qb, kf) * scale
        n = q1 - q0
        qpos = torch.arange(kl[b] - n, kl[b], device=q.device).view(1, n, 1)
        kpos = torch.arange(kl[b], device=q.device).view(1, 1, -1)
        mask = kpos <= qpos
        if window > 0:
            mask = mask & (kpos > qpos - window)
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.einsum("hqk,khd->qhd", p, vf).to(q.dtype)
    return out.reshape(t, hq * d)


def dense_causal_attention(q, k, v, scale=None):
    """Unpaged oracle: q [T,Hq,D], k/v [T,Hkv,D], one sequence, causal."""
    t, hq, d = q.shape
    group = hq // k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    kf = k.float().repeat_interleave(group, dim=1)
    vf = v.float().repeat_interleave(group, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    mask = torch.tril(torch.ones(t, t, dtype=torch.bool, device=q.device))
    s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vf).to(q.dtype)


# ----------------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------------
def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Row-wise argmax; ties resolve to the lowest index."""
    lf = logits.float()
    m = lf.max(dim=-1, keepdim=True).values
    idx = torch.arange(lf.shape[-1], device=lf.device).expand_as(lf)
    big = torch.full_like(idx, lf.shape[-1])
    return torch.where(lf == m, idx, big).min(dim=-1).values.to(torch.int32)


def filtered_probs(logits, temperature, top_k, top_p, min_p):
    """Temperature softmax followed by top-k, top-p and min-p filtering, renormalised.
    All controls are per-row tensors.  The keep-set is a threshold on the probability: every
    token at least as likely as the k-th most likely one, and at least as likely as the token
    at which the descending cumulative mass crosses ``top_p`` (so tokens that tie with the
    last kept one are all kept, as in threshold-based samplers), and at least ``min_p`` times
    the most likely one."""
    lf = logits.float() / temperature.clamp_min(1e-6).unsqueeze(-1)
    probs = torch.softmax(lf, dim=-1)
    sp, si = probs.sort(dim=-1, descending=True)
    v = probs.shape[-1]
    k = torch.where(top_k > 0, top_k, torch.full_like(top_k, v)).clamp(max=v).long().unsqueeze(-1)
    thr_k = sp.gather(-1, k - 1)
    csum = sp.double().cumsum(-1)
    before = csum - sp.double()
    crossing = ((before < top_p.double().unsqueeze(-1)).sum(-1, keepdim=True) - 1).clamp_min(0)  # last position still below top_p
    thr_p = sp.gather(-1, crossing)
    keep = (probs >= thr_k) & (probs >= thr_p) & (probs >= min_p.unsqueeze(-1) * sp[:, :1])
    keep |= probs >= sp[:, :1]
    out = probs * keep
    return out / out.sum(-1, keepdim=True)


def logprobs_topk(logits, picked, k):
    lp = torch.log_softmax(logits.float(), dim=-1)
    chosen = lp.gather(-1, picked.long().unsqueeze(-1)).squeeze(-1)
    if k > 0:
        tv, ti = lp.topk(k, dim=-1)
    else:
        tv = ti = None
    return chosen, tv, ti


def sample(logits, temperature, top_k, top_p, min_p, u):
    """Inverse-CDF draw (in vocabulary order) from the filtered distribution using
    one uniform ``u`` per row.  Deterministic given ``u``."""
    probs = filtered_probs(logits, temperature, top_k, top_p, min_p)
    cdf = probs.double().cumsum(-1)
    target = (u.double() * cdf[:, -1]).unsqueeze(-1)
    idx = (cdf <= target).sum(-1).clamp_max(probs.shape[-1] - 1)
    # never return a filtered-out token because of rounding at the tail
    ok = probs.gather(-1, idx.unsqueeze(-1)).squeeze(-1) > 0
    fallback = probs.argmax(-1)
    return torch.where(ok, idx, fallback).to(torch.int32)


# ----------------------------------------------------------------------------------
# MoE routing and experts
# ----------------------------------------------------------------------------------
def router_topk(logits, top_k, scoring="softmax", bias=None, n_group=1, topk_group=1, norm_topk_prob=False, scale=1.0):
    """Expert selection.  ``logits`` [T, E] f32.  Returns (ids int32 [T,k], weights f32 [T,k]).

    softmax: probabilities over all experts, top-k by probability.
    sigmoid: scores = sigmoid(logits); selection on ``scores + bias`` restricted to the
    ``topk_group`` best of ``n_group`` expert groups (group score = sum of its two best
    biased scores); weights come from the un-biased scores.
    Ties resolve to the lowest expert id; ids are returned in selection order
    (descending score).  Weights are renormalised to sum 1 when ``norm_topk_prob`` and
    multiplied by ``scale``."""
    lf = logits.float()
    t, e = lf.shape
    scores = torch.softmax(lf, -1) if scoring == "softmax" else torch.sigmoid(lf)
    choice = scores + bias.float() if bias is not None else scores
    if n_group > 1:
        g = choice.view(t, n_group, e // n_group)
        gscore = g.topk(min(2, e // n_group), dim=-1).values.sum(-1)
        # stable: prefer lower group index on ties
        order = torch.argsort(-gscore, dim=-1, stable=True)[:, :topk_group]
        gmask = torch.zeros(t, n_group, dtype=torch.bool, device=lf.device).scatter_(1, order, True)
        choice = choice.masked_fill(~gmask.unsqueeze(-1).expand_as(g).reshape(t, e), float("-inf"))
    ids = torch.argsort(-choice, dim=-1, stable=True)[:, :top_k]
    w = scores.gather(-1, ids)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.to(torch.int32), (w * scale).float()


def dequant_int4_g32(packed, scales, group=32):
    """compressed-tensors pack-quantized INT4: ``packed`` int32 [out, K/8] holds eight
    offset-binary nibbles (value = nibble - 8), low nibble = lowest k; ``scales``
    [out, K/group].  Returns the dequantised matrix in the scale dtype."""
    out, k8 = packed.shape
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
    nib = (packed.unsqueeze(-1) >> shifts) & 0xF
    q = (nib.to(torch.int32) - 8).reshape(out, k8 * 8).float()
    s = scales.float().repeat_interleave(group, dim=1)
    return (q * s).to(scales.dtype)


def quant_int4_g32(w, group=32):
    """Symmetric INT4 group quantisation (inverse of ``dequant_int4_g32``)."""
    out, k = w.shape
    wf = w.float().view(out, k // group, group)
    s = (wf.abs().amax(-1) / 7.0).clamp_min(1e-8)
    q = torch.clamp(torch.round(wf / s.unsqueeze(-1)), -8, 7).to(torch.int32) + 8
    q = q.view(out, k // 8, 8)
    shifts = torch.arange(0, 32, 4, device=w.device, dtype=torch.int32)
    # keep the bit pattern: pack in int64 then reinterpret the low 32 bits
    packed64 = (q.to(torch.int64) << shifts.to(torch.int64)).sum(-1)
    packed = (packed64 & 0xFFFFFFFF)
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    return packed, s.to(w.dtype)


_PAIR_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)  # nibble position j of a pair-interleaved word holds element _PAIR_ORDER[j]


def _renibble(packed, order, chunk_rows=1 << 16):
    flat = packed.reshape(-1, packed.shape[-1])
    out = torch.empty_like(flat)
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int64)
    for r0 in range(0, flat.shape[0], chunk_rows):
        blk = flat[r0 : r0 + chunk_rows].to(torch.int64) & 0xFFFFFFFF
        nib = (blk.unsqueeze(-1) >> shifts) & 0xF
        new = torch.zeros_like(blk)
        for j, e in enumerate(order):
            new |= nib[..., e] << (4 * j)
        new = torch.where(new >= 2 ** 31, new - 2 ** 32, new)
        out[r0 : r0 + chunk_rows] = new.to(torch.int32)
    return out.reshape(packed.shape)


def repack_int4_pairs(packed):
    """Load-time repack of compressed-tensors INT4 words for the sm_100a grouped GEMM: inside
    every int32 the low 16 bits take elements 0, 2, 4, 6 and the high 16 bits elements 1, 3,
    5, 7, so that one shift + mask yields two consecutive elements as a bf16 pair."""
    out = _renibble(packed, _PAIR_ORDER)
    out._pg_nibbles = "paired"
    return out


def unrepack_int4_pairs(packed):
    inv = [0] * 8
    for j, e in enumerate(_PAIR_ORDER):
        inv[e] = j
    return _renibble(packed, inv)


def plain_int4(packed):
    """The compressed-tensors nibble order of ``packed``, whichever order it is stored in."""
    if getattr(packed, "_pg_nibbles", None) != "paired":
        return packed
    plain = getattr(packed, "_pg_plain_copy", None)
    if plain is None:
        plain = unrepack_int4_pairs(packed)
        packed._pg_plain_copy = plain
    return plain


def dequant_fp8_block(w_fp8, scale_inv, block=128):
    """Block-scaled FP8 e4m3: ``w = fp8 * scale_inv[block_row, block_col]``."""
    out, k = w_fp8.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:out].repeat_interleave(block, 1)[:, :k]
    return (w_fp8.float() * s).to(torch.bfloat16)


def moe_experts(x, ids, weights, w13, w2, expert_offset=0, act: str = "swiglu"):
    """Routed experts on local weights.  ``w13`` [E_local, 2I, H] (gate rows then up
    rows), ``w2`` [E_local, H, I].  Tokens routed to experts outside
    [expert_offset, expert_offset + E_local) contribute nothing.  Returns f32 [T, H]
    (sum over the local selections of weight * expert(x)).  ``act``: ``swiglu`` or ``situ``."""
    t, h = x.shape
    e_local = w13.shape[0]
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    for e in range(e_local):
        sel = ids == (e + expert_offset)
        rows = sel.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        xe = x[rows]
        mid = situ(linear(xe, w13[e])) if act == "situ" else swiglu(linear(xe, w13[e]))
        ye = linear(mid, w2[e]).float()
        we = (weights * sel.float()).sum(-1)[rows]
        out.index_add_(0, rows, ye * we.unsqueeze(-1))
    return out


# ----------------------------------------------------------------------------------
# MLA (multi-head latent attention), absorbed form over a paged latent cache
# ----------------------------------------------------------------------------------
def mla_append(kv_a, kv_norm_w, cos, sin, meta: AttnMeta, latent_layer, kv_lora, eps):
    """Normalise the compressed KV, rotate the shared rope key (interleaved-pair input,
    half-split output) and append ``[ckv | k_pe]`` rows to the paged latent cache
    ``[pages, page_size, kv_lora + rope]``."""
    ckv = rms_norm(kv_a[:, :kv_lora], kv_norm_w, eps)
    pos = meta.positions.long()
    kpe = _rope_interleaved_in(kv_a[:, kv_lora:].unsqueeze(1), cos[pos], sin[pos]).squeeze(1)
    ps = meta.page_size
    slots = meta.slot_mapping.long()
    latent_layer[slots // ps, slots % ps] = torch.cat([ckv, kpe], -1)


def mla_rope_q(q, cos, sin, meta: AttnMeta, nope):
    """q [T, H, nope + rope]: rotate the rope tail (interleaved input -> half-split)."""
    pos = meta.positions.long()
    qpe = _rope_interleaved_in(q[..., nope:], cos[pos], sin[pos])
    return torch.cat([q[..., :nope], qpe], -1)


def mla_attention(q, w_uk, w_uv, latent_layer, meta: AttnMeta, scale, kv_lora):
    """Absorbed MLA: ``q`` [T, H, nope + rope] (rope already applied), ``w_uk``
    [H, nope, kv_lora], ``w_uv`` [H, v, kv_lora].  Returns [T, H * v]."""
    t, h, _ = q.shape
    nope = w_uk.shape[1]
    v = w_uv.shape[1]
    q_abs = torch.einsum("thn,hnc->thc", q[..., :nope].float(), w_uk.float()).to(q.dtype)
    q_pe = q[..., nope:]
    out = torch.zeros(t, h, v, dtype=q.dtype, device=q.device)
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    kl = meta.h_kv_lens if meta.h_kv_lens is not None else meta.kv_lens.tolist()
    ps = meta.page_size
    for b in range(meta.num_seqs):
        q0, q1 = qi[b], qi[b + 1]
        if q1 == q0 or kl[b] == 0:
            continue
        pages = meta.block_table[b, : (kl[b] + ps - 1) // ps].long()
        lat = latent_layer[pages].reshape(-1, latent_layer.shape[-1])[: kl[b]].float()
        ckv, kpe = lat[:, :kv_lora], lat[:, kv_lora:]
        s = (torch.einsum("qhc,kc->hqk", q_abs[q0:q1].float(), ckv) + torch.einsum("qhr,kr->hqk", q_pe[q0:q1].float(), kpe)) * scale
        n = q1 - q0
        qpos = torch.arange(kl[b] - n, kl[b], device=q.device).view(1, n, 1)
        kpos = torch.arange(kl[b], device=q.device).view(1, 1, -1)
        s = s.masked_fill(kpos > qpos, float("-inf"))
        p = torch.softmax(s, -1)
        lo = torch.einsum("hqk,kc->qhc", p, ckv).to(q.dtype)
        out[q0:q1] = torch.einsum("qhc,hvc->qhv", lo.float(), w_uv.float()).to(q.dtype)
    return out.reshape(t, h * v)


def quant_fp8_1x128(x):
    """Per token and 128-wide k group: ``scale = amax / 448``, values rounded to e4m3.  Returns the e4m3 matrix and
    the f32 scales as ``[K / 128, T]`` (pegainfer-kernels/csrc/glm52/glm52_moe_quant.cu, plain float scales)."""
    t, k = x.shape
    g = x.float().view(t, k // 128, 128)
    scale = (g.abs().amax(-1) / 448.0).clamp_min(1e-10 / 448.0)
    q = (g / scale.unsqueeze(-1)).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(t, k)
    return q, scale.t().contiguous()


def linear_fp8_block(x, wq, w_scale, xq=None, x_scale=None):
    """``Y = dequant(Xq) . dequant(Wq)^T`` with 1 x 128 activation groups and 128 x 128 weight blocks, accumulated in f32."""
    if xq is None:
        xq, x_scale = quant_fp8_1x128(x)
    t, k = xq.shape
    xf = xq.float().view(t, k // 128, 128) * x_scale[:, :t].t().unsqueeze(-1)
    m = wq.shape[0]
    wf = wq.float() * w_scale.float().repeat_interleave(128, 0)[:m].repeat_interleave(128, 1)[:, :k]
    return (xf.view(t, k) @ wf.t()).to(torch.bfloat16 if x is None else x.dtype)


# ----------------------------------------------------------------------------------
# Sparse-attention indexer (GLM-5 / DeepSeek-V3.2 style): a light multi-head scorer picks, for every
# query, the keys the main attention may look at
# ----------------------------------------------------------------------------------
def dsa_index_append(k, norm_w, norm_b, cos, sin, meta: AttnMeta, index_layer, eps=1e-6):
    """Index keys ``[T, D]``: LayerNorm (weight and bias), half-split rotation of the leading
    ``2 * cos.shape[-1]`` dims, then append to the paged index cache ``[pages, page_size, D]``."""
    kf = torch.nn.functional.layer_norm(k.float(), (k.shape[-1],), norm_w.float(), norm_b.float(), eps).to(k.dtype)
    pos = meta.positions.long()
    kf = _rope_half(kf.unsqueeze(1), cos[pos], sin[pos]).squeeze(1)
    ps = meta.page_size
    slots = meta.slot_mapping.long()
    index_layer[slots // ps, slots % ps] = kf


def dsa_rope_q(q, cos, sin, meta: AttnMeta):
    """Index queries ``[T, H, D]``: half-split rotation of the leading rope dims."""
    pos = meta.positions.long()
    return _rope_half(q, cos[pos], sin[pos])


def dsa_index_scores(q, w, index_layer, meta: AttnMeta):
    """``score[t, j] = sum_h w[t, h] * relu(q[t, h] . k[j])`` over the keys of row ``t``'s sequence
    that are not in its future; everything else is ``-inf``.  ``q`` [T, H, D] (rotated), ``w`` [T, H]
    f32 (head weights with every constant factor folded in).  Returns ``[T, max_kv_len]`` f32."""
    t = q.shape[0]
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    kl = meta.h_kv_lens if meta.h_kv_lens is not None else meta.kv_lens.tolist()
    width = max([kl[b] for b in range(meta.num_seqs)] + [1])
    out = torch.full((t, width), float("-inf"), dtype=torch.float32, device=q.device)
    ps = meta.page_size
    for b in range(meta.num_seqs):
        q0, q1 = qi[b], qi[b + 1]
        if q1 == q0 or kl[b] == 0:
            continue
        pages = meta.block_table[b, : (kl[b] + ps - 1) // ps].long()
        keys = index_layer[pages].reshape(-1, index_layer.shape[-1])[: kl[b]].float()
        s = torch.relu(torch.einsum("qhd,kd->qhk", q[q0:q1].float(), keys))
        sc = torch.einsum("qhk,qh->qk", s, w[q0:q1].float())
        n = q1 - q0
        qpos = torch.arange(kl[b] - n, kl[b], device=q.device).view(n, 1)
        kpos = torch.arange(kl[b], device=q.device).view(1, -1)
        out[q0:q1, : kl[b]] = sc.masked_fill(kpos > qpos, float("-inf"))
    return out


def dsa_topk(scores, k: int):
    """Positions of each row's ``k`` best finite scores, ``-1`` where a row has fewer; among equal scores the
    earlier position wins (``relu`` makes exact ties common), so the choice does not depend on how wide the
    score matrix of a step happens to be.  ``[T, min(k, width)]`` int32."""
    k = min(k, scores.shape[1])
    val, idx = torch.sort(scores, dim=-1, descending=True, stable=True)
    val, idx = val[:, :k], idx[:, :k]
    return torch.where(torch.isfinite(val), idx, torch.full_like(idx, -1)).to(torch.int32)


def mla_attention_sparse(q, w_uk, w_uv, latent_layer, meta: AttnMeta, scale, kv_lora, select):
    """``mla_attention`` restricted, per query row, to the key positions listed in ``select`` [T, k]
    (``-1`` entries are skipped; the listed positions are already causal)."""
    t, h, _ = q.shape
    nope, v = w_uk.shape[1], w_uv.shape[1]
    q_abs = torch.einsum("thn,hnc->thc", q[..., :nope].float(), w_uk.float()).to(q.dtype)
    q_pe = q[..., nope:]
    out = torch.zeros(t, h, v, dtype=q.dtype, device=q.device)
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    kl = meta.h_kv_lens if meta.h_kv_lens is not None else meta.kv_lens.tolist()
    ps = meta.page_size
    for b in range(meta.num_seqs):
        q0, q1 = qi[b], qi[b + 1]
        if q1 == q0 or kl[b] == 0:
            continue
        pages = meta.block_table[b, : (kl[b] + ps - 1) // ps].long()
        lat = latent_layer[pages].reshape(-1, latent_layer.shape[-1])[: kl[b]].float()
        ckv, kpe = lat[:, :kv_lora], lat[:, kv_lora:]
        s = (torch.einsum("qhc,kc->hqk", q_abs[q0:q1].float(), ckv) + torch.einsum("qhr,kr->hqk", q_pe[q0:q1].float(), kpe)) * scale
        sel = select[q0:q1].long()
        keep = torch.zeros(q1 - q0, kl[b] + 1, dtype=torch.bool, device=q.device)
        keep.scatter_(1, torch.where(sel < 0, torch.full_like(sel, kl[b]), sel), True)
        s = s.masked_fill(~keep[:, : kl[b]].unsqueeze(0), float("-inf"))
        p = torch.softmax(s, -1)
        lo = torch.einsum("hqk,kc->qhc", p, ckv).to(q.dtype)
        out[q0:q1] = torch.einsum("qhc,hvc->qhv", lo.float(), w_uv.float()).to(q.dtype)
    return out.reshape(t, h * v)


def moe_experts_int4(x, ids, weights, w13_packed, w13_scale, w2_packed, w2_scale, expert_offset=0, group=32):
    """``moe_experts`` over INT4 group-quantised weights (dequantised per expert)."""
    t, h = x.shape
    w13_packed, w2_packed = plain_int4(w13_packed), plain_int4(w2_packed)
    e_local = w13_packed.shape[0]
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    for e in range(e_local):
        sel = ids == (e + expert_offset)
        rows = sel.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        w13 = dequant_int4_g32(w13_packed[e], w13_scale[e], group).to(x.dtype)
        w2 = dequant_int4_g32(w2_packed[e], w2_scale[e], group).to(x.dtype)
        act = swiglu(linear(x[rows], w13))
        ye = linear(act, w2).float()
        we = (weights * sel.float()).sum(-1)[rows]
        out.index_add_(0, rows, ye * we.unsqueeze(-1))
    return out


def quant_fp8_block(w, block=128):
    """Block-scaled FP8 e4m3 quantisation (inverse of ``dequant_fp8_block``): one f32
    ``scale_inv`` per ``block x block`` tile, chosen so the tile's largest magnitude maps
    to 448.  Returns ``(w_fp8 [out, K], scale_inv [ceil(out/block), ceil(K/block)])``."""
    out, k = w.shape
    ob, kb = (out + block - 1) // block, (k + block - 1) // block
    wf = torch.zeros(ob * block, kb * block, dtype=torch.float32, device=w.device)
    wf[:out, :k] = w.float()
    tiles = wf.view(ob, block, kb, block)
    scale_inv = (tiles.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
    q = (tiles / scale_inv[:, None, :, None]).view(ob * block, kb * block)[:out, :k]
    return q.to(torch.float8_e4m3fn), scale_inv


def moe_experts_fp8(x, ids, weights, w13_fp8, w13_scale, w2_fp8, w2_scale, expert_offset=0, block=128):
    """``moe_experts`` over block-scaled FP8 weights (dequantised per expert)."""
    t, h = x.shape
    e_local = w13_fp8.shape[0]
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    for e in range(e_local):
        sel = ids == (e + expert_offset)
        rows = sel.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        w13 = dequant_fp8_block(w13_fp8[e], w13_scale[e], block).to(x.dtype)
        w2 = dequant_fp8_block(w2_fp8[e], w2_scale[e], block).to(x.dtype)
        act = swiglu(linear(x[rows], w13))
        ye = linear(act, w2).float()
        we = (weights * sel.float()).sum(-1)[rows]
        out.index_add_(0, rows, ye * we.unsqueeze(-1))
    return out


# ----------------------------------------------------------------------------------
# Gated DeltaNet (linear attention with a gated delta-rule recurrent state)
# ----------------------------------------------------------------------------------
def gdn_conv1d(x, conv_w, conv_state, meta: AttnMeta):
    """Causal depthwise conv (kernel K) + SiLU over ragged sequences with carried state.
    ``x`` [T, C]; ``conv_w`` [C, K]; ``conv_state`` [slots, C, K-1] holds the last K-1
    inputs of each sequence and is updated in place.  The pre-activation sum is rounded
    to the activation dtype before SiLU."""
    t, c = x.shape
    k = conv_w.shape[1]
    out = torch.empty_like(x)
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    slots = meta.h_state_slots if meta.h_state_slots is not None else meta.state_slots.tolist()
    wf = conv_w.float()
    for b in range(meta.num_seqs):
        q0, q1 = qi[b], qi[b + 1]
        if q1 == q0 or slots[b] < 0:
            out[q0:q1] = 0
            continue
        st = conv_state[slots[b]]  # [C, K-1]
        seq = torch.cat([st.t().to(x.dtype), x[q0:q1]], 0)  # [K-1+n, C]
        win = seq.float().unfold(0, k, 1)  # [n, C, K]
        pre = (win * wf.unsqueeze(0)).sum(-1).to(x.dtype).float()
        out[q0:q1] = (pre * torch.sigmoid(pre)).to(x.dtype)
        conv_state[slots[b]] = seq[-(k - 1):].t().to(conv_state.dtype)
    return out


def gdn_gates(a, b, a_log, dt_bias):
    """``g = -exp(A_log) * softplus(a + dt_bias)`` (f32), ``beta = sigmoid(b)`` (f32)."""
    x = a.float() + dt_bias.float()
    sp = torch.where(x > 20.0, x, torch.log1p(torch.exp(x)))
    return -torch.exp(a_log.float()) * sp, torch.sigmoid(b.float())


def gdn_recurrent(q, k, v, g, beta, state, meta: AttnMeta):
    """Token-by-token gated delta rule.  ``q, k`` [T, Hk, Dk], ``v`` [T, Hv, Dv], ``g, beta``
    [T, Hv] f32, ``state`` [slots, Hv, Dk, Dv] f32 updated in place.  Returns [T, Hv, Dv]."""
    t, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    rep = hv // hk
    qf = q.float()
    kf = k.float()
    qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6) * (dk ** -0.5)
    kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    qf = qf.repeat_interleave(rep, dim=1)
    kf = kf.repeat_interleave(rep, dim=1)
    vf = v.float()
    out = torch.zeros(t, hv, dv, dtype=q.dtype, device=q.device)
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    slots = meta.h_state_slots if meta.h_state_slots is not None else meta.state_slots.tolist()
    for b in range(meta.num_seqs):
        if slots[b] < 0:
            continue
        S = state[slots[b]]
        for i in range(qi[b], qi[b + 1]):
            S = S * torch.exp(g[i]).view(hv, 1, 1)
            kv = torch.einsum("hkv,hk->hv", S, kf[i])
            delta = (vf[i] - kv) * beta[i].view(hv, 1)
            S = S + torch.einsum("hk,hv->hkv", kf[i], delta)
            out[i] = torch.einsum("hkv,hk->hv", S, qf[i]).to(q.dtype)
        state[slots[b]] = S
    return out


def kda_recurrent(q, k, v, f, b, a_log, dt_bias, lower: float, state, meta: AttnMeta):
    """Token-by-token delta rule with one decay per key channel (Kimi Delta Attention).  ``q, k`` [T, H, Dk] and ``v``
    [T, H, Dv] after the short convolution, ``f`` [T, H * Dk] the raw forget-gate projection, ``b`` [T, H] the raw beta
    projection, ``a_log`` [H], ``dt_bias`` [H * Dk], ``state`` [slots, H, Dk, Dv] f32 updated in place.  Per token
    ``dec = exp(lower * sigmoid(exp(a_log) * (f + dt_bias)))`` scales the state rows, then the delta rule of
    ``gdn_recurrent`` runs with ``beta = sigmoid(b)`` (pegainfer-k3/kernels/tilelang_defs.py:304-397).  Returns [T, H, Dv]."""
    t, h, dk = q.shape
    dv = v.shape[2]
    qf, kf, vf = q.float(), k.float(), v.float()
    qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6) * (dk ** -0.5)
    kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    raw = f.float().view(t, h, dk) + dt_bias.float().view(h, dk)
    dec = torch.exp(lower * torch.sigmoid(torch.exp(a_log.float()).view(1, h, 1) * raw))
    beta = torch.sigmoid(b.float())
    out = torch.zeros(t, h, dv, dtype=q.dtype, device=q.device)
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    slots = meta.h_state_slots if meta.h_state_slots is not None else meta.state_slots.tolist()
    for s in range(meta.num_seqs):
        if slots[s] < 0:
            continue
        S = state[slots[s]]
        for i in range(qi[s], qi[s + 1]):
            S = S * dec[i].unsqueeze(-1)
            kv = torch.einsum("hkv,hk->hv", S, kf[i])
            delta = (vf[i] - kv) * beta[i].view(h, 1)
            S = S + torch.einsum("hk,hv->hkv", kf[i], delta)
            out[i] = torch.einsum("hkv,hk->hv", S, qf[i]).to(q.dtype)
        state[slots[s]] = S
    return out


def markov_step_argmax(base, bias, block: int, step: int, next_tokens, drafts):
    """One step of a low-rank Markov head over block-drafted logits (pegainfer-qwen3/src/dspark.rs:60-100):
    row ``r`` scores with ``base[r * block + step] + bias[r]``; the argmax is written to ``next_tokens[r]``
    and ``drafts[r, step]`` (``drafts`` is ``[rows * block]`` int32)."""
    rows = bias.shape[0]
    score = base.view(rows, block, -1)[:, step].float() + bias.float()
    tok = score.argmax(-1).to(torch.int32)
    next_tokens[:rows] = tok
    drafts.view(rows, block)[:, step] = tok
    return next_tokens


def sigmoid_gate_mul(x, gate):
    return (x.float() * torch.sigmoid(gate.float())).to(x.dtype)


def lora_delta_multi_(ys, x, As, Bs, scale, slots):
    """``lora_delta_`` for several projections that read the same ``x``."""
    for y, a, b in zip(ys, As, Bs):
        lora_delta_(y, x, a, b, scale, slots)
    return ys


def lora_delta_(y, x, A, B, scale, slots):
    """In place: ``y[t] += scale[s] * B[s] @ (A[s] @ x[t])`` with ``s = slots[t]`` (negative = skip)."""
    sl = slots.tolist()
    for s_id in sorted(set(v for v in sl if v >= 0)):
        rows = torch.tensor([i for i, v in enumerate(sl) if v == s_id], device=x.device)
        tv = x[rows].float() @ A[s_id].float().t()
        y[rows] = (y[rows].float() + float(scale[s_id]) * (tv @ B[s_id].float().t())).to(y.dtype)
    return y


def prefetch_weights(w) -> None:
    """Cache hint of the sm_100a path (next GEMM's weights into L2); nothing to do here."""
