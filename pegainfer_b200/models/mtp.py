"""Multi-token-prediction head (depth 1) for the MLA + MoE line.

``h' = eh_proj([enorm(embed(next_token)) ; hnorm(hidden)])`` runs through one extra
MLA + MoE block (its own KV layer, same page table as the target), then
``shared_head.norm`` and the shared lm_head: row ``i`` of the output predicts the
token two positions after input row ``i``.  The reference engine has no MTP for this
line (pegainfer-kimi-k2/src has none); the propose / verify / accept transaction
follows its Qwen3 speculative path (pegainfer-qwen3/src/speculative.rs:133-195).
"""
from __future__ import annotations

import torch

from .. import ops


class MtpHead:
    def __init__(self, model, source, layer_index: int):
        self.model = model
        cfg, dev, dt = model.cfg, model.device, model.dtype
        p = f"{model.P}layers.{layer_index}."
        self.layer_index = layer_index
        self.block = model._load_layer(source, layer_index)
        self.enorm = source.get(p + "enorm.weight", dev, dt)
        self.hnorm = source.get(p + "hnorm.weight", dev, dt)
        self.eh_proj = source.get(p + "eh_proj.weight", dev, dt)
        self.head_norm = source.get(p + "shared_head.norm.weight", dev, dt)

    def forward(self, next_tokens: torch.Tensor, hidden: torch.Tensor, meta, kv) -> torch.Tensor:
        """``hidden``: the target's last-layer residual stream [T, H] (before the final
        norm); ``next_tokens`` [T]: the token that follows each row.  Returns normalised
        hidden states [T, H] ready for the shared lm_head."""
        m, eps = self.model, self.model.cfg.rms_eps
        e = ops.rms_norm(ops.embedding(next_tokens, m.embed), self.enorm, eps)
        h = ops.rms_norm(hidden, self.hnorm, eps)
        residual = ops.linear(torch.cat([e, h], -1), self.eh_proj)
        x = ops.rms_norm(residual, self.block.input_norm, eps)
        return m.block(self.block, x, residual, meta, kv.layer(self.layer_index), self.head_norm)
