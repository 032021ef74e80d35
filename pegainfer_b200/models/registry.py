"""Model-line registry: one builder per architecture family.

Reference parity: pegainfer-server/src/main.rs:24-41 (compiled-in model lines),
pegainfer-frontend/src/model_line.rs:453-586 (registry, detect by config.json).
"""
from __future__ import annotations

from ..config import ModelConfig


def _qwen3(cfg, **kw):
    from .qwen3 import Qwen3Model

    kw.pop("ep", None)
    return Qwen3Model(cfg, **kw)


def _qwen35(cfg, **kw):
    from .qwen35 import Qwen35Model

    kw.pop("ep", None)
    return Qwen35Model(cfg, **kw)


def _mla_moe(cfg, **kw):
    from .mla_moe import MlaMoeModel

    return MlaMoeModel(cfg, **kw)


BUILDERS = {"qwen3": _qwen3, "qwen35": _qwen35, "deepseek_v2": _mla_moe, "kimi_k2": _mla_moe}


def build(cfg: ModelConfig, **kw):
    if cfg.family not in BUILDERS:
        raise ValueError(f"no model line for family {cfg.family!r}; known: {sorted(BUILDERS)}")
    return BUILDERS[cfg.family](cfg, **kw)


def shapes_for(cfg: ModelConfig) -> dict:
    """Full (unsharded) tensor shapes of a model family that has no entry in ``loader.export``."""
    raise ValueError(f"no tensor-shape table for family {cfg.family!r}")


def hf_config_extras(cfg: ModelConfig) -> dict:
    """Family-specific ``config.json`` keys for ``loader.export.to_hf_config``."""
    return {}
