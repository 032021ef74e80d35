"""Golden gate: every model family against the Hugging Face implementation of the same checkpoint.

A random-weight checkpoint of a tiny preset is written in the real checkpoints' tensor names and
config layout, loaded by this package's loader and by ``transformers``, and the logits of every
prompt position are compared in fp32 (whole prompt and chunked prefill)."""
import tempfile

import pytest
import torch

from pegainfer_b200.config import preset
from pegainfer_b200.loader.export import export_checkpoint
from pegainfer_b200.utils.hf_parity import compare

pytest.importorskip("transformers")


@pytest.mark.parametrize("name,atol", [("tiny-qwen3", 2e-5), ("tiny-qwen35", 2e-5), ("tiny-dsv2", 2e-5), ("tiny-kimi", 5e-4), ("tiny-glm", 5e-4), ("tiny-gemma4", 5e-4)])
def test_prompt_logits_match_hugging_face(name, atol):
    cfg = preset(name)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()  # past tiny-gemma4's sliding window of 32
    with tempfile.TemporaryDirectory() as tmp:
        export_checkpoint(cfg, tmp, dtype=torch.float32)
        whole = compare(tmp, toks)
        chunked = compare(tmp, toks, chunk=16)
    for rep in (whole, chunked):
        assert rep.positions == 40
        assert rep.max_abs_err <= atol, rep
        assert rep.argmax_agreement == 1.0, rep
