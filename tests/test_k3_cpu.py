"""Kimi-K3 line on CPU: the new ops against plain restatements, the model against chunking / batching, MXFP4 loading.

Strategy parity: pegainfer-k3/src/model/plan.rs:693-730 (snapshot geometry), pegainfer-k3/tests/golden_decode.rs
(decode against a stored forward pass; here: chunked, batched and one-at-a-time generation against each other).
"""
import math

import torch

from pegainfer_b200.config import from_hf, preset
from pegainfer_b200.models.k3 import K3Model, k3_shapes, k3_source, layer_geometry
from pegainfer_b200.ops import reference as R
from test_models_cpu import _chunking_invariance, gen, prompts_for


def _meta(lens, slots):
    ind = [0]
    for n in lens:
        ind.append(ind[-1] + n)
    m = R.AttnMeta.__new__(R.AttnMeta)
    m.num_seqs, m.h_q_indptr, m.h_state_slots = len(lens), ind, slots
    m.q_indptr = torch.tensor(ind, dtype=torch.int32)
    m.state_slots = torch.tensor(slots, dtype=torch.int32)
    return m


def test_kda_recurrence_matches_a_per_row_spelling_and_is_chunk_invariant():
    torch.manual_seed(0)
    t, h, d = 11, 3, 32
    q, k, v = (torch.randn(t, h, d) for _ in range(3))
    f, b = torch.randn(t, h * d), torch.randn(t, h)
    a_log, dt = torch.randn(h) * 0.3, torch.randn(h * d) * 0.3
    lower = -5.0
    # plain spelling, state as [head, v, k]: one v row at a time
    S = torch.zeros(h, d, d, dtype=torch.float64)
    want = torch.zeros(t, h, d, dtype=torch.float64)
    for i in range(t):
        for hh in range(h):
            qq = q[i, hh].double() / math.sqrt(float(q[i, hh].double().pow(2).sum()) + 1e-6) * d ** -0.5
            kk = k[i, hh].double() / math.sqrt(float(k[i, hh].double().pow(2).sum()) + 1e-6)
            raw = f[i, hh * d : (hh + 1) * d].double() + dt[hh * d : (hh + 1) * d].double()
            dec = torch.exp(lower * torch.sigmoid(math.exp(float(a_log[hh])) * raw))
            beta = 1.0 / (1.0 + math.exp(-float(b[i, hh])))
            for dv in range(d):
                m = float((S[hh, dv] * dec * kk).sum())
                delta = (float(v[i, hh, dv]) - m) * beta
                S[hh, dv] = S[hh, dv] * dec + delta * kk
                want[i, hh, dv] = float((S[hh, dv] * qq).sum())
    st = torch.zeros(2, h, d, d)
    got = R.kda_recurrent(q, k, v, f, b, a_log, dt, lower, st, _meta([t], [1]))
    assert torch.allclose(got.double(), want, atol=1e-5, rtol=1e-4)
    assert torch.allclose(st[1].double(), S.transpose(1, 2), atol=1e-5, rtol=1e-4) and torch.all(st[0] == 0)
    # two chunks through the carried state give the same rows
    st2 = torch.zeros(2, h, d, d)
    a = R.kda_recurrent(q[:4], k[:4], v[:4], f[:4], b[:4], a_log, dt, lower, st2, _meta([4], [1]))
    c = R.kda_recurrent(q[4:], k[4:], v[4:], f[4:], b[4:], a_log, dt, lower, st2, _meta([t - 4], [1]))
    assert torch.allclose(torch.cat([a, c]), got, atol=1e-6) and torch.allclose(st2, st, atol=1e-6)


def test_attnres_mix_situ_and_sigmoid_gated_norm():
    torch.manual_seed(1)
    t, cap, h, nb = 5, 4, 64, 3
    cur, snaps, sw = torch.randn(t, h), torch.randn(t, cap, h), torch.randn(h)
    got = R.attnres_mix(cur, snaps, nb, sw, 1e-5)
    for i in range(t):
        cands = [snaps[i, c] for c in range(nb)] + [cur[i]]
        sc = torch.tensor([float((x * torch.rsqrt(x.pow(2).mean() + 1e-5) * sw).sum()) for x in cands])
        p = torch.softmax(sc, 0)
        assert torch.allclose(got[i], sum(p[c] * cands[c] for c in range(nb + 1)), atol=1e-5)
    assert torch.allclose(R.attnres_mix(cur, snaps, 0, sw, 1e-5), cur, atol=1e-6)  # a lone candidate is returned as it is
    gu = torch.randn(7, 32) * 8
    g, u = gu[:, :16], gu[:, 16:]
    assert torch.allclose(R.situ(gu), 4 * torch.tanh(g / 4) * torch.sigmoid(g) * 25 * torch.tanh(u / 25), atol=1e-5)
    assert R.situ(torch.full((1, 2), 1000.0)).item() <= 100.0  # saturates at 4 * 25
    x, gate, w = torch.randn(3, 2, 16), torch.randn(3, 2, 16), torch.rand(16)
    want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w * torch.sigmoid(gate)
    assert torch.allclose(R.gated_rms_norm(x, gate, w, 1e-5, act="sigmoid"), want, atol=1e-5)


def test_mxfp4_round_trip():
    torch.manual_seed(2)
    w = torch.randn(6, 64) * 0.05
    pk, sc = R.quant_mxfp4(w)
    assert pk.shape == (6, 32) and pk.dtype == torch.uint8 and sc.shape == (6, 2) and sc.dtype == torch.uint8
    d = R.dequant_mxfp4(pk, sc, torch.float32)
    assert (d - w).abs().max() <= 0.26 * w.abs().max()  # e2m1 steps are at most a quarter of the group maximum apart
    pk2, sc2 = R.quant_mxfp4(d)
    assert torch.equal(R.dequant_mxfp4(pk2, sc2, torch.float32), d)  # values that are representable survive exactly
    one = R.dequant_mxfp4(torch.tensor([[0x2A]], dtype=torch.uint8).repeat(1, 16), torch.tensor([[128]], dtype=torch.uint8), torch.float32)
    assert one[0, 0] == -2.0 and one[0, 1] == 2.0  # low nibble first: 0xA = -1.0, 0x2 = 1.0, scale 2 ** 1


def test_k3_geometry_presets_and_config_round_trip():
    geom, blocks = layer_geometry(93, 12)
    assert blocks == 8 and geom[0] == (True, 0, 1) and geom[1] == (False, 1, 1) and geom[12] == (True, 1, 2) and geom[92][2] == 8
    assert layer_geometry(4, 12)[1] == 1
    full = preset("kimi-k3")
    assert full.layer_types.count("full_attention") == 24 and full.layer_types[3] == "full_attention" and full.layer_types[92] == "full_attention" and full.layer_types[0] == "linear_attention"
    from pegainfer_b200.models.registry import hf_config_extras

    tiny = preset("tiny-k3")
    back = from_hf(hf_config_extras(tiny))
    for key in ("family", "hidden_size", "num_layers", "layer_types", "num_q_heads", "gdn_head_dim", "kda_gate_rank", "q_lora_rank", "kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim",
                "n_routed_experts", "n_shared_experts", "num_experts_per_tok", "moe_intermediate_size", "latent_moe_dim", "attn_res_block", "hidden_act", "first_k_dense_replace", "intermediate_size"):
        assert getattr(back, key) == getattr(tiny, key), key


def test_k3_chunking_and_batching_invariance():
    """tiny-k3: three KDA layers, two MLA layers, snapshots every two layers, one dense and four latent-MoE layers.
    Chunked, batched and one-at-a-time generation must agree (KDA state and conv window carried across chunks, the
    latent cache across steps, the per-token snapshots rebuilt in every pass)."""
    _chunking_invariance("tiny-k3")
    m = K3Model(preset("tiny-k3"), device="cpu", dtype=torch.float32)
    assert (m.n_lin, m.n_mla, m.blocks) == (3, 2, 3) and m.kv_geometry()["num_layers"] == 2 and not m.supports_prefix_cache
    assert [L.snapshot for L in m.layers] == [True, False, True, False, True] and m.layers[0].router is None and m.layers[1].experts["w13"].shape == (8, 128, 128)


def test_k3_mxfp4_experts_load_like_their_dequantised_values():
    cfg = preset("tiny-k3")
    src = k3_source(cfg, seed=3, dtype=torch.float32)
    shapes = k3_shapes(cfg)

    class Mx:
        """The same checkpoint with the routed experts stored as MXFP4."""

        def has(self, name):
            base = name.rsplit(".", 1)[0]
            return (name.endswith((".weight_packed", ".weight_scale")) and ".experts." in name and base + ".weight" in shapes) or (name in shapes and ".experts." not in name)

        def get(self, name, device, dtype=None, rows=None, cols=None):
            if ".experts." in name:
                pk, sc = R.quant_mxfp4(src.get(name.rsplit(".", 1)[0] + ".weight", device, torch.float32))
                return pk if name.endswith("packed") else sc
            return src.get(name, device, dtype, rows, cols)

    class Dq(Mx):
        def has(self, name):
            return name in shapes

        def get(self, name, device, dtype=None, rows=None, cols=None):
            if ".experts." in name:
                return R.dequant_mxfp4(*R.quant_mxfp4(src.get(name, device, torch.float32)), torch.float32)
            return src.get(name, device, dtype, rows, cols)

    a = K3Model(cfg, source=Mx(), device="cpu", dtype=torch.float32)
    b = K3Model(cfg, source=Dq(), device="cpu", dtype=torch.float32)
    assert torch.equal(a.layers[2].experts["w13"], b.layers[2].experts["w13"]) and torch.equal(a.layers[4].experts["w2"], b.layers[4].experts["w2"])
    plain = K3Model(cfg, source=src, device="cpu", dtype=torch.float32)
    assert not torch.equal(a.layers[2].experts["w13"], plain.layers[2].experts["w13"])  # the quantiser did something


def test_k3_generation_through_the_engine_is_deterministic():
    ps = prompts_for(3, 19, seed=5)
    one, _ = gen("tiny-k3", ps, 6)
    again, _ = gen("tiny-k3", ps, 6)
    assert one == again and all(len(t) == 6 for t in one)


def test_k3_checkpoint_directory_round_trip(tmp_path):
    """Write the tiny model as a Hugging Face style directory (wrapper config with a text_config, sharded safetensors with
    the text-tower prefix), load it back through the config probe and the safetensors source: same tokens as the preset."""
    from pegainfer_b200.config import EngineConfig, load_model_config
    from pegainfer_b200.engine.build import build_engine
    from pegainfer_b200.engine.contract import SamplingParams
    from pegainfer_b200.loader.export import export_checkpoint

    cfg = preset("tiny-k3")
    export_checkpoint(cfg, str(tmp_path), seed=0, dtype=torch.float32)
    back = load_model_config(str(tmp_path))
    assert back.family == "kimi_k3" and back.layer_types == cfg.layer_types and back.latent_moe_dim == cfg.latent_moe_dim
    prompt = [list(range(3, 30))]
    outs = []
    for ecfg, mcfg in ((EngineConfig(model_path=str(tmp_path), kv_page_size=16, num_kv_blocks=64, cuda_graph=False), back),
                       (EngineConfig(preset="tiny-k3", kv_page_size=16, num_kv_blocks=64, cuda_graph=False), cfg)):
        eng = build_engine(ecfg, mcfg, device="cpu", dtype=torch.float32)
        try:
            outs.append(eng.generate(prompt, SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=5, timeout=120)[0][0])
        finally:
            eng.shutdown()
    assert outs[0] == outs[1]
