"""Checkpoint I/O and architecture parsing: safetensors round trip, HF Llama directory loading (tied and untied
embeddings, sharded index), fused layouts, co-budget sizing, synthetic workloads, GSM8K parsing helpers."""
import json
import os

import torch

from smcsd_b200.memory.pools import KVSpec, cobudget_pages
from smcsd_b200.models import build_model
from smcsd_b200.models.config import ModelConfig, preset
from smcsd_b200.models.layers import rope_inv_freq
from smcsd_b200.models.llama import LlamaModel, interleave_gate_up, split_gate_up
from smcsd_b200.models.loader import Checkpoint, SafetensorsFile, save_safetensors


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(2, 2).bfloat16(),
         "e": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(t, p, {"format": "pt"})
    f = SafetensorsFile(p)
    assert set(f.keys()) == set(t) and f.metadata["format"] == "pt"
    for k, v in t.items():
        assert torch.equal(f.get(k), v)
    f.close()


def _write_hf_llama(tmp_path, tie: bool, sharded: bool):
    cfg = dict(architectures=["LlamaForCausalLM"], vocab_size=128, hidden_size=64, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, intermediate_size=128, rms_norm_eps=1e-5,
               rope_theta=10000.0, max_position_embeddings=256, tie_word_embeddings=tie, eos_token_id=[5, 6])
    d = tmp_path / ("tied" if tie else "untied")
    os.makedirs(d)
    g = torch.Generator().manual_seed(0)
    sd = {"model.embed_tokens.weight": torch.randn(128, 64, generator=g), "model.norm.weight": torch.randn(64, generator=g)}
    for i in range(2):
        p = f"model.layers.{i}."
        for n, shape in [("self_attn.q_proj", (64, 64)), ("self_attn.k_proj", (32, 64)), ("self_attn.v_proj", (32, 64)),
                         ("self_attn.o_proj", (64, 64)), ("mlp.gate_proj", (128, 64)), ("mlp.up_proj", (128, 64)),
                         ("mlp.down_proj", (64, 128))]:
            sd[p + n + ".weight"] = torch.randn(*shape, generator=g) * 0.1
        sd[p + "input_layernorm.weight"] = torch.randn(64, generator=g)
        sd[p + "post_attention_layernorm.weight"] = torch.randn(64, generator=g)
    if not tie:
        sd["lm_head.weight"] = torch.randn(128, 64, generator=g)
    if sharded:
        keys = sorted(sd)
        half = len(keys) // 2
        wm = {}
        for fn, ks in (("model-00001-of-00002.safetensors", keys[:half]), ("model-00002-of-00002.safetensors", keys[half:])):
            save_safetensors({k: sd[k] for k in ks}, str(d / fn))
            wm.update({k: fn for k in ks})
        with open(d / "model.safetensors.index.json", "w") as f:
            json.dump({"weight_map": wm}, f)
    else:
        save_safetensors(sd, str(d / "model.safetensors"))
    with open(d / "config.json", "w") as f:
        json.dump(cfg, f)
    with open(d / "generation_config.json", "w") as f:
        json.dump({"eos_token_id": 7}, f)
    return str(d), sd


def test_hf_llama_directory_loads_into_fused_layout(tmp_path):
    for tie, sharded in ((False, False), (True, True)):
        path, sd = _write_hf_llama(tmp_path, tie, sharded)
        cfg = ModelConfig.from_pretrained(path)
        assert cfg.arch == "llama" and cfg.head_dim == 16 and sorted(cfg.eos_token_ids) == [5, 6, 7]
        m = build_model(path, torch.float32, "cpu")
        L = m.layers[1]
        assert torch.equal(L.wqkv[:64], sd["model.layers.1.self_attn.q_proj.weight"])
        assert torch.equal(L.wqkv[96:], sd["model.layers.1.self_attn.v_proj.weight"])
        x = torch.randn(3, 64)
        g, u = split_gate_up(x @ L.wgu.t(), m.gu_block)
        assert torch.allclose(g, x @ sd["model.layers.1.mlp.gate_proj.weight"].t(), atol=1e-5)
        assert torch.allclose(u, x @ sd["model.layers.1.mlp.up_proj.weight"].t(), atol=1e-5)
        if tie:
            assert m.lm_head.data_ptr() == m.embed.data_ptr()
        else:
            assert torch.equal(m.lm_head, sd["lm_head.weight"])


def test_tensor_parallel_shards_reassemble():
    cfg = preset("tiny-target")
    full = LlamaModel(cfg, torch.float32, "cpu").init_random(1)
    parts = [LlamaModel(cfg, torch.float32, "cpu", tp_rank=r, tp_size=2).init_random(1) for r in range(2)]
    nq = cfg.q_size // 2
    assert torch.equal(torch.cat([p.layers[0].wqkv[:nq] for p in parts]), full.layers[0].wqkv[:cfg.q_size])
    assert torch.equal(torch.cat([p.layers[0].wo for p in parts], dim=1), full.layers[0].wo)
    assert torch.equal(torch.cat([p.lm_head for p in parts])[:cfg.vocab_size], full.lm_head)


def test_hybrid_tensor_parallel_shards_sum_to_the_full_layers():
    """Emulated ranks: the two shards of a hybrid model, run layer by layer on the same input with their own KV and
    recurrent-state pools, must add up to the unsharded layer outputs (attention and Gated-DeltaNet mixers, MLP), and
    their vocabulary shards must concatenate to the full logits."""
    from smcsd_b200.memory.pools import KVPool, KVSpec, StatePool
    from smcsd_b200.models.hybrid_gdn import HybridGDNModel
    from smcsd_b200.models.layers import ExtendBatch, rmsnorm, swiglu
    from smcsd_b200.models.llama import split_gate_up
    cfg = preset("tiny-hybrid")
    models = [HybridGDNModel(cfg, torch.float32, "cpu").init_random(2)] + \
             [HybridGDNModel(cfg, torch.float32, "cpu", tp_rank=r, tp_size=2).init_random(2) for r in range(2)]
    T = 11
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, cfg.hidden_size, generator=g)
    batch = ExtendBatch(torch.zeros(T, dtype=torch.long), torch.arange(T), torch.arange(1, T + 1, dtype=torch.int32),
                        torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32), extend_len=T,
                        prefix_lens_host=[0])
    bt = torch.zeros(2, 32, dtype=torch.int32)
    bt[0, :T] = torch.arange(1, T + 1)
    outs = []
    for m in models:
        kv = KVPool(KVSpec(len(cfg.attn_layers), m.n_kv_heads, cfg.head_dim, torch.float32), 64, "cpu")
        st = StatePool(m.state_spec(), 2, "cpu")
        res = {}
        for li in (0, 3):                                   # one Gated-DeltaNet layer, one attention layer
            L = m.layers[li]
            xn = rmsnorm(x, L.ln1, cfg.rms_eps, plus_one=True)
            if L.kind == "full_attention":
                res[("mix", li)] = m._attn_layer(L, xn, batch, kv, bt, m.kv_index[li])
            else:
                res[("mix", li)] = m._gdn_layer(L, xn, batch, st, m.state_index[li])
            gate, up = split_gate_up(xn @ L.wgu.t(), m.gu_block)
            res[("mlp", li)] = swiglu(gate, up) @ L.wdown.t()
        res["logits"] = (x @ m.lm_head.t())
        outs.append(res)
    full, a, b = outs
    for key in [("mix", 0), ("mix", 3), ("mlp", 0), ("mlp", 3)]:
        assert torch.allclose(a[key] + b[key], full[key], atol=2e-5, rtol=1e-4), key
    assert torch.allclose(torch.cat([a["logits"], b["logits"]], dim=-1)[:, :cfg.vocab_size], full["logits"], atol=1e-5)


def test_gate_up_interleave_is_invertible_and_llama3_rope_scaling():
    g, u = torch.randn(128, 8), torch.randn(128, 8)
    w = interleave_gate_up(g, u, 64)
    x = torch.randn(2, 8)
    a, b = split_gate_up(x @ w.t(), 64)
    assert torch.allclose(a, x @ g.t(), atol=1e-6) and torch.allclose(b, x @ u.t(), atol=1e-6)
    plain = rope_inv_freq(128, 500000.0, None)
    scaled = rope_inv_freq(128, 500000.0, preset("llama-3.1-8b").rope_scaling)
    assert torch.allclose(scaled[:20], plain[:20]) and torch.allclose(scaled[-1], plain[-1] / 8.0)


def test_cobudget_and_presets():
    t, d = KVSpec(32, 8, 128), KVSpec(16, 8, 64)
    assert t.cell_bytes == 2 * 32 * 8 * 128 * 2
    n = cobudget_pages(10 << 30, t.cell_bytes, d.cell_bytes, draft_weight_bytes=2 << 30, state_bytes=0)
    assert n == (8 << 30) // (t.cell_bytes + d.cell_bytes)
    assert abs(preset("llama-3.1-8b").param_count() - 8.03e9) < 0.1e9
    assert abs(preset("llama-3.2-1b").param_count() - 1.24e9) < 0.05e9
    h = preset("hybrid-gdn-target")
    assert len(h.gdn_layers) == 36 and len(h.attn_layers) == 12


def test_synthetic_workloads_and_gsm8k_helpers():
    from smcsd_b200.bench.accuracy_gsm8k import gold_answer, parse_answer, score
    from smcsd_b200.utils.prompts import lognormal_lengths, random_prompts, uniform_lengths
    lens = lognormal_lengths(2000, seed=3)
    assert min(lens) >= 4 and max(lens) <= 2048 and 150 < sorted(lens)[1000] < 260
    assert all(700 <= x <= 900 for x in uniform_lengths(50))
    assert [len(p) for p in random_prompts([3, 5], 100)] == [3, 5]
    assert gold_answer("blah #### 1,234") == 1234.0
    assert parse_answer("so the total is 12.\n#### 12") == 12.0 and parse_answer("no number") is None
    assert score(["#### 5", "nothing", "#### 7"], [5.0, 1.0, 8.0]) == (1 / 3, 1 / 3)
