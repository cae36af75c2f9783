"""Hybrid Gated-DeltaNet model: math against the HF implementation, checkpoint loading, incremental
decoding vs one-shot prefill, and the SMC engine end to end on a tiny hybrid target (CPU, fp32)."""
import json
import os

import pytest
import torch

from smcsd_b200.memory.pools import KVPool, KVSpec, StatePool
from smcsd_b200.models.config import ModelConfig, preset
from smcsd_b200.models.hybrid_gdn import HybridGDNModel
from smcsd_b200.models.layers import ExtendBatch
from smcsd_b200.models.loader import save_safetensors


def _hf_tiny():
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5ForCausalLM
    cfg = Qwen3_5TextConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=32, linear_num_key_heads=2,
                            linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16,
                            linear_conv_kernel_dim=4, max_position_embeddings=256, rms_norm_eps=1e-6,
                            tie_word_embeddings=False, full_attention_interval=4)
    torch.manual_seed(0)
    model = Qwen3_5ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n or "A_log" in n or "dt_bias" in n:
                p.add_(torch.randn_like(p) * 0.1)
    return cfg, model


def _run(model, ids_list, chunks=None):
    """Runs prompts through forward_torch; ``chunks`` splits each prompt into successive extend calls."""
    cfg = model.cfg
    n_pages = 512
    kv = KVPool(KVSpec(len(cfg.attn_layers), cfg.n_kv_heads, cfg.head_dim, torch.float32), n_pages, "cpu")
    st = StatePool(model.state_spec(), len(ids_list), "cpu")
    bt = torch.zeros(len(ids_list), 128, dtype=torch.int32)
    nxt = 1
    outs = []
    for b, ids in enumerate(ids_list):
        L = len(ids)
        bt[b, :L] = torch.arange(nxt, nxt + L, dtype=torch.int32)
        nxt += L
        pieces = chunks or [L]
        done = 0
        row_out = []
        for e in pieces:
            e = min(e, L - done)
            if e <= 0:
                break
            batch = ExtendBatch(torch.tensor(ids[done:done + e]), torch.arange(done, done + e), bt[b, done:done + e],
                                torch.tensor([b], dtype=torch.int32), torch.tensor([done], dtype=torch.int32),
                                extend_len=e, prefix_lens_host=[done])
            row_out.append(model.logits_torch(model.forward_torch(batch, kv, bt, st)))
            done += e
        outs.append(torch.cat(row_out))
    return outs


def test_matches_hf_qwen3_5_and_loads_its_checkpoint(tmp_path):
    hf_cfg, hf = _hf_tiny()
    d = tmp_path / "ckpt"
    os.makedirs(d)
    save_safetensors({k: v for k, v in hf.state_dict().items()}, str(d / "model.safetensors"))
    with open(d / "config.json", "w") as f:
        json.dump(hf_cfg.to_dict() | {"architectures": ["Qwen3_5ForCausalLM"]}, f)
    cfg = ModelConfig.from_pretrained(str(d))
    assert cfg.arch == "hybrid_gdn" and cfg.layer_types.count("full_attention") == 1
    ours = HybridGDNModel(cfg, torch.float32, "cpu").load_hf(str(d))
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 512, (1, 23), generator=g)
    with torch.no_grad():
        ref = hf(input_ids=ids).logits[0]
    got = _run(ours, [ids[0].tolist()])[0]
    assert (got - ref).abs().max().item() < 2e-3 * max(1.0, ref.abs().max().item())
    # incremental: 7-token prefill, then 2-token head, then single tokens -- same logits as one shot
    inc = _run(ours, [ids[0].tolist()], chunks=[7, 2] + [1] * 14)[0]
    assert (inc - ref).abs().max().item() < 2e-3 * max(1.0, ref.abs().max().item())


def test_engine_with_hybrid_target_and_hybrid_draft_cpu():
    from smcsd_b200 import SMCEngine
    tgt = preset("tiny-hybrid")
    drf = ModelConfig(arch="hybrid_gdn", vocab_size=4096, hidden_size=64, n_layers=2, n_heads=2, n_kv_heads=1,
                      head_dim=32, ffn_size=128, max_position=2048, layer_types=["linear_attention", "full_attention"],
                      gdn_n_k_heads=2, gdn_n_v_heads=2, gdn_head_k_dim=16, gdn_head_v_dim=16, partial_rotary=0.5,
                      attn_output_gate=True, qk_norm=True, norm_plus_one=True, rms_eps=1e-6, name="tiny-hybrid-draft")
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 4096, (14,), generator=g).tolist() for _ in range(3)]
    for defer in (True, False):
        eng = SMCEngine(tgt, drf, n_particles=4, gamma=3, dtype="float32", device="cpu", max_running_requests=2,
                        draft_temperature=0.7, target_temperature=0.7, defer_bonus=defer)
        outs = eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 13, "ignore_eos": True})
        assert [o["completion_tokens"] for o in outs] == [13, 13, 13]
        eng._sched.check_idle_invariants()


def test_hybrid_state_follows_particles_through_resampling():
    """draft == target (same weights): if recurrent state and KV follow the ancestors correctly through
    resampling, the verify pass reproduces the draft probabilities and all log-weights stay ~0."""
    from smcsd_b200.config import EngineArgs
    from smcsd_b200.io_types import GenerateRequest, ParticleOutput, SamplingParams
    from smcsd_b200.models import build_model
    from smcsd_b200.runtime.scheduler import SMCScheduler
    cfg = preset("tiny-hybrid")
    model = build_model(cfg, torch.float32, "cpu", seed=0)
    args = EngineArgs(model_path=cfg, draft_model_path=cfg, n_particles=4, gamma=3, dtype="float32", device="cpu",
                      max_running_requests=1, draft_temperature=0.8, target_temperature=0.8,
                      resample_threshold=2.0).finalize()       # threshold > 1: resample every cycle
    sched = SMCScheduler(args, target=model, draft=model)
    g = torch.Generator().manual_seed(3)
    sched.add_request(GenerateRequest("r", torch.randint(0, 4096, (11,), generator=g).tolist(),
                                      SamplingParams(max_new_tokens=21, ignore_eos=True)))
    outs = sched.run_until_idle()
    po = [o for o in outs if isinstance(o, ParticleOutput)][0]
    assert sched.stats["resampled_groups"] > 0
    assert max(abs(w) for w in po.log_w_tilde) < 1e-3


def test_chunked_delta_rule_equals_token_recurrence():
    from smcsd_b200.models.hybrid_gdn import gdn_chunked, gdn_recurrent_step
    g_ = torch.Generator().manual_seed(0)
    T, H, dk, dv = 150, 3, 16, 24
    q = torch.randn(T, H, dk, generator=g_)
    k = torch.randn(T, H, dk, generator=g_)
    q = q / q.norm(dim=-1, keepdim=True) * dk ** -0.5
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(T, H, dv, generator=g_)
    g = -torch.rand(T, H, generator=g_) * 0.3
    beta = torch.rand(T, H, generator=g_)
    S0 = torch.randn(H, dk, dv, generator=g_) * 0.1
    S, outs = S0.clone(), []
    for t in range(T):
        S, o = gdn_recurrent_step(S, q[t], k[t], v[t], g[t], beta[t])
        outs.append(o)
    ref = torch.stack(outs)
    S2, out2 = gdn_chunked(S0.clone(), q, k, v, g, beta, chunk=64)
    assert (out2 - ref).abs().max() < 1e-4 and (S2 - S).abs().max() < 1e-4
