"""The whole-forward persistent kernel against the one-kernel-per-step chain and the fp32 PyTorch model
(needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(kind):
    from smcsd_b200.models.config import ModelConfig
    if kind == "wide":        # head size 128, GQA group 4
        return ModelConfig(arch="llama", vocab_size=8192, hidden_size=512, n_layers=3, n_heads=8, n_kv_heads=2,
                           head_dim=128, ffn_size=1536, max_position=2048, name="t")
    if kind == "narrow":      # head size 64, tied embeddings
        return ModelConfig(arch="llama", vocab_size=8192, hidden_size=256, n_layers=2, n_heads=4, n_kv_heads=2,
                           head_dim=64, ffn_size=768, max_position=2048, tie_embeddings=True, name="d")
    # short reduction, many gate/up slabs (CTAs own whole slabs), vocabulary that is not a multiple of 128
    return ModelConfig(arch="llama", vocab_size=1000, hidden_size=128, n_layers=1, n_heads=2, n_kv_heads=1,
                       head_dim=64, ffn_size=12800, max_position=2048, name="s")


def _setup(kind, bs, E, P, seed=0):
    """Engine with the given target config; a cached prefix of P tokens per row written by the PyTorch forward."""
    from smcsd_b200 import SMCEngine
    from smcsd_b200.models.layers import ExtendBatch
    import dataclasses
    cfg = _cfg(kind)
    eng = SMCEngine(cfg, dataclasses.replace(_cfg("narrow"), vocab_size=cfg.vocab_size), n_particles=4, gamma=4, draft_temperature=0.7, target_temperature=0.7,
                    max_running_requests=4, context_length=2048, device="cuda", max_total_tokens=32768, random_seed=1,
                    backend="native", cycle_graph=False)
    s = eng._sched
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    rows = torch.arange(bs, dtype=torch.int32, device=dev)
    for b in range(bs):
        s.bt.table[b, :P + E] = s.alloc.alloc(P + E)
    ids = torch.randint(0, cfg.vocab_size, (bs * P,), generator=g, device=dev)
    pos = torch.arange(P, device=dev).repeat(bs)
    locs = s.bt.table[:bs, :P].reshape(-1)
    pre = ExtendBatch(ids, pos, locs, rows, torch.zeros(bs, dtype=torch.int32, device=dev), extend_len=0,
                      extend_lens=[P] * bs, prefix_lens_host=[0] * bs)
    s.target.forward_torch(pre, s.kv_t, s.bt.table)
    ids2 = torch.randint(0, cfg.vocab_size, (bs * E,), generator=g, device=dev, dtype=torch.int32)
    pos2 = (torch.arange(E, device=dev) + P).repeat(bs).to(torch.int32)
    locs2 = s.bt.table[:bs, P:P + E].reshape(-1).contiguous()
    pref = torch.full((bs,), P, dtype=torch.int32, device=dev)
    return eng, s, cfg, rows, ids2, pos2, locs2, pref


@pytest.mark.parametrize("kind,bs,E,P", [("wide", 4, 5, 37), ("wide", 4, 5, 700), ("narrow", 8, 1, 300),
                                          ("narrow", 8, 2, 40), ("slabs", 3, 1, 20), ("wide", 8, 9, 130)])
def test_persistent_forward_matches_chain_and_torch(kind, bs, E, P):
    from smcsd_b200.models.layers import ExtendBatch
    from smcsd_b200.ops import native as K
    from smcsd_b200.ops.native_forward import PersistentLlama, supported
    eng, s, cfg, rows, ids2, pos2, locs2, pref = _setup(kind, bs, E, P)
    m, nm = s.target, s.native_runner.target
    assert supported(m, bs * E)
    M = bs * E
    dev = "cuda"
    # fp32 PyTorch reference of the same pass
    ext = ExtendBatch(ids2.long(), pos2.long(), locs2, rows, pref, extend_len=E, prefix_lens_host=[P] * bs)
    ref_logits = m.logits_torch(m.forward_torch(ext, s.kv_t, s.bt.table))
    # kernel chain
    nm.set_context(P + E, bs, (E,))
    nm.forward(ids2, pos2, locs2, rows, pref, bs, E)
    chain_logits = nm.lm_head(M)[:M].clone()
    chain_hb = nm.hb[:M].float().clone()
    li = len(m.layers) - 1
    chain_k = s.kv_t.k[li][locs2.long()].float().clone()
    chain_v = s.kv_t.v[li][locs2.long()].float().clone()
    s.kv_t.k[:, locs2.long()] = 0
    s.kv_t.v[:, locs2.long()] = 0
    # sampler inputs: even rows score a token, odd rows sample
    tokens_in = torch.full((M,), -1, dtype=torch.int32, device=dev)
    tokens_in[::2] = torch.randint(0, cfg.vocab_size, (tokens_in[::2].numel(),), device=dev, dtype=torch.int32)
    counters = torch.tensor([5, 0, 0, 0], dtype=torch.int64, device=dev)
    T, alpha, seed, call_id = 0.7, 1.3, 1234, 3
    scratch = torch.empty(K.sample_scratch_bytes(M, 32), dtype=torch.uint8, device=dev)
    tok_c = torch.zeros(M, dtype=torch.int32, device=dev)
    lp_c = torch.zeros(M, dtype=torch.float32, device=dev)
    lz_c = torch.zeros(M, dtype=torch.float32, device=dev)
    K.sample_or_score(chain_logits, rows=M, V=cfg.vocab_size, splits=1, split_stride=0,
                      row_stride=chain_logits.stride(0), temperature=T, alpha=alpha, softcap=0.0, tokens_in=tokens_in,
                      seed=seed, cycle_counter=counters, call_id=call_id, scratch=scratch, nchunks=32, tok_out=tok_c,
                      logp_out=lp_c, logz_out=lz_c)
    # persistent kernel
    pf = PersistentLlama(m, s.kv_t, s.bt.table, 128, s.native_runner.status)
    pf.set_context(P + E, bs, (E,))
    tok_p = torch.zeros(M, dtype=torch.int32, device=dev)
    lp_p = torch.zeros(M, dtype=torch.float32, device=dev)
    lz_p = torch.zeros(M, dtype=torch.float32, device=dev)
    for _ in range(2):          # twice: the barrier counters must rearm themselves
        pf.run(ids2, pos2, locs2, rows, pref, bs, E, lm_rows=M, temperature=T, alpha=alpha, tokens_in=tokens_in,
               seed=seed, cycle_counter=counters, call_id=call_id, tok_out=tok_p, logp_out=lp_p, logz_out=lz_p)
    torch.cuda.synchronize()
    assert s.native_runner.check_status() == 0
    assert pf.sync[:3].tolist() == [0, 0, 0]
    # final hidden rows and the K/V rows of the last layer
    hb = pf.hb[:M].float()
    scale = chain_hb.abs().max().item()
    assert (hb - chain_hb).abs().max().item() < 2e-2 * scale
    assert (s.kv_t.k[li][locs2.long()].float() - chain_k).abs().max().item() < 2e-2 * chain_k.abs().max().item()
    assert (s.kv_t.v[li][locs2.long()].float() - chain_v).abs().max().item() < 2e-2 * chain_v.abs().max().item()
    # scored rows against the fp32 PyTorch model and against the chain's sampler
    sc = tokens_in >= 0
    ref_lp = torch.log_softmax(ref_logits / T, dim=-1)[torch.arange(M, device=dev)[sc], tokens_in[sc].long()]
    assert (lp_p[sc] - ref_lp).abs().max().item() < 0.05 * max(1.0, ref_lp.abs().max().item())
    assert (lp_p[sc] - lp_c[sc]).abs().max().item() < 2e-2
    assert (tok_p[sc] == tokens_in[sc]).all()
    # sampled rows: same noise, (almost) the same logits -> the same draws on nearly every row
    sm = ~sc
    same = tok_p[sm] == tok_c[sm]
    assert same.float().mean().item() >= 0.8
    assert (lp_p[sm][same] - lp_c[sm][same]).abs().max().item() < 2e-2
    assert (lz_p[sm] - lz_c[sm]).abs().max().item() < 2e-2
    assert (lz_p[sc] == 0).all()


def test_persistent_head_rows_and_no_sampling_pass():
    """Draft-head shape: two tokens per sequence, only the second is sampled; and a pass that only writes K/V."""
    from smcsd_b200.ops.native_forward import PersistentLlama
    bs, E, P = 8, 2, 64
    eng, s, cfg, rows, ids2, pos2, locs2, pref = _setup("narrow", bs, E, P)
    m, nm = s.target, s.native_runner.target
    dev = "cuda"
    nm.set_context(P + E, bs, (E,))
    nm.forward(ids2, pos2, locs2, rows, pref, bs, E)
    logits = nm.lm_head(bs, row_offset=1, row_step=2)[:bs].clone()
    counters = torch.tensor([9, 0, 0, 0], dtype=torch.int64, device=dev)
    pf = PersistentLlama(m, s.kv_t, s.bt.table, 128, s.native_runner.status)
    pf.set_context(P + E, bs, (E,))
    tok = torch.zeros(bs, dtype=torch.int32, device=dev)
    lp = torch.zeros(bs, dtype=torch.float32, device=dev)
    pf.run(ids2, pos2, locs2, rows, pref, bs, E, lm_rows=bs, lm_off=1, lm_step=2, temperature=0.7, alpha=1.0,
           seed=77, cycle_counter=counters, call_id=0, tok_out=tok, logp_out=lp)
    torch.cuda.synchronize()
    assert s.native_runner.check_status() == 0
    ref = torch.log_softmax(logits / 0.7, dim=-1)
    got_ref = ref[torch.arange(bs, device=dev), tok.long()]
    assert (lp - got_ref).abs().max().item() < 2e-2
    # K/V-only pass (the over-draft step of the legacy schedule): no lm_head phases, counters still rearm
    pf.run(ids2, pos2, locs2, rows, pref, bs, E)
    torch.cuda.synchronize()
    assert s.native_runner.check_status() == 0
    assert pf.sync[:3].tolist() == [0, 0, 0]


def test_engine_runs_on_the_persistent_path(monkeypatch):
    """The decode cycle with SMC_PERSISTENT=1: a dozen launches per cycle, clean status, conserved pages."""
    monkeypatch.setenv("SMC_PERSISTENT", "1")
    from smcsd_b200 import SMCEngine
    eng = SMCEngine(_cfg("wide"), _cfg("narrow"), n_particles=4, gamma=4, draft_temperature=0.7, target_temperature=0.7,
                    max_running_requests=2, context_length=1024, device="cuda", max_total_tokens=16384, random_seed=3,
                    backend="native", cycle_graph=True)
    r = eng._sched.native_runner
    assert r.pf_target is not None and r.pf_draft is not None
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 8192, (40,), generator=g).tolist() for _ in range(2)]
    outs = eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 40, "ignore_eos": True})
    assert [o["completion_tokens"] for o in outs] == [40, 40]
    assert r.check_status() == 0
    assert 0 < r.launches_per_cycle <= 40
    eng._sched.check_idle_invariants()
    eng._sched.alloc.check_conservation()
