"""The sm_100a execution path end to end (needs a B200): kernel-chain forward vs the
PyTorch forward, graph vs eager cycles, engine invariants."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfgs():
    from smcsd_b200.models.config import ModelConfig
    tgt = ModelConfig(arch="llama", vocab_size=8192, hidden_size=512, n_layers=3, n_heads=8, n_kv_heads=2,
                      head_dim=128, ffn_size=1536, max_position=2048, name="t")
    drf = ModelConfig(arch="llama", vocab_size=8192, hidden_size=256, n_layers=2, n_heads=4, n_kv_heads=2,
                      head_dim=64, ffn_size=768, max_position=2048, tie_embeddings=True, name="d")
    return tgt, drf


def _engine(**kw):
    from smcsd_b200 import SMCEngine
    tgt, drf = _cfgs()
    base = dict(n_particles=4, gamma=4, draft_temperature=0.7, target_temperature=0.7, max_running_requests=4,
                context_length=1024, device="cuda", max_total_tokens=16384, random_seed=1)
    base.update(kw)
    return SMCEngine(tgt, drf, **base)


def _prompts(n, L=40, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 8192, (L,), generator=g).tolist() for _ in range(n)]


def test_native_forward_matches_torch_forward():
    """One verify-shaped pass (bs rows x 5 tokens over a cached prefix) through both executions."""
    from smcsd_b200.models.layers import ExtendBatch
    eng = _engine(backend="native", cycle_graph=False)
    s = eng._sched
    m, nm = s.target, s.native_runner.target
    bs, E, P = 4, 5, 37
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    # build a prefix with the torch path
    rows = torch.arange(bs, dtype=torch.int32, device=dev)
    for b in range(bs):
        s.bt.table[b, :P + E] = s.alloc.alloc(P + E)
    ids = torch.randint(0, 8192, (bs * P,), generator=g, device=dev)
    pos = torch.arange(P, device=dev).repeat(bs)
    locs = s.bt.table[:bs, :P].reshape(-1)
    pre = ExtendBatch(ids, pos, locs, rows, torch.zeros(bs, dtype=torch.int32, device=dev), extend_len=0,
                      extend_lens=[P] * bs, prefix_lens_host=[0] * bs)
    m.forward_torch(pre, s.kv_t, s.bt.table)
    ids2 = torch.randint(0, 8192, (bs * E,), generator=g, device=dev, dtype=torch.int32)
    pos2 = (torch.arange(E, device=dev) + P).repeat(bs).to(torch.int32)
    locs2 = s.bt.table[:bs, P:P + E].reshape(-1).contiguous()
    pref = torch.full((bs,), P, dtype=torch.int32, device=dev)
    ext = ExtendBatch(ids2.long(), pos2.long(), locs2, rows, pref, extend_len=E, prefix_lens_host=[P] * bs)
    hid = m.forward_torch(ext, s.kv_t, s.bt.table)
    ref = m.logits_torch(hid)
    nm.forward(ids2, pos2, locs2, rows, pref, bs, E)
    got = nm.lm_head(bs * E)[: bs * E].clone()
    torch.cuda.synchronize()
    assert s.native_runner.check_status() == 0
    scale = ref.abs().max().item()
    err = (got - ref).abs().max().item()
    assert err < 0.06 * scale, (err, scale)
    # top-1 agreement on nearly every row
    agree = (got.argmax(-1) == ref.argmax(-1)).float().mean().item()
    assert agree >= 0.9


def test_engine_native_end_to_end_and_graph_equals_eager():
    outs = {}
    for graph in (False, True):
        eng = _engine(backend="native", cycle_graph=graph)
        o = eng.generate(input_ids=_prompts(3), sampling_params={"max_new_tokens": 40, "ignore_eos": True})
        assert [x["completion_tokens"] for x in o] == [40, 40, 40]
        assert eng._sched.native_runner.check_status() == 0
        eng._sched.check_idle_invariants()
        eng._sched.alloc.check_conservation()
        outs[graph] = o
    for a, b in zip(outs[False], outs[True]):
        assert a["output_ids"] == b["output_ids"]
        assert abs(a["smc_log_Z_hat"] - b["smc_log_Z_hat"]) < 1e-6


def test_engine_native_eos_and_queueing():
    eng = _engine(backend="native", max_running_requests=2)
    o = eng.generate(input_ids=_prompts(5, L=20), sampling_params={"max_new_tokens": 30, "stop_token_ids": list(range(64))})
    assert len(o) == 5
    for x in o:
        assert 1 <= x["completion_tokens"] <= 30
        if x["finish_reason"]["type"] == "stop":
            assert x["output_ids"][-1] < 64
    eng._sched.check_idle_invariants()


def test_weights_track_target_over_draft():
    """With draft == target (same weights, same temperature) every log-weight increment is ~0:
    the verify pass re-derives the probabilities the draft sampled from."""
    from smcsd_b200.config import EngineArgs
    from smcsd_b200.io_types import GenerateRequest, ParticleOutput, SamplingParams
    from smcsd_b200.models import build_model
    from smcsd_b200.runtime.scheduler import SMCScheduler
    tgt, _ = _cfgs()
    model = build_model(tgt, torch.bfloat16, "cuda", seed=0)
    args = EngineArgs(model_path=tgt, draft_model_path=tgt, n_particles=4, gamma=4, draft_temperature=0.7,
                      target_temperature=0.7, max_running_requests=2, context_length=512, device="cuda",
                      max_total_tokens=8192, backend="native", resample_threshold=0.0).finalize()
    sched = SMCScheduler(args, target=model, draft=model)
    sched.add_request(GenerateRequest("r", _prompts(1)[0], SamplingParams(max_new_tokens=30, ignore_eos=True)))
    outs = sched.run_until_idle()
    po = [o for o in outs if isinstance(o, ParticleOutput)][0]
    assert max(abs(w) for w in po.log_w_tilde) < 0.35, po.log_w_tilde
    assert sched.native_runner.check_status() == 0


@pytest.mark.parametrize("capacity", [None, 64])
def test_native_prefill_matches_torch_prefill(capacity):
    """Prompt pass through the kernel chains (16-token blocks as batch rows) vs the plain PyTorch forward:
    same cache contents, same last-token logits.  With a small token capacity the prompts run in several passes."""
    from smcsd_b200.runtime.worker import PrefillItem
    eng = _engine(backend="native", cycle_graph=False)
    s = eng._sched
    r = s.native_runner
    if capacity:
        r.PREFILL_MAX_TOKENS = capacity
    lens = [37, 16, 5, 70]
    g = torch.Generator().manual_seed(4)
    items = []
    for L in lens:
        row = s.bt.alloc_parent_row()
        s.bt.table[row, :L] = s.alloc.alloc(L)
        items.append(PrefillItem(row, torch.randint(0, 8192, (L,), generator=g).tolist()))
    x0_native = r.prefill(s.worker, items)
    torch.cuda.synchronize()
    assert r.check_status() == 0
    kt, vt, kd = s.kv_t.k.clone(), s.kv_t.v.clone(), s.kv_d.k.clone()
    s.kv_t.k.zero_(); s.kv_t.v.zero_(); s.kv_d.k.zero_()
    native, s.worker.native = s.worker.native, None
    s.worker.gen_prefill.manual_seed(int(s.args.random_seed) * 7919 + 17)
    x0_torch = s.worker.prefill(items)
    s.worker.native = native
    for it, L in zip(items, lens):
        pages = s.bt.table[it.row, :L].long()
        for a, b in ((kt, s.kv_t.k), (vt, s.kv_t.v), (kd, s.kv_d.k)):
            ref = b[:, pages].float()
            assert (a[:, pages].float() - ref).abs().max().item() < 0.06 * max(1.0, ref.abs().max().item())
    assert x0_native.shape == x0_torch.shape


def test_graph_equals_eager_across_attention_split_plans():
    """A request whose context grows through several attention split plans (each has its own captured graph)
    produces the same tokens as the eager kernel chain."""
    from smcsd_b200.ops import native as K
    outs, keys = {}, None
    for graph in (False, True):
        eng = _engine(backend="native", cycle_graph=graph, max_running_requests=1, context_length=2048,
                      max_total_tokens=32768)
        o = eng.generate(input_ids=_prompts(1, L=180, seed=5), sampling_params={"max_new_tokens": 700, "ignore_eos": True})
        assert o[0]["completion_tokens"] == 700
        assert eng._sched.native_runner.check_status() == 0
        eng._sched.check_idle_invariants()
        outs[graph] = o[0]
        if graph:
            keys = set(eng._sched.native_runner.graphs.keys())
    assert outs[False]["output_ids"] == outs[True]["output_ids"]
    assert len(keys) >= 2, keys                      # the split plan changed at least once along the way
    assert K.attn_kv_splits(1500, 4, 2, 1, 4, 128) >= K.attn_kv_splits(100, 4, 2, 1, 4, 128)


def test_overlapped_loop_equals_sequential_loop():
    """Post-processing cycle t-1 after enqueuing cycle t only delays finish detection: same outputs."""
    outs = {}
    for overlap in (False, True):
        eng = _engine(backend="native", enable_overlap=overlap)
        outs[overlap] = eng.generate(input_ids=_prompts(3, L=24, seed=9),
                                     sampling_params={"max_new_tokens": 33, "stop_token_ids": list(range(16))})
        eng._sched.check_idle_invariants()
    for a, b in zip(outs[False], outs[True]):
        assert a["output_ids"] == b["output_ids"] and a["finish_reason"] == b["finish_reason"]


def test_abort_mid_decode_releases_pages_and_slots():
    from smcsd_b200.io_types import GenerateRequest, RequestOutput, SamplingParams
    eng = _engine(backend="native", max_running_requests=2)
    s = eng._sched
    for i, p in enumerate(_prompts(2, L=30, seed=11)):
        s.add_request(GenerateRequest(f"r{i}", p, SamplingParams(max_new_tokens=200, ignore_eos=True)))
    for _ in range(6):
        s.step()
    assert len(s.running) == 2
    s.abort("r0")
    outs = s.run_until_idle()
    done = {o.rid: o for o in outs if isinstance(o, RequestOutput)}
    assert done["r0"].aborted and not done["r1"].aborted and len(done["r1"].output_ids) == 200
    s.check_idle_invariants()
    s.alloc.check_conservation()
    assert s.native_runner.check_status() == 0


def test_staggered_arrivals_with_changing_batch_sizes():
    """Requests of different lengths join and leave while others decode: every batch size gets its own captured
    graph, finished groups free their slots for the queue, and nothing leaks."""
    from smcsd_b200.io_types import GenerateRequest, RequestOutput, SamplingParams
    eng = _engine(backend="native", max_running_requests=3)
    s = eng._sched
    g = torch.Generator().manual_seed(21)
    want = {}
    done = {}
    arrivals = {0: 2, 3: 1, 5: 2, 11: 1, 12: 3}          # step -> number of new requests
    k = 0
    for step in range(400):
        for _ in range(arrivals.get(step, 0)):
            L = int(torch.randint(8, 90, (1,), generator=g))
            n = int(torch.randint(5, 70, (1,), generator=g))
            rid = f"r{k}"
            k += 1
            want[rid] = n
            s.add_request(GenerateRequest(rid, torch.randint(64, 8192, (L,), generator=g).tolist(),
                                          SamplingParams(max_new_tokens=n, stop_token_ids=list(range(8)))))
        for o in s.step():
            if isinstance(o, RequestOutput) and o.finished:
                done[o.rid] = o
        if step > 12 and not s.has_work():
            break
    assert set(done) == set(want)
    for rid, o in done.items():
        assert not o.aborted and 1 <= len(o.output_ids) <= want[rid]
        if len(o.output_ids) < want[rid]:
            assert o.finish_reason["type"] == "stop" and o.output_ids[-1] < 8
    assert len(s.native_runner.graphs) >= 2
    s.check_idle_invariants()
    s.alloc.check_conservation()
    assert s.native_runner.check_status() == 0


def _gen(eng, n=2, new=45):
    o = eng.generate(input_ids=_prompts(n, L=30, seed=21), sampling_params={"max_new_tokens": new, "ignore_eos": True})
    assert eng._sched.native_runner.check_status() == 0
    eng._sched.check_idle_invariants()
    eng._sched.alloc.check_conservation()
    return o


def test_write_back_switch_and_draft_phase_graph_equal_the_eager_chain():
    """SMC_FUSED_WRITE_BACK=0 routes the state transition to the PyTorch reference, and the draft-only graph replays
    the same draft launches: both must reproduce the eager kernel chain token for token."""
    base = _gen(_engine(backend="native", cycle_graph=False))
    wb = _engine(backend="native", cycle_graph=False, fused_write_back=False)
    assert wb._sched.native_runner.switched_off and not wb._sched.native_runner.can_run_cycle(wb._sched.state)
    out_wb = _gen(wb)
    dpg = _engine(backend="native", cycle_graph=False, draft_phase_graph=True)
    out_dpg = _gen(dpg)
    assert len(dpg._sched.native_runner.draft_graphs) >= 1
    for a, b, c in zip(base, out_wb, out_dpg):
        assert a["output_ids"] == b["output_ids"] == c["output_ids"]
        assert abs(a["smc_log_Z_hat"] - b["smc_log_Z_hat"]) < 1e-5
        assert abs(a["smc_log_Z_hat"] - c["smc_log_Z_hat"]) < 1e-6


def test_sampling_and_verify_switches_run_the_pytorch_steps():
    """SMC_FUSED_SAMPLING=0 / SMC_FAST_VERIFY=0: the cycle graph is dropped with a warning and the PyTorch sampler /
    PyTorch verify forward take over; outputs stay well-formed and the importance weights stay finite."""
    import math
    for kw in (dict(fused_sampling=False), dict(fast_verify=False)):
        eng = _engine(backend="native", **kw)
        r = eng._sched.native_runner
        assert r.switched_off and not r.use_graph
        o = _gen(eng)
        assert [x["completion_tokens"] for x in o] == [45, 45]
        assert all(math.isfinite(x["smc_log_Z_hat"]) for x in o)


def test_attention_split_cap_is_honoured():
    eng = _engine(backend="native", attention_num_kv_splits=1, max_running_requests=1, context_length=2048,
                  max_total_tokens=32768)
    nm = eng._sched.native_runner.target
    nm.set_context(1800, 4, (5,))
    assert nm._ks(4, 5) == 1
    eng2 = _engine(backend="native", max_running_requests=1, context_length=2048, max_total_tokens=32768)
    nm2 = eng2._sched.native_runner.target
    nm2.set_context(1800, 4, (5,))
    assert nm2._ks(4, 5) >= 2


def test_score_tokens_rpc_native_matches_pytorch():
    """The diagnostic scoring RPC (prompt pass + one verify-shaped pass + fused scorer) against the PyTorch model."""
    prompt, cont = _prompts(1, L=50, seed=12)[0], _prompts(1, L=10, seed=13)[0]
    a = _engine(backend="native")._sched.score_tokens(prompt, cont, 0.7)
    b = _engine(backend="torch")._sched.score_tokens(prompt, cont, 0.7)
    assert len(a) == len(b) == 9
    assert max(abs(x - y) for x, y in zip(a, b)) < 0.05, (a, b)


@pytest.mark.parametrize("tc", [False, True])
def test_shared_prefix_attention_in_the_decode_cycle(monkeypatch, tc):
    """The shared-prefix passes forced on for short prompts (draft steps: 4 particles per group pass, verify: 2; with
    ``tc`` the group pass runs on the tcgen05 kernel, whole groups at once).
    With draft == target every log-weight increment must stay ~0, which it only does if the single-token, two-token
    and verify attention paths all compute the same softmax; and the graph replays match the eager launches."""
    from smcsd_b200.config import EngineArgs
    from smcsd_b200.io_types import GenerateRequest, ParticleOutput, SamplingParams
    from smcsd_b200.models import build_model
    from smcsd_b200.runtime.scheduler import SMCScheduler
    monkeypatch.setenv("SMC_CASCADE_MIN_PROMPT", "32")
    monkeypatch.setenv("SMC_CASCADE_VERIFY", "1")
    monkeypatch.setenv("SMC_ATTN_TC", "2" if tc else "0")
    tgt, _ = _cfgs()
    model = build_model(tgt, torch.bfloat16, "cuda", seed=0)
    outs = {}
    for graph in (False, True):
        args = EngineArgs(model_path=tgt, draft_model_path=tgt, n_particles=4, gamma=4, draft_temperature=0.7,
                          target_temperature=0.7, max_running_requests=2, context_length=512, device="cuda",
                          max_total_tokens=8192, backend="native", resample_threshold=0.0, cycle_graph=graph).finalize()
        sched = SMCScheduler(args, target=model, draft=model)
        sched.add_request(GenerateRequest("r", _prompts(1, L=70)[0], SamplingParams(max_new_tokens=30, ignore_eos=True)))
        o = sched.run_until_idle()
        assert sched.native_runner.target._cascade and sched.native_runner.draft._cascade     # the plans were on
        assert all(pl["tc"] == tc for pl in sched.native_runner.target._cascade.values())
        po = [x for x in o if isinstance(x, ParticleOutput)][0]
        assert max(abs(w) for w in po.log_w_tilde) < 0.35, po.log_w_tilde
        assert sched.native_runner.check_status() == 0
        outs[graph] = po.particle_output_ids
    assert outs[False] == outs[True]


def test_fp8_quantised_engine(monkeypatch):
    """quantization='fp8': the kernel chain serves e4m3 weights with per-row scales and per-token quantised activations.
    (1) One forward against the PyTorch model whose projection weights were replaced by the dequantised e4m3 values:
    only the activation quantisation separates the two.  (2) A decode run: graph replays equal the eager launches and
    the importance weights stay small when draft == target (both quantised the same way)."""
    from smcsd_b200.config import EngineArgs
    from smcsd_b200.io_types import GenerateRequest, ParticleOutput, SamplingParams
    from smcsd_b200.models import build_model
    from smcsd_b200.models.layers import ExtendBatch
    from smcsd_b200.ops import native as K
    from smcsd_b200.runtime.scheduler import SMCScheduler
    tgt, _ = _cfgs()
    model = build_model(tgt, torch.bfloat16, "cuda", seed=0)
    outs = {}
    for graph in (False, True):
        args = EngineArgs(model_path=tgt, draft_model_path=tgt, n_particles=4, gamma=4, draft_temperature=0.7,
                          target_temperature=0.7, max_running_requests=2, context_length=512, device="cuda",
                          max_total_tokens=8192, backend="native", resample_threshold=0.0, cycle_graph=graph,
                          quantization="fp8").finalize()
        sched = SMCScheduler(args, target=model, draft=model)
        nm = sched.native_runner.target
        assert nm.quant == "fp8" and not nm.fold
        if not graph:
            # (1) logits of a 4 x 5 token forward
            dev = "cuda"
            bs, E = 4, 5
            g = torch.Generator(device=dev).manual_seed(1)
            rows = torch.arange(bs, dtype=torch.int32, device=dev)
            for b in range(bs):
                sched.bt.table[b, :E + 3] = sched.alloc.alloc(E + 3)
            ids = torch.randint(0, 8192, (bs * E,), generator=g, device=dev, dtype=torch.int32)
            pos = torch.arange(E, device=dev).repeat(bs).to(torch.int32)
            locs = sched.bt.table[:bs, :E].reshape(-1).contiguous()
            pref = torch.zeros(bs, dtype=torch.int32, device=dev)
            nm.forward(ids, pos, locs, rows, pref, bs, E)
            got = nm.lm_head(bs * E)[: bs * E].clone()
            torch.cuda.synchronize()
            saved = [(L.wqkv, L.wo, L.wgu, L.wdown) for L in model.layers]
            for L, w8 in zip(model.layers, model._w8):
                for name in ("wqkv", "wo", "wgu", "wdown"):
                    q, s = w8[name]
                    setattr(L, name, (q.view(torch.float8_e4m3fn).float() * s[:, None]).bfloat16())
            ext = ExtendBatch(ids.long(), pos.long(), locs, rows, pref, extend_len=E, prefix_lens_host=[0] * bs)
            ref = model.logits_torch(model.forward_torch(ext, sched.kv_t, sched.bt.table))
            for L, ws in zip(model.layers, saved):
                L.wqkv, L.wo, L.wgu, L.wdown = ws
            scale = ref.abs().max().item()
            assert (got - ref).abs().max().item() < 0.08 * scale
            for b in range(bs):
                sched.alloc.free(sched.bt.table[b, :E + 3].clone())
                sched.bt.table[b].zero_()
        sched.add_request(GenerateRequest("r", _prompts(1, L=40)[0], SamplingParams(max_new_tokens=30, ignore_eos=True)))
        o = sched.run_until_idle()
        po = [x for x in o if isinstance(x, ParticleOutput)][0]
        assert max(abs(w) for w in po.log_w_tilde) < 0.35, po.log_w_tilde
        assert sched.native_runner.check_status() == 0
        outs[graph] = po.particle_output_ids
    assert outs[False] == outs[True]


def test_capture_warm_up_restores_token_histories_and_group_flags():
    """The warm-up cycle that precedes a graph capture runs on live state and is then rolled back; the roll-back list
    must cover everything a cycle (including a resampling step) writes: token histories and group flags too."""
    eng = _engine(backend="native")
    sched = eng._sched
    r, st = sched.native_runner, sched.state
    listed = r._mutable(st)
    for name in ("all_token_ids", "seq_lens", "log_weights", "counters"):
        assert any(t is getattr(st, name) for t in listed), name
    assert any(t is st.bt.table for t in listed)
    if getattr(st, "group_active", None) is not None:
        assert any(t is st.group_active for t in listed)
    # a run that captures a new graph key while a request is in flight (batch shrinks from two groups to one) yields
    # the same tokens as the same run without graphs
    outs = {}
    for graph in (False, True):
        e = _engine(backend="native", cycle_graph=graph, max_running_requests=2, random_seed=3)
        o = e.generate(input_ids=[p for p in _prompts(2, L=30, seed=9)],
                       sampling_params=[{"max_new_tokens": 12, "ignore_eos": True}, {"max_new_tokens": 40, "ignore_eos": True}])
        outs[graph] = [x["smc_particle_output_ids"] for x in o]
        assert e._sched.native_runner.check_status() == 0
    assert outs[False] == outs[True]


def test_e4m3_kv_cache_engine():
    """kv_cache_dtype='fp8_e4m3': both KV pools hold e4m3 rows with per-(token, head) scales.  Prompt pass (rope kernel +
    quantising store), draft steps and verify passes all read and write that layout; graph replays equal the eager
    launches, and with draft == target the importance weights stay small (both see the same quantised history)."""
    from smcsd_b200.config import EngineArgs
    from smcsd_b200.io_types import GenerateRequest, ParticleOutput, SamplingParams
    from smcsd_b200.models import build_model
    from smcsd_b200.runtime.scheduler import SMCScheduler
    tgt, _ = _cfgs()
    model = build_model(tgt, torch.bfloat16, "cuda", seed=0)
    outs = {}
    for graph in (False, True):
        args = EngineArgs(model_path=tgt, draft_model_path=tgt, n_particles=4, gamma=4, draft_temperature=0.7,
                          target_temperature=0.7, max_running_requests=2, context_length=512, device="cuda",
                          max_total_tokens=8192, backend="native", resample_threshold=0.5, cycle_graph=graph,
                          kv_cache_dtype="fp8_e4m3").finalize()
        sched = SMCScheduler(args, target=model, draft=model)
        assert sched.kv_t.k.dtype == torch.uint8 and sched.kv_t.spec.cell_bytes < 0.6 * 2 * 3 * 2 * 128 * 2
        sched.add_request(GenerateRequest("r", _prompts(1, L=70)[0], SamplingParams(max_new_tokens=40, ignore_eos=True)))
        o = sched.run_until_idle()
        po = [x for x in o if isinstance(x, ParticleOutput)][0]
        assert max(abs(w) for w in po.log_w_tilde) < 0.5, po.log_w_tilde
        assert sched.native_runner.check_status() == 0
        sched.check_idle_invariants()
        outs[graph] = po.particle_output_ids
    assert outs[False] == outs[True]
