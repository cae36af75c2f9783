"""Hybrid Gated-DeltaNet model on the sm_100a kernel chain (needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _hybrid_cfg(gdn_dim: int = 64):
    from smcsd_b200.models.config import ModelConfig
    lt = ["linear_attention", "linear_attention", "linear_attention", "full_attention"] * 2
    return ModelConfig(arch="hybrid_gdn", vocab_size=8192, hidden_size=512, n_layers=8, n_heads=4, n_kv_heads=2,
                       head_dim=128, ffn_size=1024, rope_theta=10000.0, max_position=2048, layer_types=lt,
                       gdn_n_k_heads=2, gdn_n_v_heads=4, gdn_head_k_dim=gdn_dim, gdn_head_v_dim=gdn_dim, gdn_conv_width=4,
                       partial_rotary=0.25, attn_output_gate=True, qk_norm=True, norm_plus_one=True, rms_eps=1e-6,
                       name="hybrid-test")


def _dense_draft():
    from smcsd_b200.models.config import ModelConfig
    return ModelConfig(arch="llama", vocab_size=8192, hidden_size=256, n_layers=2, n_heads=4, n_kv_heads=2,
                       head_dim=64, ffn_size=768, max_position=2048, tie_embeddings=True, name="dense-draft")


def test_native_hybrid_forward_matches_torch():
    from smcsd_b200 import SMCEngine
    from smcsd_b200.models.layers import ExtendBatch
    eng = SMCEngine(_hybrid_cfg(), _dense_draft(), n_particles=4, gamma=4, max_running_requests=2, context_length=512,
                    device="cuda", max_total_tokens=8192, backend="native", cycle_graph=False)
    s = eng._sched
    m, nm = s.target, s.native_runner.target
    dev = "cuda"
    bs, P = 4, 19
    g = torch.Generator(device=dev).manual_seed(0)
    rows = torch.arange(bs, dtype=torch.int32, device=dev)
    for b in range(bs):
        s.bt.table[b, :P + 8] = s.alloc.alloc(P + 8)
    ids = torch.randint(0, 8192, (bs * P,), generator=g, device=dev)
    pre = ExtendBatch(ids, torch.arange(P, device=dev).repeat(bs), s.bt.table[:bs, :P].reshape(-1), rows,
                      torch.zeros(bs, dtype=torch.int32, device=dev), extend_len=0, extend_lens=[P] * bs,
                      prefix_lens_host=[0] * bs)
    m.forward_torch(pre, s.kv_t, s.bt.table, s.state_t)
    conv0, temp0 = s.state_t.conv.clone(), s.state_t.temporal.clone()
    kk, vv = s.kv_t.k.clone(), s.kv_t.v.clone()
    for E in (5, 1, 2):
        ids2 = torch.randint(0, 8192, (bs * E,), generator=g, device=dev, dtype=torch.int32)
        pos2 = (torch.arange(E, device=dev) + P).repeat(bs).to(torch.int32)
        locs2 = s.bt.table[:bs, P:P + E].reshape(-1).contiguous()
        pref = torch.full((bs,), P, dtype=torch.int32, device=dev)
        ext = ExtendBatch(ids2.long(), pos2.long(), locs2, rows, pref, extend_len=E, prefix_lens_host=[P] * bs)
        ref = m.logits_torch(m.forward_torch(ext, s.kv_t, s.bt.table, s.state_t))
        conv_ref, temp_ref = s.state_t.conv.clone(), s.state_t.temporal.clone()
        # rewind the recurrent state and the cache, then run the kernel chain on the same inputs
        s.state_t.conv.copy_(conv0); s.state_t.temporal.copy_(temp0); s.kv_t.k.copy_(kk); s.kv_t.v.copy_(vv)
        nm.forward(ids2, pos2, locs2, rows, pref, bs, E)
        got = nm.lm_head(bs * E)[: bs * E].clone()
        torch.cuda.synchronize()
        assert s.native_runner.check_status() == 0
        scale = ref.abs().max().item()
        assert (got - ref).abs().max().item() < 0.08 * scale, E
        assert (s.state_t.temporal[:, :bs] - temp_ref[:, :bs]).abs().max().item() < 0.05 * max(1.0, temp_ref.abs().max().item())
        assert (s.state_t.conv[:, :bs] - conv_ref[:, :bs]).abs().max().item() < 0.05 * max(1.0, conv_ref.abs().max().item())
        s.state_t.conv.copy_(conv0); s.state_t.temporal.copy_(temp0); s.kv_t.k.copy_(kk); s.kv_t.v.copy_(vv)


def test_engine_hybrid_target_dense_draft_native():
    from smcsd_b200 import SMCEngine
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 8192, (30,), generator=g).tolist() for _ in range(3)]
    outs = {}
    for graph in (False, True):
        eng = SMCEngine(_hybrid_cfg(), _dense_draft(), n_particles=4, gamma=4, max_running_requests=2,
                        context_length=512, device="cuda", max_total_tokens=8192, backend="native", cycle_graph=graph,
                        draft_temperature=0.7, target_temperature=0.7, random_seed=2)
        o = eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 31, "ignore_eos": True})
        assert [x["completion_tokens"] for x in o] == [31] * 3
        assert eng._sched.native_runner.check_status() == 0
        eng._sched.check_idle_invariants()
        outs[graph] = o
    for a, b in zip(outs[False], outs[True]):
        assert a["output_ids"] == b["output_ids"]


def test_hybrid_state_follows_resampling_native():
    from smcsd_b200.config import EngineArgs
    from smcsd_b200.io_types import GenerateRequest, ParticleOutput, SamplingParams
    from smcsd_b200.models import build_model
    from smcsd_b200.runtime.scheduler import SMCScheduler
    cfg = _hybrid_cfg()
    model = build_model(cfg, torch.bfloat16, "cuda", seed=0)
    args = EngineArgs(model_path=cfg, draft_model_path=cfg, n_particles=4, gamma=3, max_running_requests=1,
                      context_length=512, device="cuda", max_total_tokens=8192, backend="native",
                      draft_temperature=0.8, target_temperature=0.8, resample_threshold=2.0).finalize()
    sched = SMCScheduler(args, target=model, draft=model)
    g = torch.Generator().manual_seed(3)
    sched.add_request(GenerateRequest("r", torch.randint(0, 8192, (17,), generator=g).tolist(),
                                      SamplingParams(max_new_tokens=25, ignore_eos=True)))
    outs = sched.run_until_idle()
    po = [o for o in outs if isinstance(o, ParticleOutput)][0]
    assert int(sched.state.counters[2]) > 0
    # the draft advances its state token by token, the target in gamma+1-token passes; bf16 noise only
    assert max(abs(w) for w in po.log_w_tilde) < 0.6, po.log_w_tilde
    assert sched.native_runner.check_status() == 0


@pytest.mark.parametrize("gdn_dim,lens", [(64, [37, 16, 5, 70]), (128, [137, 16, 5, 270])])
def test_native_hybrid_prefill_matches_torch_prefill(gdn_dim, lens):
    """Prompt pass of a hybrid target and a hybrid draft through the kernel chains (attention layers over 16-token
    blocks, Gated-DeltaNet layers walking each prompt once) vs the plain PyTorch forward: same cache contents and
    the same recurrent state, the draft's one token short under the deferred schedule.  With 128 x 128 heads and
    long prompts the Gated-DeltaNet layers take the chunk-parallel tcgen05 kernel."""
    from smcsd_b200.config import EngineArgs
    from smcsd_b200.models import build_model
    from smcsd_b200.runtime.scheduler import SMCScheduler
    from smcsd_b200.runtime.worker import PrefillItem
    cfg = _hybrid_cfg(gdn_dim)
    model = build_model(cfg, torch.bfloat16, "cuda", seed=0)
    args = EngineArgs(model_path=cfg, draft_model_path=cfg, n_particles=4, gamma=3, max_running_requests=4,
                      context_length=512, device="cuda", max_total_tokens=8192, backend="native",
                      cycle_graph=False).finalize()
    s = SMCScheduler(args, target=model, draft=model)
    r = s.native_runner
    if gdn_dim == 128:
        assert r.target.gdn_chunked
    g = torch.Generator().manual_seed(4)
    items = []
    for L in lens:
        row = s.bt.alloc_parent_row()
        s.bt.table[row, :L] = s.alloc.alloc(L)
        items.append(PrefillItem(row, torch.randint(0, 8192, (L,), generator=g).tolist()))
    rows = torch.tensor([it.row for it in items], device="cuda")
    for pool in (s.state_t, s.state_d):
        pool.clear_rows(rows)
    r.prefill(s.worker, items)
    torch.cuda.synchronize()
    assert r.check_status() == 0
    got = [x.clone() for x in (s.kv_t.k, s.kv_t.v, s.kv_d.k, s.state_t.temporal, s.state_t.conv, s.state_d.temporal,
                               s.state_d.conv)]
    s.kv_t.k.zero_(); s.kv_t.v.zero_(); s.kv_d.k.zero_()
    for pool in (s.state_t, s.state_d):
        pool.clear_rows(rows)
    native, s.worker.native = s.worker.native, None
    s.worker.prefill(items)
    s.worker.native = native
    ref = [s.kv_t.k, s.kv_t.v, s.kv_d.k, s.state_t.temporal, s.state_t.conv, s.state_d.temporal, s.state_d.conv]
    names = ["target K", "target V", "draft K", "target temporal", "target conv", "draft temporal", "draft conv"]
    for it, L in zip(items, lens):
        for a, b, name in zip(got[:3], ref[:3], names):
            # the stateful draft stops one token short, so its last prompt page is only written by the kernel path
            n = L - 1 if name.startswith("draft") else L
            pages = s.bt.table[it.row, :n].long()
            x = b[:, pages].float()
            err = (a[:, pages].float() - x).abs().max().item()
            assert err < 0.06 * max(1.0, x.abs().max().item()), (name, L, err)
    for a, b, name in zip(got[3:], ref[3:], names[3:]):
        x = b[:, rows].float()
        err = (a[:, rows].float() - x).abs().max().item()
        assert err < 0.05 * max(1.0, x.abs().max().item()), (name, err)
    # the two pools must differ: the draft's state stops one token before the target's
    assert (s.state_t.temporal[:, rows] - s.state_d.temporal[:, rows]).abs().max().item() > 0


@pytest.mark.parametrize("lens", [[150, 64, 1, 300], [512, 37]])
def test_gdn_chunked_prefill_kernel_matches_recurrence(lens):
    """Chunk-parallel delta rule on tcgen05 (64 tokens per step, dk = dv = 128) against the token-by-token recurrence in
    fp32 PyTorch and against the token-serial kernel: outputs after the gated RMSNorm and the final recurrent state,
    from a non-zero initial state, rows of different lengths (partial last chunks, a single-token row)."""
    import torch.nn.functional as F
    from smcsd_b200.models.hybrid_gdn import gdn_recurrent_step
    from smcsd_b200.ops import native as K
    torch.manual_seed(5)
    dev = "cuda"
    Hk, Hv, dk, dv, W, eps = 2, 4, 128, 128, 4, 1e-6
    key_dim, value_dim = Hk * dk, Hv * dv
    conv_dim = 2 * key_dim + value_dim
    ldp = conv_dim + value_dim + 2 * Hv
    ldp += (-ldp) % 8
    T, bs = sum(lens), len(lens)
    proj = torch.randn(T, ldp, device=dev)
    proj[:, conv_dim + value_dim:] *= 2.0                        # spread the gates
    conv_w = (torch.randn(conv_dim, W, device=dev) * 0.3).bfloat16()
    dt_bias = torch.ones(Hv, device=dev)
    A_log = torch.log(torch.empty(Hv, device=dev).uniform_(0.5, 8.0))
    gnorm_w = (1.0 + 0.1 * torch.randn(dv, device=dev)).bfloat16()
    rows = torch.tensor([3, 0, 2, 5][:bs], dtype=torch.int32, device=dev)
    conv0 = torch.randn(8, conv_dim, W - 1, device=dev) * 0.5
    temp0 = torch.randn(8, Hv, dk, dv, device=dev) * 0.2
    off = torch.tensor([sum(lens[:i]) for i in range(bs)], dtype=torch.int32, device=dev)
    ln = torch.tensor(lens, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    # fp32 reference
    ref_out = torch.zeros(T, value_dim, device=dev)
    ref_temp = temp0.clone()
    rep = Hv // Hk
    for b, n in enumerate(lens):
        t0, r = int(off[b]), int(rows[b])
        seq = torch.cat([conv0[r], proj[t0:t0 + n, :conv_dim].t()], dim=1)
        conv = F.silu(F.conv1d(seq.unsqueeze(0), conv_w.float().unsqueeze(1), groups=conv_dim).squeeze(0)).t()
        q = conv[:, :key_dim].reshape(n, Hk, dk)
        k = conv[:, key_dim:2 * key_dim].reshape(n, Hk, dk)
        v = conv[:, 2 * key_dim:].reshape(n, Hv, dv)
        q = (q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5).repeat_interleave(rep, dim=1)
        k = (k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(rep, dim=1)
        z = proj[t0:t0 + n, conv_dim:conv_dim + value_dim].view(n, Hv, dv)
        beta = torch.sigmoid(proj[t0:t0 + n, conv_dim + value_dim:conv_dim + value_dim + Hv])
        g = -A_log.exp() * F.softplus(proj[t0:t0 + n, conv_dim + value_dim + Hv:conv_dim + value_dim + 2 * Hv] + dt_bias)
        S = ref_temp[r].clone()
        for t in range(n):
            S, o = gdn_recurrent_step(S, q[t], k[t], v[t], g[t], beta[t])
            y = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)
            ref_out[t0 + t] = (y.bfloat16().float() * gnorm_w.float() * F.silu(z[t])).reshape(-1)
        ref_temp[r] = S

    got = {}
    for chunked in (False, True):
        conv_s, temp_s = conv0.clone(), temp0.clone()
        conv_out = torch.zeros(T, conv_dim, device=dev)
        out = torch.zeros(T, value_dim, device=dev, dtype=torch.bfloat16)
        K.gdn_step(proj, conv_s, temp_s, rows, conv_w, dt_bias, A_log, gnorm_w, conv_out, out, bs=bs, E=0, Hk=Hk, Hv=Hv,
                   dk=dk, dv=dv, W=W, eps=eps, tok_off=off, tok_len=ln, chunked=chunked, status=status,
                   max_len=max(lens) if chunked else 0)
        torch.cuda.synchronize()
        assert int(status) == 0
        got[chunked] = (out.float(), temp_s)
    o_scale, s_scale = ref_out.abs().max().item(), ref_temp.abs().max().item()
    for chunked in (False, True):
        o, s = got[chunked]
        tol = 2e-2 if chunked else 1e-2                           # bf16 operands in the chunked form, fp32 otherwise
        assert (o - ref_out).abs().max().item() < tol * o_scale, (chunked, (o - ref_out).abs().max().item(), o_scale)
        assert (s - ref_temp).abs().max().item() < tol * s_scale, (chunked, (s - ref_temp).abs().max().item(), s_scale)
    used = [int(r) for r in rows]
    untouched = [r for r in range(8) if r not in used]
    assert torch.equal(got[True][1][untouched], temp0[untouched])
