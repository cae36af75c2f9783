"""sm_100a kernels against plain-PyTorch fp32 references (needs a B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _K():
    from smcsd_b200.ops import native as K
    K.lib()
    return K


def _status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


# ------------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("N,Kd,M,splits", [
    (3072, 2048, 8, 0), (6144, 4096, 72, 0), (2048, 8192, 8, 0), (4096, 14336, 72, 0), (512, 256, 16, 1),
    (1024, 688, 5, 2), (2048, 2048, 200, 1), (2048, 1024, 300, 3), (128256, 2048, 8, 1), (4096, 4096, 33, 0),
    (300, 512, 100, 1),
])
def test_gemm_partials(N, Kd, M, splits):
    K = _K()
    torch.manual_seed(0)
    W = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    X = torch.randn(M, Kd, device="cuda").bfloat16()
    s = splits or K.gemm_default_splits(N, Kd, M)
    out = torch.full((s, M, N), float("nan"), device="cuda")
    st = _status()
    K.gemm_skinny(W, X, out, M=M, splits=s, epi=K.EPI_PARTIAL_F32, status=st)
    torch.cuda.synchronize()
    assert int(st) == 0
    ref = X.float() @ W.float().t()
    got = out.sum(0)
    err = (got - ref).abs().max().item()
    # bf16 products are exact in fp32, so only the accumulation order differs from the fp32 reference
    assert err < 1e-3 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("N,Kd,M,splits", [
    (3072, 2048, 8, 8), (2048, 8192, 8, 8), (6144, 4096, 72, 4), (4096, 14336, 72, 4), (2048, 2048, 8, 1),
    (1024, 512, 40, 2), (128256, 2048, 8, 1), (300, 1024, 9, 4), (2048, 2048, 200, 2), (4096, 4096, 72, 0),
    (6144, 4096, 72, 3), (3072, 2048, 8, 6), (3072, 2048, 16, 5), (2048, 4096, 33, 7), (4096, 14336, 600, 0),
])
def test_gemm_cluster_splitk(N, Kd, M, splits):
    """Split-K reduced on chip through distributed shared memory: plain store and residual accumulate."""
    K = _K()
    torch.manual_seed(11)
    W = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    X = torch.randn(M, Kd, device="cuda").bfloat16()
    s = splits or K.gemm_cluster_splits(N, Kd, M)
    ref = X.float() @ W.float().t()
    st = _status()
    out = torch.full((M, N), float("nan"), device="cuda")
    K.gemm_skinny(W, X, out, M=M, splits=s, epi=K.EPI_STORE_F32, ldo=N, status=st)
    h0 = torch.randn(M, N, device="cuda")
    h = h0.clone()
    K.gemm_skinny(W, X, h, M=M, splits=s, epi=K.EPI_RESID_F32, ldo=N, status=st)
    out2 = torch.full((M, N), float("nan"), device="cuda")
    K.gemm_skinny(W, X, out2, M=M, splits=s, epi=K.EPI_STORE_F32, ldo=N, status=st, pdl=True)
    torch.cuda.synchronize()
    assert int(st) == 0
    tol = 1e-3 * max(1.0, ref.abs().max().item())
    assert (out - ref).abs().max().item() < tol
    assert (h - h0 - ref).abs().max().item() < tol
    assert torch.equal(out, out2), "the cluster reduction must be bit-deterministic"


@pytest.mark.parametrize("N,Kd,M", [(4096, 4096, 1152), (6144, 4096, 513), (1024, 512, 400)])
def test_gemm_large_batches(N, Kd, M):
    """Prompt-pass sized batches (several token tiles per weight slab): bf16 store, fp32 store and residual
    accumulate, against fp32 PyTorch."""
    K = _K()
    torch.manual_seed(17)
    W = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    X = torch.randn(M, Kd, device="cuda").bfloat16()
    ref = X.float() @ W.float().t()
    st = _status()
    ob = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    K.gemm_skinny(W, X, ob, M=M, splits=1, epi=K.EPI_BF16, status=st)
    of = torch.full((M, N), float("nan"), device="cuda")
    K.gemm_skinny(W, X, of, M=M, splits=1, epi=K.EPI_STORE_F32, ldo=N, status=st)
    h0 = torch.randn(M, N, device="cuda")
    h = h0.clone()
    K.gemm_skinny(W, X, h, M=M, splits=1, epi=K.EPI_RESID_F32, ldo=N, status=st, pdl=True)
    torch.cuda.synchronize()
    assert int(st) == 0
    tol = 1e-3 * max(1.0, ref.abs().max().item())
    assert (of - ref).abs().max().item() < tol
    assert (h - h0 - ref).abs().max().item() < tol
    assert (ob.float() - ref).abs().max().item() < 6e-3 * max(1.0, ref.abs().max().item())


def test_gemm_bf16_and_strided_rows():
    K = _K()
    torch.manual_seed(1)
    N, Kd, M = 1024, 512, 8
    W = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    X2 = torch.randn(2 * M, Kd, device="cuda").bfloat16()
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    st = _status()
    # every second row starting at row 1 (the draft head reads only its x0 rows this way)
    K.gemm_skinny(W, X2[1:], out, M=M, splits=1, epi=K.EPI_BF16, ldx=2 * Kd, status=st)
    torch.cuda.synchronize()
    ref = X2[1::2].float() @ W.float().t()
    assert int(st) == 0
    assert (out.float() - ref).abs().max().item() < 6e-3 * ref.abs().max().item()      # one bf16 rounding of the output


@pytest.mark.parametrize("ffn,d,M", [(8192, 2048, 8), (14336, 4096, 72), (1024, 256, 40), (14336, 4096, 700)])
def test_gemm_swiglu_epilogue(ffn, d, M):
    K = _K()
    from smcsd_b200.models.llama import interleave_gate_up
    torch.manual_seed(2)
    Wg = (torch.randn(ffn, d, device="cuda") * 0.05).bfloat16()
    Wu = (torch.randn(ffn, d, device="cuda") * 0.05).bfloat16()
    Wgu = interleave_gate_up(Wg, Wu, 64)
    X = torch.randn(M, d, device="cuda").bfloat16()
    act = torch.zeros(M, ffn, device="cuda", dtype=torch.bfloat16)
    st = _status()
    K.gemm_skinny(Wgu, X, act, M=M, splits=1, epi=K.EPI_SWIGLU_BF16, ldo=ffn, status=st)
    torch.cuda.synchronize()
    g, u = X.float() @ Wg.float().t(), X.float() @ Wu.float().t()
    ref = torch.nn.functional.silu(g) * u
    assert int(st) == 0
    assert (act.float() - ref).abs().max().item() < 6e-3 * max(1.0, ref.abs().max().item())
    # the unfused path (partials + separate activation kernel) agrees
    s = 2
    part = torch.zeros(s, M, 2 * ffn, device="cuda")
    K.gemm_skinny(Wgu, X, part, M=M, splits=s, epi=K.EPI_PARTIAL_F32, status=st)
    act2 = torch.zeros_like(act)
    K.swiglu_partials(part, s, M * 2 * ffn, act2, M=M, ffn=ffn, blk=64)
    torch.cuda.synchronize()
    assert (act2.float() - ref).abs().max().item() < 6e-3 * max(1.0, ref.abs().max().item())
    # split-K reduced inside a cluster before the activation
    for s in (2, 4, 3):
        act3 = torch.zeros_like(act)
        K.gemm_skinny(Wgu, X, act3, M=M, splits=s, epi=K.EPI_SWIGLU_BF16, ldo=ffn, status=st, pdl=True)
        torch.cuda.synchronize()
        assert int(st) == 0
        assert (act3.float() - ref).abs().max().item() < 6e-3 * max(1.0, ref.abs().max().item()), s


# ------------------------------------------------------------------------------- norm / rope
def test_add_rmsnorm_and_embed():
    K = _K()
    from smcsd_b200.models.layers import rmsnorm
    torch.manual_seed(3)
    M, d, S = 9, 2048, 3
    h = torch.randn(M, d, device="cuda")
    part = torch.randn(S, M, d, device="cuda")
    w = torch.randn(d, device="cuda").bfloat16()
    xn = torch.zeros(M, d, device="cuda", dtype=torch.bfloat16)
    h_ref = h + part.sum(0)
    K.add_rmsnorm(h, w, xn, M=M, d=d, eps=1e-5, partials=part, splits=S, split_stride=M * d)
    torch.cuda.synchronize()
    assert torch.allclose(h, h_ref, atol=1e-5)
    ref = rmsnorm(h_ref, w.float(), 1e-5)
    assert (xn.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    emb = torch.randn(100, d, device="cuda").bfloat16()
    ids = torch.randint(0, 100, (M,), device="cuda", dtype=torch.int32)
    K.add_rmsnorm(h, w, xn, M=M, d=d, eps=1e-5, ids=ids, embed=emb, plus_one=True)
    torch.cuda.synchronize()
    assert torch.equal(h, emb[ids.long()].float())
    ref = rmsnorm(h, w.float(), 1e-5, plus_one=True)
    assert (xn.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("Hq,Hkv,D,rd", [(32, 8, 64, 64), (32, 8, 128, 128), (4, 2, 256, 64)])
def test_rope_kv_write(Hq, Hkv, D, rd):
    K = _K()
    from smcsd_b200.models.layers import apply_rope, rope_table
    torch.manual_seed(4)
    M, S, pages = 7, 2, 50
    n = (Hq + 2 * Hkv) * D
    part = torch.randn(S, M, n, device="cuda")
    pos = torch.randint(0, 500, (M,), device="cuda", dtype=torch.int32)
    locs = torch.randperm(pages, device="cuda")[:M].to(torch.int32) + 1
    table = rope_table(rd, 10000.0, None, 512, "cuda")
    q = torch.zeros(M, Hq * D, device="cuda", dtype=torch.bfloat16)
    kp = torch.zeros(pages + 1, Hkv * D, device="cuda", dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    st = _status()
    K.rope_kv_write(part, S, M * n, pos, locs, table, q, kp, vp, M=M, Hq=Hq, Hkv=Hkv, D=D, status=st)
    torch.cuda.synchronize()
    full = part.sum(0)
    qr = apply_rope(full[:, :Hq * D].view(M, Hq, D), pos, table).reshape(M, -1)
    kr = apply_rope(full[:, Hq * D:(Hq + Hkv) * D].view(M, Hkv, D), pos, table).reshape(M, -1)
    vr = full[:, (Hq + Hkv) * D:]
    assert int(st) == 0
    assert (q.float() - qr).abs().max().item() < 3e-2
    assert (kp[locs.long()].float() - kr).abs().max().item() < 3e-2
    assert (vp[locs.long()].float() - vr).abs().max().item() < 3e-2


# ------------------------------------------------------------------------------- sampling
def _sample(K, logits, T, alpha, tokens_in, seed=7, counter=0, call_id=0, softcap=0.0):
    rows, V = logits.shape
    nch = 32
    scratch = torch.empty(K.sample_scratch_bytes(rows, nch), dtype=torch.uint8, device="cuda")
    tok = torch.zeros(rows, dtype=torch.int32, device="cuda")
    lp = torch.zeros(rows, device="cuda")
    lz = torch.zeros(rows, device="cuda")
    ctr = torch.tensor([counter], dtype=torch.int64, device="cuda")
    K.sample_or_score(logits, rows=rows, V=V, splits=1, split_stride=0, row_stride=logits.stride(0), temperature=T,
                      alpha=alpha, softcap=softcap, tokens_in=tokens_in, seed=seed, cycle_counter=ctr, call_id=call_id,
                      scratch=scratch, nchunks=nch, tok_out=tok, logp_out=lp, logz_out=lz)
    torch.cuda.synchronize()
    return tok, lp, lz


def test_score_mode_matches_torch():
    K = _K()
    from smcsd_b200.smc.math import chosen_logprob
    torch.manual_seed(6)
    logits = torch.randn(72, 128256, device="cuda") * 3
    toks = torch.randint(0, 128256, (72,), device="cuda", dtype=torch.int32)
    _, lp, _ = _sample(K, logits, 0.7, 1.0, toks)
    ref = chosen_logprob(logits, toks.long(), 0.7)
    assert (lp - ref).abs().max().item() < 2e-3


def test_sample_mode_logp_logz_and_determinism():
    K = _K()
    torch.manual_seed(7)
    logits = torch.randn(8, 128256, device="cuda") * 2
    alpha, T = 1.7, 0.7
    tok, lp, lz = _sample(K, logits, T, alpha, None)
    scaled = alpha * logits / T
    ref_lp = scaled.gather(1, tok.long().unsqueeze(1)).squeeze(1) - torch.logsumexp(scaled, -1)
    ref_lz = torch.logsumexp(scaled, -1) - alpha * torch.logsumexp(logits / T, -1)
    assert (lp - ref_lp).abs().max().item() < 2e-3
    assert (lz - ref_lz).abs().max().item() < 2e-3
    _, _, lz1 = _sample(K, logits, T, 1.0, None)
    assert lz1.abs().max().item() == 0.0
    tok2, _, _ = _sample(K, logits, T, alpha, None)
    assert torch.equal(tok, tok2)
    tok3, _, _ = _sample(K, logits, T, alpha, None, counter=1)
    assert not torch.equal(tok, tok3)
    # mixed rows: given tokens are scored, the rest sampled
    given = torch.full((8,), -1, dtype=torch.int32, device="cuda")
    given[:4] = 5
    tok4, lp4, _ = _sample(K, logits, T, 1.0, given)
    assert (tok4[:4] == 5).all()
    ref = (logits / T)[:4, 5] - torch.logsumexp(logits[:4] / T, -1)
    assert (lp4[:4] - ref).abs().max().item() < 2e-3


def test_sample_distribution_tv():
    K = _K()
    torch.manual_seed(8)
    V, rows = 512, 2000
    base = torch.randn(V, device="cuda") * 1.5
    logits = base.unsqueeze(0).repeat(rows, 1).contiguous()
    counts = torch.zeros(V, device="cuda")
    for it in range(10):
        tok, _, _ = _sample(K, logits, 0.7, 1.0, None, counter=it)
        counts += torch.bincount(tok.long(), minlength=V).float()
    emp = counts / counts.sum()
    p = torch.softmax(base / 0.7, -1)
    assert 0.5 * (emp - p).abs().sum().item() < 0.08


# ------------------------------------------------------------------------------- SMC state kernels
def _make_states(N=4, groups=3, gamma=4, seed=0):
    from smcsd_b200.memory.pools import BlockTable, PageAllocator
    from smcsd_b200.ops.native_backend import NativeState
    from smcsd_b200.runtime.slot_state import SlotState
    out = []
    for native in (False, True):
        alloc = PageAllocator(4096, "cuda")
        bt = BlockTable(groups * N, 4, 256, "cuda")
        ns = NativeState(groups * N, gamma, torch.device("cuda")) if native else None
        st = SlotState(max_groups=groups, n_particles=N, gamma=gamma, max_output_len=256, block_table=bt,
                       allocator=alloc, device="cuda", seed=seed, resample_threshold=0.5, native=ns)
        for gi in range(groups):
            L = 10 + gi
            row = bt.alloc_parent_row()
            pages = alloc.alloc(L)
            bt.table[row, :L] = pages
            st.allocate_group(f"g{gi}", prompt_len=L, x0=100 + gi, last_prompt_token=7, max_new_tokens=20 - 6 * gi,
                              ignore_eos=(gi == 1), eos_ids=[3, 5], parent_row=row)
            bt.free_parent_row(row)
        out.append(st)
    return out


def test_state_kernels_match_torch_reference():
    _K()
    from smcsd_b200.runtime.slot_state import CycleOutputs
    ref, nat = _make_states()
    g = torch.Generator(device="cuda").manual_seed(0)
    for cyc in range(5):
        cr, cn = ref.prepare_cycle(), nat.prepare_cycle()
        assert torch.equal(cr.orig_seq_lens, cn.orig_seq_lens) and torch.equal(cr.x0, cn.x0)
        assert torch.equal(cr.prev, cn.prev)
        bs = cr.slots.numel()
        tokens = torch.randint(0, 12, (bs, 5), generator=g, device="cuda", dtype=torch.int32)
        diff = torch.randn(bs, 4, generator=g, device="cuda") * 2.0
        logz = torch.randn(bs, generator=g, device="cuda") * 0.1
        out = CycleOutputs(tokens, diff, logz)
        ref.write_back(cr, out)
        nat.write_back(cn, out)
        torch.cuda.synchronize()
        for f in ("token_counts", "finished", "finished_len", "finish_code", "matched_eos", "verified_ids", "prev_ids"):
            assert torch.equal(getattr(ref, f), getattr(nat, f)), (cyc, f)
        assert torch.allclose(ref.log_weights, nat.log_weights, atol=1e-5)
        assert torch.equal(ref.all_token_ids, nat.all_token_ids)
        ref.resample()
        nat.resample()
        torch.cuda.synchronize()
        assert torch.equal(ref.seq_lens, nat.seq_lens)
        assert torch.allclose(ref.interval_weights, nat.interval_weights, atol=1e-5), cyc
        assert torch.allclose(ref.group_log_Z, nat.group_log_Z, atol=1e-5), cyc
        assert torch.equal(ref.all_token_ids, nat.all_token_ids)
        assert torch.equal(ref.token_counts, nat.token_counts)
        # same sharing structure: each row's pages have the same refcounts in both worlds
        for s in range(ref.max_slots):
            L = int(ref.seq_lens[s])
            rr = ref.alloc.refcount[ref.bt.table[s, :L].long()]
            rn = nat.alloc.refcount[nat.bt.table[s, :L].long()]
            assert torch.equal(rr, rn), (cyc, s)
        assert ref.alloc.available() == nat.alloc.available()
        nat.alloc.check_conservation()
    assert int(nat.counters[2]) > 0, "no group resampled: the test did not exercise the copy path"
    for gi in range(3):
        nat.free_group(f"g{gi}")
        ref.free_group(f"g{gi}")
    nat.alloc.check_conservation()
    assert nat.alloc.available() == nat.alloc.size


# ------------------------------------------------------------------------------- fused attention step
@pytest.mark.parametrize("bs,E,Hq,Hkv,D,ctx,KS,rd,extras", [
    (8, 9, 32, 8, 128, 1500, 1, 128, False), (8, 1, 32, 8, 64, 700, 1, 64, False), (5, 2, 32, 8, 64, 300, 1, 64, False),
    (8, 9, 32, 8, 128, 3, 1, 128, False), (3, 9, 4, 4, 64, 200, 1, 64, False), (4, 9, 16, 2, 256, 260, 1, 64, True),
    (2, 5, 4, 2, 64, 0, 1, 64, False), (4, 9, 32, 8, 128, 2500, 1, 128, False), (4, 9, 32, 8, 128, 2500, 2, 128, False),
    (3, 1, 8, 2, 128, 900, 4, 128, True), (8, 9, 64, 8, 128, 100, 1, 128, False),
    (8, 9, 32, 8, 128, 4000, 4, 128, False), (8, 1, 32, 8, 64, 4000, 8, 64, False), (4, 9, 16, 2, 256, 1000, 2, 64, True),
    (3, 2, 8, 2, 64, 40, 4, 64, False), (8, 9, 16, 2, 128, 300, 2, 128, False), (2, 9, 32, 2, 128, 700, 4, 128, True),
])
def test_attention_fused(bs, E, Hq, Hkv, D, ctx, KS, rd, extras):
    K = _K()
    from smcsd_b200.models.layers import ExtendBatch, apply_rope, paged_attention_reference, rmsnorm, rope_table
    torch.manual_seed(9)
    dev = "cuda"
    T = bs * E
    pages = bs * (ctx + E) + 64
    kp = torch.randn(pages + 1, Hkv * D, device=dev).bfloat16()
    vp = torch.randn(pages + 1, Hkv * D, device=dev).bfloat16()
    max_ctx = ctx + E + 8
    bt = torch.zeros(bs + 2, max_ctx, device=dev, dtype=torch.int32)
    perm = (torch.randperm(pages, device=dev) + 1).to(torch.int32)
    prefix = torch.tensor([max(0, ctx - 17 * i) for i in range(bs)], device=dev, dtype=torch.int32)
    rows = torch.arange(bs, device=dev, dtype=torch.int32) + 1
    locs = torch.zeros(T, device=dev, dtype=torch.int32)
    pos = torch.zeros(T, device=dev, dtype=torch.int32)
    off = 0
    for b in range(bs):
        P = int(prefix[b])
        L = P + E
        bt[b + 1, :L] = perm[off:off + L]
        locs[b * E:(b + 1) * E] = perm[off + P:off + L]
        pos[b * E:(b + 1) * E] = torch.arange(P, L, device=dev)
        off += L
    gate = extras
    nq, nk = Hq * D, Hkv * D
    ld = nq * (2 if gate else 1) + 2 * nk
    qkv = torch.randn(T, ld, device=dev)
    q_off, gate_off = 0, (nq if gate else -1)
    k_off = nq * (2 if gate else 1)
    v_off = k_off + nk
    table = rope_table(rd, 10000.0, None, max_ctx + 8, dev)
    qn = (torch.randn(D, device=dev) * 0.1).bfloat16() if extras else None
    kn = (torch.randn(D, device=dev) * 0.1).bfloat16() if extras else None
    # reference
    q = qkv[:, :nq].view(T, Hq, D)
    k = qkv[:, k_off:k_off + nk].view(T, Hkv, D)
    v = qkv[:, v_off:v_off + nk].view(T, Hkv, D)
    if extras:
        q = rmsnorm(q, qn.float(), 1e-6, plus_one=True)
        k = rmsnorm(k, kn.float(), 1e-6, plus_one=True)
    qr = apply_rope(q, pos, table).bfloat16()
    kr = apply_rope(k, pos, table).bfloat16()
    kp_ref, vp_ref = kp.clone(), vp.clone()
    kp_ref[locs.long()] = kr.reshape(T, -1)
    vp_ref[locs.long()] = v.bfloat16().reshape(T, -1)
    batch = ExtendBatch(None, None, None, rows, prefix, extend_len=E)
    ref = paged_attention_reference(qr, kp_ref, vp_ref, bt, batch, Hkv).float()
    if gate:
        ref = ref * torch.sigmoid(qkv[:, nq:2 * nq].view(T, Hq, D))
    ref = ref.reshape(T, -1)
    out = torch.zeros(T, nq, device=dev, dtype=torch.bfloat16)
    pa = torch.zeros(T * Hq * KS * D, device=dev)
    pm = torch.zeros(T * Hq * KS * 2, device=dev)
    st = _status()
    K.attention_fused(qkv, pos, locs, table, kp, vp, bt, rows, prefix, out, pa, pm, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D,
                      KS=KS, scale=D ** -0.5, status=st, q_off=q_off, gate_off=gate_off, k_off=k_off, v_off=v_off,
                      qn_w=qn, kn_w=kn, norm_eps=1e-6, norm_plus_one=True)
    torch.cuda.synchronize()
    assert int(st) == 0
    assert torch.equal(kp[locs.long()], kp_ref[locs.long()]) or \
        (kp[locs.long()].float() - kp_ref[locs.long()].float()).abs().max().item() < 4e-2
    assert (vp[locs.long()].float() - vp_ref[locs.long()].float()).abs().max().item() < 1e-6
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("bs,E,Hq,Hkv,D,ctx,KS,two_pass", [
    (8, 9, 32, 8, 128, 1500, 1, False), (8, 1, 32, 8, 64, 700, 1, False), (5, 2, 32, 8, 64, 300, 2, False),
    (4, 9, 32, 8, 128, 2500, 4, False), (3, 9, 8, 2, 128, 200, 1, True), (2, 5, 4, 2, 64, 0, 1, False),
    (4, 9, 16, 2, 256, 260, 1, False), (6, 16, 32, 8, 128, 180, 1, True),
])
def test_attention_fused_e4m3_kv_cache(bs, E, Hq, Hkv, D, ctx, KS, two_pass):
    """The e4m3 KV cache (value bytes + one scale per token and kv head in every page row): cached tiles are expanded
    to bf16 after they land, new rows are quantised on their way to the pages (inside the attention step, or by the
    store kernel behind the rope kernel for prompt passes).  Oracle: PyTorch attention over the dequantised pages."""
    K = _K()
    from smcsd_b200.memory.pools import kv_rows_from_float, kv_rows_to_float
    from smcsd_b200.models.layers import ExtendBatch, apply_rope, paged_attention_reference, rope_table
    torch.manual_seed(19)
    dev = "cuda"
    T = bs * E
    pages = bs * (ctx + E) + 64
    rw = K.kv_row_bytes_e4m3(Hkv, D)
    kp = kv_rows_from_float(torch.randn(pages + 1, Hkv, D, device=dev), rw)
    vp = kv_rows_from_float(torch.randn(pages + 1, Hkv, D, device=dev), rw)
    kp[0].zero_(); vp[0].zero_()
    max_ctx = ctx + E + 8
    bt = torch.zeros(bs + 2, max_ctx, device=dev, dtype=torch.int32)
    perm = (torch.randperm(pages, device=dev) + 1).to(torch.int32)
    prefix = torch.tensor([max(0, ctx - 17 * i) for i in range(bs)], device=dev, dtype=torch.int32)
    rows = torch.arange(bs, device=dev, dtype=torch.int32) + 1
    locs = torch.zeros(T, device=dev, dtype=torch.int32)
    pos = torch.zeros(T, device=dev, dtype=torch.int32)
    off = 0
    for b in range(bs):
        P = int(prefix[b])
        L = P + E
        bt[b + 1, :L] = perm[off:off + L]
        locs[b * E:(b + 1) * E] = perm[off + P:off + L]
        pos[b * E:(b + 1) * E] = torch.arange(P, L, device=dev)
        off += L
    nq, nk = Hq * D, Hkv * D
    qkv = torch.randn(T, nq + 2 * nk, device=dev)
    table = rope_table(D, 10000.0, None, max_ctx + 8, dev)
    qr = apply_rope(qkv[:, :nq].view(T, Hq, D), pos, table).bfloat16()
    kr = apply_rope(qkv[:, nq:nq + nk].view(T, Hkv, D), pos, table).bfloat16()
    vr = qkv[:, nq + nk:].view(T, Hkv, D).bfloat16()
    kp_ref, vp_ref = kp.clone(), vp.clone()
    kp_ref[locs.long()] = kv_rows_from_float(kr, rw)
    vp_ref[locs.long()] = kv_rows_from_float(vr, rw)
    batch = ExtendBatch(None, None, None, rows, prefix, extend_len=E)
    ref = paged_attention_reference(qr, kp_ref, vp_ref, bt, batch, Hkv).float().reshape(T, -1)
    out = torch.zeros(T, nq, device=dev, dtype=torch.bfloat16)
    st = _status()
    if two_pass:
        q_rot = torch.zeros(T, nq, device=dev, dtype=torch.bfloat16)
        K.rope_kv_write(qkv, 1, 0, pos, locs, table, q_rot, kp, vp, M=T, Hq=Hq, Hkv=Hkv, D=D, status=st)
        K.attention_fused(qkv, pos, locs, table, kp, vp, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D, KS=KS,
                          scale=D ** -0.5, status=st, q_in=q_rot)
    else:
        K.attention_fused(qkv, pos, locs, table, kp, vp, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D, KS=KS,
                          scale=D ** -0.5, status=st)
    torch.cuda.synchronize()
    assert int(st) == 0
    # the rows written by the kernels dequantise to (nearly) the same values as the PyTorch quantiser's
    got_k = kv_rows_to_float(kp[locs.long()], Hkv, D)
    want_k = kv_rows_to_float(kp_ref[locs.long()], Hkv, D)
    assert (got_k - want_k).abs().max().item() < 0.07 * want_k.abs().max().item()
    got_v = kv_rows_to_float(vp[locs.long()], Hkv, D)
    want_v = kv_rows_to_float(vp_ref[locs.long()], Hkv, D)
    assert (got_v - want_v).abs().max().item() < 0.07 * want_v.abs().max().item()
    untouched = torch.ones(pages + 1, dtype=torch.bool, device=dev)
    untouched[locs.long()] = False
    assert torch.equal(kp[untouched], kp_ref[untouched]) and torch.equal(vp[untouched], vp_ref[untouched])
    err = (out.float() - ref).abs().max().item()
    # in the single-launch form the step attends its own new tokens in bf16 (before quantisation); the oracle reads
    # them back from the e4m3 pages
    assert err < 6e-2 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("N,E,Hq,Hkv,D,P,suffix,KSg,KSs", [(8, 1, 32, 8, 64, 1500, 300, 4, 2), (8, 2, 32, 8, 64, 900, 70, 2, 1),
                                                         (4, 2, 8, 2, 128, 333, 5, 1, 1)])
def test_attention_shared_prefix_two_launches(N, E, Hq, Hkv, D, P, suffix, KSg, KSs):
    """Draft-step form of the shared-prefix passes: the group pass takes the fp32 projections, rotates the (at most 16)
    tokens' queries itself and writes nothing; the per-particle pass is the ordinary step (rope, KV write, new-token
    tile) started behind the shared keys.  Must equal the single launch and the PyTorch oracle."""
    K = _K()
    from smcsd_b200.models.layers import ExtendBatch, apply_rope, paged_attention_reference, rope_table
    torch.manual_seed(23)
    dev = "cuda"
    bs, T = N, N * E
    pages = P + bs * (suffix + E) + 64
    kp = torch.randn(pages + 1, Hkv * D, device=dev).bfloat16()
    vp = torch.randn(pages + 1, Hkv * D, device=dev).bfloat16()
    perm = (torch.randperm(pages, device=dev) + 1).to(torch.int32)
    bt = torch.zeros(bs + 2, P + suffix + E + 8, device=dev, dtype=torch.int32)
    prefix = torch.zeros(bs, device=dev, dtype=torch.int32)
    locs = torch.zeros(T, device=dev, dtype=torch.int32)
    pos = torch.zeros(T, device=dev, dtype=torch.int32)
    off = P
    for b in range(bs):
        own = max(suffix - (b % 3), 0)
        bt[b + 1, :P] = perm[:P]
        bt[b + 1, P:P + own + E] = perm[off:off + own + E]
        locs[b * E:(b + 1) * E] = perm[off + own:off + own + E]
        pos[b * E:(b + 1) * E] = torch.arange(P + own, P + own + E, device=dev)
        off += own + E
        prefix[b] = P + own
    rows = torch.arange(bs, device=dev, dtype=torch.int32) + 1
    nq, nk = Hq * D, Hkv * D
    qkv = torch.randn(T, nq + 2 * nk, device=dev)
    table = rope_table(D, 10000.0, None, P + suffix + E + 16, dev)
    qr = apply_rope(qkv[:, :nq].view(T, Hq, D), pos, table).bfloat16()
    kr = apply_rope(qkv[:, nq:nq + nk].view(T, Hkv, D), pos, table).bfloat16()
    kp_ref, vp_ref = kp.clone(), vp.clone()
    kp_ref[locs.long()] = kr.reshape(T, -1)
    vp_ref[locs.long()] = qkv[:, nq + nk:].bfloat16()
    ref = paged_attention_reference(qr, kp_ref, vp_ref, bt, ExtendBatch(None, None, None, rows, prefix, extend_len=E),
                                    Hkv).float().reshape(T, -1)
    st = _status()
    state = torch.zeros(T, Hq, D + 2, device=dev)
    shared = torch.full((bs,), P, device=dev, dtype=torch.int32)
    out2 = torch.zeros(T, nq, device=dev, dtype=torch.bfloat16)
    kp2, vp2 = kp.clone(), vp.clone()
    K.attention_fused(qkv, pos, locs, table, kp2, vp2, bt, rows[::N].contiguous(), shared[::N].contiguous(), None, bs=1,
                      E=N * E, Hq=Hq, Hkv=Hkv, D=D, KS=KSg, scale=D ** -0.5, status=st, part_out=state, causal=False)
    assert torch.equal(kp2, kp) and torch.equal(vp2, vp)              # the group pass writes no K/V rows
    K.attention_fused(qkv, pos, locs, table, kp2, vp2, bt, rows, prefix, out2, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D, KS=KSs,
                      scale=D ** -0.5, status=st, key_begin=shared, part_in=state)
    out1 = torch.zeros_like(out2)
    K.attention_fused(qkv, pos, locs, table, kp, vp, bt, rows, prefix, out1, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D, KS=1,
                      scale=D ** -0.5, status=st)
    # the tcgen05 group pass in the same role: rotates the fp32 queries itself, one parked state per key split
    kst = K.attention_tc_splits(1, Hkv, P, N * E * (Hq // Hkv))
    state_tc = torch.full((kst, T, Hq, D + 2), float("nan"), device=dev)
    out3 = torch.zeros_like(out2)
    kp3, vp3 = kp2.clone(), vp2.clone()
    K.attention_prefix_tc(None, kp3, vp3, bt, rows[::N].contiguous(), shared[::N].contiguous(), state_tc, n_seq=1,
                          E=N * E, T=T, Hq=Hq, Hkv=Hkv, D=D, KS=kst, scale=D ** -0.5, status=st, qkv=qkv, q_off=0,
                          positions=pos, rope=table)
    K.attention_fused(qkv, pos, locs, table, kp3, vp3, bt, rows, prefix, out3, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D, KS=KSs,
                      scale=D ** -0.5, status=st, key_begin=shared, part_in=state_tc, part_in_n=kst,
                      part_in_stride=state_tc.stride(0))
    torch.cuda.synchronize()
    assert int(st) == 0
    assert torch.equal(kp2, kp) and torch.equal(vp2, vp)              # both forms wrote the same new rows
    tol = 3e-2 * max(1.0, ref.abs().max().item())
    assert (out1.float() - ref).abs().max().item() < tol
    assert (out2.float() - ref).abs().max().item() < tol
    assert (out3.float() - ref).abs().max().item() < tol


@pytest.mark.parametrize("groups,N,NP,E,Hq,Hkv,D,P,suffix,KSg,KSs", [
    (1, 8, 8, 1, 32, 8, 64, 1500, 300, 4, 2), (1, 8, 2, 9, 32, 8, 128, 2100, 200, 4, 1), (2, 4, 4, 2, 8, 2, 64, 700, 40, 2, 1),
    (1, 8, 8, 1, 32, 8, 64, 100, 1200, 1, 4), (1, 4, 2, 5, 8, 2, 128, 333, 0, 1, 1),
])
@pytest.mark.parametrize("tc", [False, "scattered", "runs"])
def test_attention_shared_prefix_passes(groups, N, NP, E, Hq, Hkv, D, P, suffix, KSg, KSs, tc):
    """Shared-prefix attention: one pass over the prompt keys for NP particles at a time (state parked per token and
    head), then the per-particle pass over the remaining keys folds it in.  Must equal plain causal attention.
    ``tc``: the group pass runs on the tcgen05 kernel (one parked state per key split) instead of the mma.sync one,
    with every prompt page scattered (row gather) or with the prompt in consecutive pages except for one reversed and
    one shuffled stretch (ascending and descending TMA tiles and gathered tiles in the same launch)."""
    K = _K()
    from smcsd_b200.models.layers import ExtendBatch, paged_attention_reference
    torch.manual_seed(13)
    dev = "cuda"
    bs = groups * N
    T = bs * E
    pages = groups * P + bs * (suffix + E) + 64
    kp = torch.randn(pages + 1, Hkv * D, device=dev).bfloat16()
    vp = torch.randn(pages + 1, Hkv * D, device=dev).bfloat16()
    perm = (torch.randperm(pages, device=dev) + 1).to(torch.int32)
    bt = torch.zeros(bs + 2, P + suffix + E + 8, device=dev, dtype=torch.int32)
    off = 0
    shared = []
    if tc == "runs":
        # prompts take pages 1 .. groups * P in order; keys 128..191 of each are shuffled so that one tile is gathered
        rest = torch.arange(groups * P, pages, device=dev)
        perm = torch.cat([torch.arange(groups * P, device=dev), rest[torch.randperm(rest.numel(), device=dev)]])
        perm = (perm + 1).to(torch.int32)
    for gi in range(groups):
        pg = perm[off:off + P].clone()
        if tc == "runs" and P >= 192:
            pg[128:192] = pg[128:192].flip(0)                      # a descending run: still one TMA box
        if tc == "runs" and P >= 320:
            pg[256:320] = pg[256:320][torch.randperm(64, device=dev)]   # a scattered tile: gathered row by row
        shared.append(pg)
        off += P
    prefix = torch.zeros(bs, device=dev, dtype=torch.int32)
    for b in range(bs):
        gi = b // N
        own = suffix - (b % 3)                      # particles of a group may differ in length in this test
        own = max(own, 0)
        bt[b + 1, :P] = shared[gi]
        bt[b + 1, P:P + own + E] = perm[off:off + own + E]
        off += own + E
        prefix[b] = P + own
    rows = torch.arange(bs, device=dev, dtype=torch.int32) + 1
    q = torch.randn(T, Hq, D, device=dev).bfloat16()                 # rotated queries; new K/V already in their pages
    batch = ExtendBatch(None, None, None, rows, prefix, extend_len=E)
    ref = paged_attention_reference(q, kp, vp, bt, batch, Hkv).float().reshape(T, -1)
    st = _status()
    dummy = torch.zeros(8, device=dev)
    qkv = torch.zeros(T, (Hq + 2 * Hkv) * D, device=dev)
    pos = torch.zeros(T, device=dev, dtype=torch.int32)
    locs = torch.zeros(T, device=dev, dtype=torch.int32)
    table = torch.zeros(16, D, device=dev)
    state = torch.zeros(T, Hq, D + 2, device=dev)
    n_super = bs // NP
    rows_g = rows[::NP].contiguous()
    shared_len = torch.full((bs,), P, device=dev, dtype=torch.int32)
    out = torch.zeros(T, Hq * D, device=dev, dtype=torch.bfloat16)
    if tc:
        if D == 256:
            pytest.skip("the tcgen05 pass is built for head sizes 64 and 128")
        state = torch.full((KSg, T, Hq, D + 2), float("nan"), device=dev)
        K.attention_prefix_tc(q.reshape(T, -1), kp, vp, bt, rows_g, shared_len[::NP].contiguous(), state, n_seq=n_super,
                              E=NP * E, T=T, Hq=Hq, Hkv=Hkv, D=D, KS=KSg, scale=D ** -0.5, status=st)
        K.attention_fused(qkv, pos, locs, table, kp, vp, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D, KS=KSs,
                          scale=D ** -0.5, status=st, q_in=q.reshape(T, -1), key_begin=shared_len, part_in=state,
                          part_in_n=KSg, part_in_stride=state.stride(0))
    else:
        K.attention_fused(qkv, pos, locs, table, kp, vp, bt, rows_g, shared_len[::NP].contiguous(), None, bs=n_super,
                          E=NP * E, Hq=Hq, Hkv=Hkv, D=D, KS=KSg, scale=D ** -0.5, status=st, q_in=q.reshape(T, -1),
                          part_out=state, causal=False)
        K.attention_fused(qkv, pos, locs, table, kp, vp, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D, KS=KSs,
                          scale=D ** -0.5, status=st, q_in=q.reshape(T, -1), key_begin=shared_len, part_in=state)
    torch.cuda.synchronize()
    assert int(st) == 0
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2 * max(1.0, ref.abs().max().item()), err


# ------------------------------------------------------------------------------- FP8 (W8A8) GEMM
def test_quant_rows_e4m3_matches_torch():
    K = _K()
    torch.manual_seed(31)
    M, Kd = 37, 4096
    x = (torch.randn(M, Kd, device="cuda") * torch.rand(M, 1, device="cuda") * 3).bfloat16()
    q = torch.zeros(M, Kd, device="cuda", dtype=torch.uint8)
    sc = torch.zeros(M, device="cuda")
    K.quant_rows_e4m3(x, q, sc, M=M, K=Kd)
    torch.cuda.synchronize()
    ref_sc = x.float().abs().amax(dim=1) / 448.0
    assert torch.allclose(sc, ref_sc, rtol=1e-6)
    deq = q.view(torch.float8_e4m3fn).float() * sc[:, None]
    # e4m3 keeps 3 mantissa bits: round-to-nearest error <= 2^-4 of the value (plus the subnormal step near zero)
    err = (deq - x.float()).abs()
    assert (err <= x.float().abs() * 2 ** -4 + sc[:, None] * 2 ** -9 * 1.001).all()
    ref_q = (x.float() / ref_sc[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    assert (q != ref_q).float().mean().item() < 1e-3          # x * (1 / scale) against x / scale: rare one-step ties


@pytest.mark.parametrize("N,Kd,M,splits", [
    (3072, 2048, 8, 8), (6144, 4096, 72, 4), (4096, 14336, 72, 4), (2048, 8192, 8, 8), (1024, 512, 40, 2),
    (4096, 4096, 200, 1), (300, 1024, 9, 1),
])
def test_gemm_fp8_matches_dequantised_reference(N, Kd, M, splits):
    """W8A8 on tcgen05 kind::f8f6f4: e4m3 products are exact in fp32, so against an fp32 matmul of the dequantised
    operands only the accumulation order differs.  Plain store, residual accumulate and bf16 store epilogues."""
    K = _K()
    torch.manual_seed(32)
    W = torch.randn(N, Kd, device="cuda") * 0.05
    X = torch.randn(M, Kd, device="cuda").bfloat16()
    W8, ws = K.quantize_weight_e4m3(W)
    X8 = torch.zeros(M, Kd, device="cuda", dtype=torch.uint8)
    xs = torch.zeros(M, device="cuda")
    K.quant_rows_e4m3(X, X8, xs, M=M, K=Kd)
    ref = (X8.view(torch.float8_e4m3fn).float() * xs[:, None]) @ (W8.view(torch.float8_e4m3fn).float() * ws[:, None]).t()
    st = _status()
    out = torch.full((M, N), float("nan"), device="cuda")
    K.gemm_skinny_fp8(W8, ws, X8, xs, out, M=M, splits=splits, epi=K.EPI_STORE_F32, ldo=N, status=st)
    h0 = torch.randn(M, N, device="cuda")
    h = h0.clone()
    K.gemm_skinny_fp8(W8, ws, X8, xs, h, M=M, splits=splits, epi=K.EPI_RESID_F32, ldo=N, status=st, pdl=True)
    ob = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    K.gemm_skinny_fp8(W8, ws, X8, xs, ob, M=M, splits=1, epi=K.EPI_BF16, ldo=N, status=st)
    torch.cuda.synchronize()
    assert int(st) == 0
    tol = 1e-3 * max(1.0, ref.abs().max().item())
    assert (out - ref).abs().max().item() < tol
    assert (h - h0 - ref).abs().max().item() < tol
    assert (ob.float() - ref).abs().max().item() < 6e-3 * max(1.0, ref.abs().max().item())
    # and the quantised product stays close to the bf16 one (e4m3 noise averages out over K)
    full = X.float() @ W.t()
    assert (out - full).abs().max().item() < 0.08 * full.abs().max().item()


@pytest.mark.parametrize("ffn,d,M,splits", [(8192, 2048, 8, 1), (14336, 4096, 72, 1), (1024, 256, 40, 2)])
def test_gemm_fp8_swiglu_epilogue(ffn, d, M, splits):
    K = _K()
    from smcsd_b200.models.llama import interleave_gate_up
    torch.manual_seed(33)
    Wg, Wu = torch.randn(ffn, d, device="cuda") * 0.05, torch.randn(ffn, d, device="cuda") * 0.05
    Wgu = interleave_gate_up(Wg.bfloat16(), Wu.bfloat16(), 64)
    W8, ws = K.quantize_weight_e4m3(Wgu)
    X = torch.randn(M, d, device="cuda").bfloat16()
    X8 = torch.zeros(M, d, device="cuda", dtype=torch.uint8)
    xs = torch.zeros(M, device="cuda")
    K.quant_rows_e4m3(X, X8, xs, M=M, K=d)
    from smcsd_b200.models.llama import split_gate_up
    full = (X8.view(torch.float8_e4m3fn).float() * xs[:, None]) @ (W8.view(torch.float8_e4m3fn).float() * ws[:, None]).t()
    g, u = split_gate_up(full, 64)
    ref = torch.nn.functional.silu(g) * u
    act = torch.zeros(M, ffn, device="cuda", dtype=torch.bfloat16)
    st = _status()
    K.gemm_skinny_fp8(W8, ws, X8, xs, act, M=M, splits=splits, epi=K.EPI_SWIGLU_BF16, ldo=ffn, status=st)
    torch.cuda.synchronize()
    assert int(st) == 0
    assert (act.float() - ref).abs().max().item() < 6e-3 * max(1.0, ref.abs().max().item())


# ------------------------------------------------------------------------------- RMSNorm folded into the GEMMs
@pytest.mark.parametrize("d,ffn,M", [(2048, 8192, 8), (4096, 14336, 72), (512, 1536, 20)])
def test_gemm_with_folded_rmsnorm(d, ffn, M):
    """Producer: h += X W^T also emits bf16(h) and per-slab sums of squares.  Consumer: GEMM on the raw bf16 rows,
    scaled per token by 1/rms in the epilogue == GEMM on the normalised rows."""
    K = _K()
    from smcsd_b200.models.llama import interleave_gate_up
    torch.manual_seed(21)
    dev = "cuda"
    st = _status()
    Wd = (torch.randn(d, ffn, device=dev) * 0.03).bfloat16()
    act = torch.randn(M, ffn, device=dev).bfloat16()
    h0 = torch.randn(M, d, device=dev)
    h = h0.clone()
    parts = (d + 127) // 128
    ssq = torch.zeros(parts, 128, device=dev)          # leading dimension 128 > M on purpose
    hb = torch.zeros(M, d, device=dev, dtype=torch.bfloat16)
    s = K.gemm_cluster_splits(d, ffn, M)
    K.gemm_skinny_norm(Wd, act, h, M=M, splits=s, epi=K.EPI_RESID_F32, ldo=d, status=st, ssq_out=ssq, hb_out=hb)
    torch.cuda.synchronize()
    h_ref = h0 + act.float() @ Wd.float().t()
    assert (h - h_ref).abs().max().item() < 2e-2 * max(1.0, h_ref.abs().max().item())
    assert torch.equal(hb, h.bfloat16())
    ssq_ref = (h.float() ** 2).view(M, parts, -1).sum(-1).t()
    assert torch.allclose(ssq[:, :M], ssq_ref, rtol=1e-4, atol=1e-3)
    # consumer with SwiGLU epilogue
    Wg = (torch.randn(ffn, d, device=dev) * 0.03).bfloat16()
    Wu = (torch.randn(ffn, d, device=dev) * 0.03).bfloat16()
    Wgu = interleave_gate_up(Wg, Wu, 64)
    out = torch.zeros(M, ffn, device=dev, dtype=torch.bfloat16)
    K.gemm_skinny_norm(Wgu, hb, out, M=M, splits=1, epi=K.EPI_SWIGLU_BF16, ldo=ffn, status=st, ssq_in=ssq,
                       ssq_parts=parts, norm_d=d, norm_eps=1e-5)
    xn = hb.float() * torch.rsqrt((h.float() ** 2).mean(-1, keepdim=True) + 1e-5)
    ref = torch.nn.functional.silu(xn @ Wg.float().t()) * (xn @ Wu.float().t())
    torch.cuda.synchronize()
    assert (out.float() - ref).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item())
    # consumer with the clustered fp32 store and a strided row selection (every second row from row 1)
    Wq = (torch.randn(1024, d, device=dev) * 0.03).bfloat16()
    rows = (M - 1 + 1) // 2
    q = torch.zeros(rows, 1024, device=dev)
    K.gemm_skinny_norm(Wq, hb[1:], q, M=rows, splits=K.gemm_cluster_splits(1024, d, rows), epi=K.EPI_STORE_F32,
                       ldo=1024, status=st, ssq_in=ssq[:, 1:], ssq_parts=parts, norm_d=d, norm_eps=1e-5,
                       ldx=2 * d, ssq_ld=ssq.stride(0), ssq_mstride=2)
    torch.cuda.synchronize()
    ref = xn[1::2][:rows] @ Wq.float().t()
    assert int(st) == 0
    assert (q - ref).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item())


# ------------------------------------------------------------------------------- lm_head fused with sampling
@pytest.mark.parametrize("V,d,M,step", [(128256, 2048, 8, 1), (128256, 4096, 72, 1), (1000, 256, 8, 2), (8192, 512, 130, 1)])
def test_lm_head_sampling_epilogue_matches_sampler_on_stored_logits(V, d, M, step):
    """Sampling / scoring inside the lm_head epilogue against the stand-alone sampler run on the stored logits of the
    same GEMM (same noise stream): same tokens, same log-probabilities; and against fp32 PyTorch for the scored rows."""
    K = _K()
    torch.manual_seed(4)
    W = (torch.randn(V, d, device="cuda") * 0.05).bfloat16()
    X = torch.randn(M * step, d, device="cuda").bfloat16()
    st = _status()
    logits = torch.zeros(M, V, device="cuda")
    K.gemm_skinny(W, X[step - 1:], logits, M=M, splits=1, epi=K.EPI_STORE_F32, ldx=d * step, ldo=V, status=st)
    tokens_in = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    tokens_in[::2] = torch.randint(0, V, (tokens_in[::2].numel(),), device="cuda", dtype=torch.int32)
    counters = torch.tensor([3, 0, 0, 0], dtype=torch.int64, device="cuda")
    T, alpha = 0.7, 1.4
    tok_a, lp_a, lz_a = _sample(K, logits, T, alpha, tokens_in, seed=99, counter=3, call_id=2)
    parts = torch.empty(K.lm_parts_bytes(M, V), dtype=torch.uint8, device="cuda")
    tok_b = torch.zeros(M, dtype=torch.int32, device="cuda")
    lp_b = torch.zeros(M, device="cuda")
    lz_b = torch.zeros(M, device="cuda")
    K.lm_head_sample(W, X[step - 1:], M=M, V=V, ldx=d * step, status=st, temperature=T, alpha=alpha, softcap=0.0,
                     tokens_in=tokens_in, seed=99, cycle_counter=counters, call_id=2, parts=parts, tok_out=tok_b,
                     logp_out=lp_b, logz_out=lz_b)
    torch.cuda.synchronize()
    assert int(st) == 0
    assert torch.equal(tok_a, tok_b)
    assert (lp_a - lp_b).abs().max().item() < 2e-3
    assert (lz_a - lz_b).abs().max().item() < 2e-3
    ref = torch.log_softmax(X[step - 1::step].float() @ W.float().t() / T, dim=-1)
    sc = tokens_in >= 0
    got_ref = ref[torch.arange(M, device="cuda")[sc], tokens_in[sc].long()]
    assert (lp_b[sc] - got_ref).abs().max().item() < 5e-3


def test_add_rmsnorm_with_e4m3_output_matches_separate_quantisation():
    """The norm kernel's fused e4m3 output equals a separate quantisation pass over its bf16 output."""
    K = _K()
    torch.manual_seed(41)
    M, d = 19, 4096
    h = torch.randn(M, d, device="cuda")
    w = (1.0 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    xn = torch.zeros(M, d, device="cuda", dtype=torch.bfloat16)
    q8 = torch.zeros(M, d, device="cuda", dtype=torch.uint8)
    qs = torch.zeros(M, device="cuda")
    K.add_rmsnorm_q8(h.clone(), w, xn, q8, qs, M=M, d=d, eps=1e-5)
    ref_q = torch.zeros_like(q8)
    ref_s = torch.zeros_like(qs)
    K.quant_rows_e4m3(xn, ref_q, ref_s, M=M, K=d)
    torch.cuda.synchronize()
    ref_xn = (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()).bfloat16()
    assert (xn.float() - ref_xn.float()).abs().max().item() < 2e-2
    assert torch.allclose(qs, ref_s, rtol=1e-6)
    assert torch.equal(q8, ref_q)
