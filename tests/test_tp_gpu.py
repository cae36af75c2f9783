"""Tensor-parallel kernel path.

Single-GPU part: several ranks are emulated on one device (each rank has its own heap buffer, KV
shard and weights shard; the ranks' kernel chains are advanced in lockstep on one stream, so a
kernel never waits for a launch that comes later).  This exercises the all-gather-by-peer-store,
the reduce-scatter GEMM epilogue, the vocab-parallel sampler and the bounded-wait timeout path
without a second GPU.  The multi-GPU part runs the same check as real processes over NVLink.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    from smcsd_b200.models.config import ModelConfig
    return ModelConfig(arch="llama", vocab_size=8192, hidden_size=512, n_layers=2, n_heads=8, n_kv_heads=4,
                       head_dim=64, ffn_size=1536, max_position=1024, name="tp-test")


def _setup_batch(bs, E, P, bt, dev, gen):
    rows = torch.arange(bs, dtype=torch.int32, device=dev)
    ids = torch.randint(0, 8192, (bs * E,), generator=gen, device=dev, dtype=torch.int32)
    pos = (torch.arange(E, device=dev) + P).repeat(bs).to(torch.int32)
    locs = bt[:bs, P:P + E].reshape(-1).contiguous()
    pref = torch.full((bs,), P, dtype=torch.int32, device=dev)
    return ids, pos, locs, rows, pref


@pytest.mark.parametrize("tp,bs,E", [(2, 4, 5), (4, 3, 3), (2, 8, 1)])
def test_tp_chain_emulated_ranks_match_single_rank(tp, bs, E):
    from smcsd_b200.memory.pools import KVPool, KVSpec
    from smcsd_b200.models.llama import LlamaModel
    from smcsd_b200.ops import native as K
    from smcsd_b200.ops.native_backend import NativeLlama
    from smcsd_b200.ops.native_tp import NativeLlamaTP
    from smcsd_b200.parallel.symm import FakeHeap
    K.lib()
    dev = torch.device("cuda")
    cfg = _cfg()
    P, T = 21, bs * E
    n_pages = 512
    bt = torch.zeros(16, 256, dtype=torch.int32, device=dev)
    perm = (torch.randperm(n_pages, device=dev) + 1).to(torch.int32)
    for b in range(bs):
        bt[b, :P + E] = perm[b * 40:b * 40 + P + E]
    gen = torch.Generator(device=dev).manual_seed(0)
    ids, pos, locs, rows, pref = _setup_batch(bs, E, P, bt, dev, gen)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # single-rank reference through the same kernels
    full = LlamaModel(cfg, torch.bfloat16, dev).init_random(3)
    kv_full = KVPool(KVSpec(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim), n_pages, dev)
    kv_full.k.normal_(0, 0.5)
    kv_full.v.normal_(0, 0.5)
    ref = NativeLlama(full, kv_full, bt, T, T, 8, status, False)
    kfull, vfull = kv_full.k.clone(), kv_full.v.clone()
    ref.forward(ids, pos, locs, rows, pref, bs, E)
    ref_logits = ref.lm_head(T)[:T].clone()
    # emulated TP ranks
    heap = FakeHeap(64 << 20, dev, tp)
    ranks = []
    for r in range(tp):
        m = LlamaModel(cfg, torch.bfloat16, dev, tp_rank=r, tp_size=tp).init_random(3)
        kv = KVPool(KVSpec(cfg.n_layers, m.n_kv_heads, cfg.head_dim), n_pages, dev)
        w = m.n_kv_heads * cfg.head_dim
        kv.k.copy_(kfull[:, :, r * w:(r + 1) * w])
        kv.v.copy_(vfull[:, :, r * w:(r + 1) * w])
        h = FakeHeap.__new__(FakeHeap)
        h.__dict__.update(heap.__dict__)
        h._cursor = 0
        nm = NativeLlamaTP(m, kv, bt, T, T, 8, status, False, h,
                           heap_view=lambda off, shape, dt, r=r: heap.view(r, off, shape, dt))
        ranks.append(nm)
    gens = [nm.stages(ids, pos, locs, rows, pref, bs, E) for nm in ranks]
    while True:
        done = 0
        for g in gens:
            try:
                next(g)
            except StopIteration:
                done += 1
        if done == tp:
            break
    for nm in ranks:
        nm.lm_head(T)
    torch.cuda.synchronize()
    assert int(status) == 0
    got = torch.cat([nm.logits[:T] for nm in ranks], dim=1)[:, :cfg.vocab_size]
    scale = ref_logits.abs().max().item()
    assert (got - ref_logits).abs().max().item() < 0.05 * scale
    # vocab-parallel fused sampling / scoring: every rank gets the same answer as the single-rank sampler
    given = torch.full((T,), -1, dtype=torch.int32, device=dev)
    given[::2] = torch.randint(0, 8192, (len(given[::2]),), device=dev, dtype=torch.int32)
    ctr = torch.tensor([5], dtype=torch.int64, device=dev)
    outs = []
    for phase in (1, 2):
        for nm in ranks:
            if phase == 1:
                nm._o = (torch.zeros(T, dtype=torch.int32, device=dev), torch.zeros(T, device=dev),
                         torch.zeros(T, device=dev))
            nm.tp_sample(rows=T, temperature=0.7, alpha=1.3, tokens_in=given, seed=42, cycle_counter=ctr, call_id=2,
                         tok_out=nm._o[0], logp_out=nm._o[1], logz_out=nm._o[2], phase=phase)
    scratch = torch.empty(K.sample_scratch_bytes(T, 32), dtype=torch.uint8, device=dev)
    tok = torch.zeros(T, dtype=torch.int32, device=dev)
    lp, lz = torch.zeros(T, device=dev), torch.zeros(T, device=dev)
    K.sample_or_score(got.contiguous(), rows=T, V=cfg.vocab_size, splits=1, split_stride=0, row_stride=cfg.vocab_size,
                      temperature=0.7, alpha=1.3, softcap=0.0, tokens_in=given, seed=42, cycle_counter=ctr, call_id=2,
                      scratch=scratch, nchunks=32, tok_out=tok, logp_out=lp, logz_out=lz)
    torch.cuda.synchronize()
    assert int(status) == 0
    for nm in ranks:
        assert torch.equal(nm._o[0], ranks[0]._o[0]) and torch.equal(nm._o[1], ranks[0]._o[1])
        assert torch.equal(nm._o[0], tok)
        assert (nm._o[1] - lp).abs().max().item() < 2e-3
        assert (nm._o[2] - lz).abs().max().item() < 2e-3


@pytest.mark.parametrize("tp", [2, 4])
def test_tp_prompt_pass_emulated_ranks_match_single_rank(tp):
    """Prompt pass through the tensor-parallel chain (16-token blocks as batch rows, K/V written before attention):
    every rank ends with the same normalised last-layer rows as the single-rank chain, and its K/V shard matches."""
    from smcsd_b200.memory.pools import KVPool, KVSpec
    from smcsd_b200.models.llama import LlamaModel
    from smcsd_b200.ops import native as K
    from smcsd_b200.ops.native_backend import NativeLlama
    from smcsd_b200.ops.native_tp import NativeLlamaTP
    from smcsd_b200.parallel.symm import FakeHeap
    K.lib()
    dev = torch.device("cuda")
    cfg = _cfg()
    B = 16
    lens = [37, 16, 50]
    n_blocks = [(L + B - 1) // B for L in lens]
    bs = sum(n_blocks)
    T = bs * B
    n_pages = 512
    bt = torch.zeros(16, 256, dtype=torch.int32, device=dev)
    perm = (torch.randperm(n_pages, device=dev) + 1).to(torch.int32)
    gen = torch.Generator().manual_seed(1)
    ids = torch.zeros(T, dtype=torch.int32)
    pos = torch.zeros(T, dtype=torch.int32)
    locs = torch.zeros(T, dtype=torch.int32)
    rows, pref, last = [], [], []
    t = 0
    for i, (L, nb) in enumerate(zip(lens, n_blocks)):
        bt[i, :L] = perm[i * 64:i * 64 + L]
        ids[t:t + L] = torch.randint(0, 8192, (L,), generator=gen, dtype=torch.int32)
        pos[t:t + nb * B] = torch.arange(nb * B, dtype=torch.int32).clamp_(max=L - 1)
        locs[t:t + L] = bt[i, :L].cpu()
        rows += [i] * nb
        pref += [j * B for j in range(nb)]
        last.append(t + L - 1)
        t += nb * B
    ids, pos, locs = ids.to(dev), pos.to(dev), locs.to(dev)
    rows = torch.tensor(rows, dtype=torch.int32, device=dev)
    pref = torch.tensor(pref, dtype=torch.int32, device=dev)
    last = torch.tensor(last, dtype=torch.long, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    full = LlamaModel(cfg, torch.bfloat16, dev).init_random(3)
    kv_full = KVPool(KVSpec(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim), n_pages, dev)
    ref = NativeLlama(full, kv_full, bt, T, 8, 8, status, False)
    ref.set_context(max(lens), bs)
    ref.forward(ids, pos, locs, rows, pref, bs, B, two_pass=True)
    ref_rows = ref.final_hidden(last).float()
    heap = FakeHeap(64 << 20, dev, tp)
    ranks = []
    for r in range(tp):
        m = LlamaModel(cfg, torch.bfloat16, dev, tp_rank=r, tp_size=tp).init_random(3)
        kv = KVPool(KVSpec(cfg.n_layers, m.n_kv_heads, cfg.head_dim), n_pages, dev)
        h = FakeHeap.__new__(FakeHeap)
        h.__dict__.update(heap.__dict__)
        h._cursor = 0
        nm = NativeLlamaTP(m, kv, bt, T, 8, 8, status, False, h,
                           heap_view=lambda off, shape, dt, r=r: heap.view(r, off, shape, dt))
        nm.set_context(max(lens), bs)
        ranks.append(nm)
    gens = [nm.stages(ids, pos, locs, rows, pref, bs, B, True) for nm in ranks]
    while True:
        done = 0
        for g in gens:
            try:
                next(g)
            except StopIteration:
                done += 1
        if done == tp:
            break
    torch.cuda.synchronize()
    assert int(status) == 0
    scale = ref_rows.abs().max().item()
    valid = locs.long()[ids.new_zeros(T, dtype=torch.bool).index_fill_(0, torch.cat([torch.arange(s0, s0 + L, device=dev) for s0, L in zip([0, 48, 64], lens)]), True)]
    for r, nm in enumerate(ranks):
        got = nm.xn_a[last].float()
        assert (got - ref_rows).abs().max().item() < 0.05 * scale
        w = nm.nkv * cfg.head_dim
        for li in range(cfg.n_layers):
            a = nm.kv.k[li][valid].float()
            b = kv_full.k[li][valid][:, r * w:(r + 1) * w].float()
            assert (a - b).abs().max().item() < 0.06 * max(1.0, b.abs().max().item())


def test_bounded_peer_wait_times_out_and_reports():
    """A counter that no peer ever bumps: the wait gives up after about a second, sets the status
    bit and returns, and the context stays usable."""
    from smcsd_b200.ops import native as K
    K.tp_lib()
    dev = "cuda"
    flag = torch.zeros(1, dtype=torch.int64, device=dev)
    outcome = torch.full((1,), -1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    K.tp_wait_counter(flag.data_ptr(), 1, outcome, status)
    torch.cuda.synchronize()
    assert int(outcome) == 0 and int(status) & K.ERR_PEER_TIMEOUT
    # once the peer shows up the same wait succeeds
    K.tp_bump_counter(flag.data_ptr(), 1)
    status.zero_()
    K.tp_wait_counter(flag.data_ptr(), 1, outcome, status)
    torch.cuda.synchronize()
    assert int(outcome) == 1 and int(status) == 0


@pytest.mark.multigpu
@pytest.mark.parametrize("tp", [2])
def test_tp_chain_real_ranks(tp, tmp_path):
    if torch.cuda.device_count() < tp:
        pytest.skip("needs more GPUs")
    out = tmp_path / "res.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={tp}", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "mp_tp_check.py"), str(out)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads(out.read_text())
    assert res["status"] == 0 and res["logit_err"] < 0.05 and res["tokens_equal"] and res["ranks_agree"]
