"""Particle-parallel resampling kernels (in-kernel gather of ancestor KV pages and recurrent state
fused with the block-table rewrite), checked against the plain-PyTorch plan on emulated ranks:
two ranks share one GPU, each with its own pools, and their kernels are launched phase by phase on
one stream so that no kernel waits for a later launch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _make_rank(native: bool, n_local: int, groups: int, gamma: int, dev, with_state: bool):
    from smcsd_b200.memory.pools import BlockTable, KVPool, KVSpec, PageAllocator, StatePool, StateSpec
    from smcsd_b200.ops.native_backend import NativeState
    from smcsd_b200.runtime.slot_state import SlotState
    alloc = PageAllocator(2048, dev)
    bt = BlockTable(groups * n_local, 4, 128, dev)
    ns = NativeState(groups * n_local, gamma, torch.device(dev)) if native else None
    pools = []
    if with_state:
        spec = StateSpec(2, 24, 4, 2, 8, 8, conv_dtype=torch.float32, state_dtype=torch.float32)
        pools = [StatePool(spec, groups * n_local + 4, dev)]
    st = SlotState(max_groups=groups, n_particles=n_local, gamma=gamma, max_output_len=128, block_table=bt,
                   allocator=alloc, device=dev, seed=7, resample_threshold=0.9, native=ns, state_pools=pools)
    kvs = [KVPool(KVSpec(3, 2, 16), 2048, dev), KVPool(KVSpec(2, 1, 8), 2048, dev)]
    return st, kvs


@pytest.mark.parametrize("with_state", [False, True])
def test_cross_rank_resample_matches_reference(with_state):
    from smcsd_b200.ops import native as K
    from smcsd_b200.parallel.particle_parallel import ParticleParallel, apply_reference, plan_global
    from smcsd_b200.runtime.slot_state import CycleOutputs
    K.lib()
    dev, R, n_local, groups, gamma = "cuda", 2, 2, 2, 3
    G = gamma + 1
    nat = [_make_rank(True, n_local, groups, gamma, dev, with_state) for _ in range(R)]
    ref = [_make_rank(False, n_local, groups, gamma, dev, with_state) for _ in range(R)]
    gen = torch.Generator(device=dev).manual_seed(0)
    # prompts: same length and same (replicated) prompt KV on every rank
    for world in (nat, ref):
        for r, (st, kvs) in enumerate(world):
            for gi in range(groups):
                L = 9 + gi
                row = st.bt.alloc_parent_row()
                pages = st.alloc.alloc(L)
                st.bt.table[row, :L] = pages
                for kv in kvs:
                    base = torch.arange(L, device=dev).float().view(1, L, 1) + 100 * gi
                    kv.k[:, pages.long()] = (base + 0.25).expand(kv.k.shape[0], L, kv.k.shape[2]).to(kv.k.dtype)
                    kv.v[:, pages.long()] = (base + 0.5).expand(kv.v.shape[0], L, kv.v.shape[2]).to(kv.v.dtype)
                st.allocate_group(f"g{gi}", prompt_len=L, x0=50 + gi, last_prompt_token=3, max_new_tokens=64,
                                  ignore_eos=True, eos_ids=[], parent_row=row)
                st.bt.free_parent_row(row)
    # wire the emulated ranks: "peer address" of a tensor = address of the same attribute on that rank
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    comm = [torch.zeros(ParticleParallel.comm_bytes_needed(R, groups, n_local), dtype=torch.uint8, device=dev)
            for _ in range(R)]
    pps = []
    for r, (st, kvs) in enumerate(nat):
        table = {}
        for q, (st_q, kvs_q) in enumerate(nat):
            names = [("st", f, getattr(st, f), getattr(st_q, f)) for f in
                     ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished", "finished_len", "finish_code",
                      "matched_eos", "all_token_ids", "group_to_slots")]
            names.append(("bt", "table", st.bt.table, st_q.bt.table))
            for a, b in zip(kvs, kvs_q):
                names += [("kv", "k", a.k, b.k), ("kv", "v", a.v, b.v)]
            for a, b in zip(st.state_pools, st_q.state_pools):
                names += [("sp", "c", a.conv, b.conv), ("sp", "t", a.temporal, b.temporal)]
            for _, _, mine, theirs in names:
                table[(q, mine.data_ptr())] = theirs.data_ptr()
        st.native.bind(st)
        st.native.sync_membership(st)
        pps.append(ParticleParallel(st, st.native, kvs, r, R, lambda q, t, table=table: table[(q, t.data_ptr())],
                                    [c.data_ptr() for c in comm], comm[r], status))
    n_cross = 0
    for cyc in range(1, 6):
        outs = []
        for r in range(R):
            (sn, kn), (sr, kr) = nat[r], ref[r]
            cn, cr = sn.prepare_cycle(), sr.prepare_cycle()
            assert torch.equal(cn.orig_seq_lens, cr.orig_seq_lens)
            bs = cn.slots.numel()
            # KV rows of the new tokens: unique per (rank, slot, position) so a wrong copy is visible
            for (cin, kvs_) in ((cn, kn), (cr, kr)):
                for kv in kvs_:
                    val = (cin.orig_seq_lens.view(bs, 1) + torch.arange(G, device=dev).view(1, G)).float() \
                          + 1000.0 * (r + 1) + 10.0 * cin.slots.view(bs, 1).float()
                    rows = val.reshape(-1, 1).expand(bs * G, kv.k.shape[2])
                    kv.k[:, cin.cache_locs.reshape(-1).long()] = rows.to(kv.k.dtype)
                    kv.v[:, cin.cache_locs.reshape(-1).long()] = (rows + 0.5).to(kv.v.dtype)
            for st_ in (sn, sr):
                for pool in st_.state_pools:
                    sl = cn.slots.long()
                    pool.conv[:, sl] = float(cyc * 10 + r) + sl.view(1, -1, 1, 1).float()
                    pool.temporal[:, sl] = float(cyc * 100 + r) + sl.view(1, -1, 1, 1, 1).float()
            tokens = torch.randint(5, 90, (bs, G), generator=gen, device=dev, dtype=torch.int32)
            diff = torch.randn(bs, gamma, generator=gen, device=dev) * 3.0
            out = CycleOutputs(tokens, diff, None)
            sn.write_back(cn, out)
            sr.write_back(cr, out)
        torch.cuda.synchronize()
        # reference plan over the gathered weights, executed in plain PyTorch
        for gi in range(groups):
            row = ref[0][0].group_rows[f"g{gi}"]
            ws = [st.interval_weights[torch.tensor(st.row_slots[row], device=dev)] for st, _ in ref]
            go, jobs, inc = plan_global(ws, 0.9, 7, cyc, row)
            if go:
                n_cross += sum(1 for j in jobs if j[0] != j[2])
                apply_reference([s for s, _ in ref], [k for _, k in ref], jobs, row)
                for st, _ in ref:
                    idx = torch.tensor(st.row_slots[row], device=dev)
                    st.interval_weights[idx] = 0.0
                    st.log_weights[idx] = 0.0
                    st.group_log_Z[row] += inc
        # kernels, phase by phase across the emulated ranks
        for pp in pps:
            pp.share()
        for pp in pps:
            pp.collect_and_apply(phase=1)
        for pp in pps:
            pp.collect_and_apply(phase=2)
        for pp in pps:
            pp.barrier(phase=1)
        for pp in pps:
            pp.barrier(phase=2)
        torch.cuda.synchronize()
        assert int(status) == 0
        for r in range(R):
            (sn, kn), (sr, kr) = nat[r], ref[r]
            for f in ("seq_lens", "token_counts", "verified_ids", "prev_ids", "finished", "finished_len"):
                assert torch.equal(getattr(sn, f), getattr(sr, f)), (cyc, r, f)
            assert torch.equal(sn.all_token_ids, sr.all_token_ids)
            assert torch.allclose(sn.interval_weights, sr.interval_weights, atol=1e-6)
            assert torch.allclose(sn.group_log_Z, sr.group_log_Z, atol=1e-6)
            for s in range(sn.max_slots):
                L = int(sn.seq_lens[s])
                pn, pr_ = sn.bt.table[s, :L].long(), sr.bt.table[s, :L].long()
                for a, b in zip(kn, kr):
                    assert torch.equal(a.k[:, pn], b.k[:, pr_]), (cyc, r, s)
                    assert torch.equal(a.v[:, pn], b.v[:, pr_]), (cyc, r, s)
            for a, b in zip(sn.state_pools, sr.state_pools):
                assert torch.equal(a.conv[:, :sn.max_slots], b.conv[:, :sn.max_slots])
                assert torch.equal(a.temporal[:, :sn.max_slots], b.temporal[:, :sn.max_slots])
            sn.alloc.check_conservation()
            assert sn.alloc.available() == sr.alloc.available()
    assert n_cross > 0, "no cross-rank ancestor was drawn: the test did not exercise the NVLink path"


@pytest.mark.multigpu
def test_cross_rank_resample_real_ranks(tmp_path):
    import json
    import os
    import subprocess
    import sys
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "res.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29544", os.path.join(root, "tests", "mp_pp_check.py"), str(out)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads(out.read_text())
    assert res["ok"] and res["status"] == 0 and res["n_cross"] > 0
