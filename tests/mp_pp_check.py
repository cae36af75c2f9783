"""Worker of the multi-GPU particle-parallel check (launched by torchrun).

Each rank owns N_local particles of every group with its own pools inside a symmetric heap, runs a few
synthetic cycles and the particle-parallel resampling kernels over NVLink; every rank then replays the
same cycles with the plain-PyTorch reference over all ranks' states (rebuilt locally from the same
seeds) and compares its own shard."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def make_rank(native, n_local, groups, gamma, dev):
    from smcsd_b200.memory.pools import BlockTable, KVPool, KVSpec, PageAllocator
    from smcsd_b200.ops.native_backend import NativeState
    from smcsd_b200.runtime.slot_state import SlotState
    alloc = PageAllocator(2048, dev)
    bt = BlockTable(groups * n_local, 4, 128, dev)
    ns = NativeState(groups * n_local, gamma, torch.device(dev)) if native else None
    st = SlotState(max_groups=groups, n_particles=n_local, gamma=gamma, max_output_len=128, block_table=bt,
                   allocator=alloc, device=dev, seed=7, resample_threshold=0.9, native=ns)
    kvs = [KVPool(KVSpec(3, 2, 16), 2048, dev), KVPool(KVSpec(2, 1, 8), 2048, dev)]
    return st, kvs


def init_groups(st, kvs, groups, dev):
    for gi in range(groups):
        L = 9 + gi
        row = st.bt.alloc_parent_row()
        pages = st.alloc.alloc(L)
        st.bt.table[row, :L] = pages
        for kv in kvs:
            base = torch.arange(L, device=dev).float().view(1, L, 1) + 100 * gi
            kv.k[:, pages.long()] = (base + 0.25).expand(kv.k.shape[0], L, kv.k.shape[2]).to(kv.k.dtype)
            kv.v[:, pages.long()] = (base + 0.5).expand(kv.v.shape[0], L, kv.v.shape[2]).to(kv.v.dtype)
        st.allocate_group(f"g{gi}", prompt_len=L, x0=50 + gi, last_prompt_token=3, max_new_tokens=64, ignore_eos=True,
                          eos_ids=[], parent_row=row)
        st.bt.free_parent_row(row)


def cycle_inputs(r, cyc, bs, G, gamma, dev):
    g = torch.Generator().manual_seed(1000 * cyc + r)
    tokens = torch.randint(5, 90, (bs, G), generator=g, dtype=torch.int32).to(dev)
    diff = (torch.randn(bs, gamma, generator=g) * 3.0).to(dev)
    return tokens, diff


def fill_new_kv(cin, kvs, r, G, dev):
    bs = cin.slots.numel()
    for kv in kvs:
        val = (cin.orig_seq_lens.view(bs, 1) + torch.arange(G, device=dev).view(1, G)).float() \
              + 1000.0 * (r + 1) + 10.0 * cin.slots.view(bs, 1).float()
        rows = val.reshape(-1, 1).expand(bs * G, kv.k.shape[2])
        kv.k[:, cin.cache_locs.reshape(-1).long()] = rows.to(kv.k.dtype)
        kv.v[:, cin.cache_locs.reshape(-1).long()] = (rows + 0.5).to(kv.v.dtype)


def main(out_path):
    from smcsd_b200.ops import native as K
    from smcsd_b200.parallel.particle_parallel import ParticleParallel, apply_reference, plan_global
    from smcsd_b200.parallel.symm import SymmHeap
    from smcsd_b200.runtime.slot_state import CycleOutputs
    rank, R = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    K.lib()
    n_local, groups, gamma = 2, 2, 3
    G = gamma + 1
    st, kvs = make_rank(True, n_local, groups, gamma, dev)
    heap = SymmHeap(64 << 20, dev, dist.group.WORLD, rank, R)
    # move everything peers must read into the symmetric heap (same order on every rank => same offsets)
    offsets = {}

    def migrate(obj, name):
        t = getattr(obj, name)
        off = heap.alloc(name, t.numel() * t.element_size())
        v = heap.view(off, t.shape, t.dtype)
        v.copy_(t)
        setattr(obj, name, v)
        offsets[v.data_ptr()] = off
    for f in ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished", "finished_len", "finish_code",
              "matched_eos", "all_token_ids", "group_to_slots"):
        migrate(st, f)
    migrate(st.bt, "table")
    for kv in kvs:
        migrate(kv, "k")
        migrate(kv, "v")
    comm_off = heap.alloc("pp_comm", ParticleParallel.comm_bytes_needed(R, groups, n_local))
    comm_local = heap.view(comm_off, (ParticleParallel.comm_bytes_needed(R, groups, n_local),), torch.uint8)
    init_groups(st, kvs, groups, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    st.native.bind(st)
    st.native.sync_membership(st)
    pp = ParticleParallel(st, st.native, kvs, rank, R, lambda q, t: heap.ptrs[q] + offsets[t.data_ptr()],
                          [p + comm_off for p in heap.ptrs], comm_local, status)
    # the reference world (all ranks, plain PyTorch) lives on every process
    ref = [make_rank(False, n_local, groups, gamma, dev) for _ in range(R)]
    for s_, k_ in ref:
        init_groups(s_, k_, groups, dev)
    heap.barrier()
    n_cross, ok = 0, True
    for cyc in range(1, 6):
        cn = st.prepare_cycle()
        fill_new_kv(cn, kvs, rank, G, dev)
        tokens, diff = cycle_inputs(rank, cyc, cn.slots.numel(), G, gamma, dev)
        st.write_back(cn, CycleOutputs(tokens, diff, None))
        pp.resample()
        for r, (sr, kr) in enumerate(ref):
            cr = sr.prepare_cycle()
            fill_new_kv(cr, kr, r, G, dev)
            t2, d2 = cycle_inputs(r, cyc, cr.slots.numel(), G, gamma, dev)
            sr.write_back(cr, CycleOutputs(t2, d2, None))
        for gi in range(groups):
            row = ref[0][0].group_rows[f"g{gi}"]
            ws = [s_.interval_weights[torch.tensor(s_.row_slots[row], device=dev)] for s_, _ in ref]
            go, jobs, inc = plan_global(ws, 0.9, 7, cyc, row)
            if go:
                n_cross += sum(1 for j in jobs if j[0] != j[2])
                apply_reference([s_ for s_, _ in ref], [k_ for _, k_ in ref], jobs, row)
                for s_, _ in ref:
                    idx = torch.tensor(s_.row_slots[row], device=dev)
                    s_.interval_weights[idx] = 0.0
                    s_.log_weights[idx] = 0.0
                    s_.group_log_Z[row] += inc
        torch.cuda.synchronize()
        sr, kr = ref[rank]
        for f in ("seq_lens", "token_counts", "verified_ids", "prev_ids", "finished"):
            ok &= bool(torch.equal(getattr(st, f), getattr(sr, f)))
        ok &= bool(torch.equal(st.all_token_ids, sr.all_token_ids))
        ok &= bool(torch.allclose(st.group_log_Z, sr.group_log_Z, atol=1e-6))
        for s in range(st.max_slots):
            L = int(st.seq_lens[s])
            pn, pr_ = st.bt.table[s, :L].long(), sr.bt.table[s, :L].long()
            for a, b in zip(kvs, kr):
                ok &= bool(torch.equal(a.k[:, pn], b.k[:, pr_])) and bool(torch.equal(a.v[:, pn], b.v[:, pr_]))
        st.alloc.check_conservation()
    flag = torch.tensor([int(ok), int(status), n_cross], device=dev)
    allf = [torch.empty_like(flag) for _ in range(R)]
    dist.all_gather(allf, flag)
    if rank == 0:
        res = {"ok": all(int(f[0]) == 1 for f in allf), "status": max(int(f[1]) for f in allf), "n_cross": int(flag[2])}
        with open(out_path, "w") as f:
            json.dump(res, f)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
