"""Roll-back of the eager cycle that precedes a graph capture, for particle-parallel groups: a cross-GPU adoption in
that cycle refills the destination's released pages with the ancestor's KV rows, so the rows behind every active
slot's post-prompt pages are saved and put back along with the block table."""
import torch


def _state(n_local=2, groups=2, gamma=3):
    from smcsd_b200.memory.pools import BlockTable, KVPool, KVSpec, PageAllocator
    from smcsd_b200.runtime.slot_state import SlotState
    alloc = PageAllocator(512, "cpu")
    bt = BlockTable(groups * n_local, 4, 96, "cpu")
    st = SlotState(max_groups=groups, n_particles=n_local, gamma=gamma, max_output_len=64, block_table=bt,
                   allocator=alloc, device="cpu", seed=3, resample_threshold=0.5)
    kvs = [KVPool(KVSpec(3, 2, 16, dtype=torch.float32), 512, "cpu"),
           KVPool(KVSpec(2, 1, 8, dtype=torch.float32), 512, "cpu")]
    for gi in range(groups):
        L = 7 + gi
        row = bt.alloc_parent_row()
        bt.table[row, :L] = alloc.alloc(L)
        st.allocate_group(f"g{gi}", prompt_len=L, x0=11 + gi, last_prompt_token=3, max_new_tokens=32, ignore_eos=True,
                          eos_ids=[], parent_row=row)
        bt.free_parent_row(row)
    return st, kvs


def test_kv_rows_behind_suffix_pages_come_back():
    from smcsd_b200.ops.native_backend import restore_kv_suffix, save_kv_suffix
    st, kvs = _state()
    g = torch.Generator().manual_seed(0)
    # two cycles' worth of tokens past the prompt on every active slot, each on a page of its own
    for s in st.active_slots.tolist():
        P = int(st.prompt_lens[s])
        new = st.alloc.alloc(8)
        st.bt.table[s, P:P + 8] = new
        st.seq_lens[s] = P + 8
    for kv in kvs:
        kv.k.copy_(torch.randn(kv.k.shape, generator=g))
        kv.v.copy_(torch.randn(kv.v.shape, generator=g))
    before = [(kv.k.clone(), kv.v.clone()) for kv in kvs]
    saved = save_kv_suffix(st, kvs)
    pages = saved[0]
    assert pages.numel() == st.active_slots.numel() * 8 and torch.unique(pages).numel() == pages.numel()
    # what an adoption does to a destination: its post-prompt pages are refilled with another particle's rows
    dst = int(st.active_slots[1])
    P, L = int(st.prompt_lens[dst]), int(st.seq_lens[dst])
    hit = st.bt.table[dst, P:L].long()
    for kv in kvs:
        kv.k[:, hit] = -7.0
        kv.v[:, hit] = 9.0
    assert not torch.equal(kvs[0].k, before[0][0])
    restore_kv_suffix(saved, kvs)
    for kv, (k0, v0) in zip(kvs, before):
        assert torch.equal(kv.k, k0) and torch.equal(kv.v, v0)


def test_nothing_to_save_before_the_first_token():
    from smcsd_b200.ops.native_backend import restore_kv_suffix, save_kv_suffix
    st, kvs = _state()
    for s in st.active_slots.tolist():          # sequence lengths still equal the prompt lengths
        st.seq_lens[s] = st.prompt_lens[s]
    assert save_kv_suffix(st, kvs) is None
    restore_kv_suffix(None, kvs)
