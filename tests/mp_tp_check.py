"""Worker of the multi-GPU tensor-parallel check (launched by torchrun from test_tp_gpu.py).

Every rank builds its weight / KV shard and the symmetric heap, runs the TP kernel chain and the
vocab-parallel sampler over NVLink peer memory, and rank 0 compares with the single-GPU chain on
the unsharded model.  NVLS is switched off by the caller; the kernels use plain peer stores.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(out_path: str) -> None:
    from smcsd_b200.memory.pools import KVPool, KVSpec
    from smcsd_b200.models.config import ModelConfig
    from smcsd_b200.models.llama import LlamaModel
    from smcsd_b200.ops import native as K
    from smcsd_b200.ops.native_backend import NativeLlama
    from smcsd_b200.ops.native_tp import NativeLlamaTP
    from smcsd_b200.parallel.symm import SymmHeap
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    K.tp_lib()
    cfg = ModelConfig(arch="llama", vocab_size=8192, hidden_size=512, n_layers=2, n_heads=8, n_kv_heads=4,
                      head_dim=64, ffn_size=1536, max_position=1024, name="tp-test")
    bs, E, P = 4, 5, 21
    T = bs * E
    n_pages = 512
    torch.manual_seed(0)
    bt = torch.zeros(16, 256, dtype=torch.int32, device=dev)
    perm = (torch.randperm(n_pages, generator=torch.Generator().manual_seed(1)) + 1).to(torch.int32).to(dev)
    for b in range(bs):
        bt[b, :P + E] = perm[b * 40:b * 40 + P + E]
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 8192, (T,), generator=g, dtype=torch.int32).to(dev)
    pos = (torch.arange(E) + P).repeat(bs).to(torch.int32).to(dev)
    locs = bt[:bs, P:P + E].reshape(-1).contiguous()
    rows = torch.arange(bs, dtype=torch.int32, device=dev)
    pref = torch.full((bs,), P, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    kfull = (torch.randn(cfg.n_layers, n_pages + 1, cfg.n_kv_heads * cfg.head_dim, generator=g) * 0.5).bfloat16().to(dev)
    vfull = (torch.randn(cfg.n_layers, n_pages + 1, cfg.n_kv_heads * cfg.head_dim, generator=g) * 0.5).bfloat16().to(dev)
    m = LlamaModel(cfg, torch.bfloat16, dev, tp_rank=rank, tp_size=world).init_random(3)
    kv = KVPool(KVSpec(cfg.n_layers, m.n_kv_heads, cfg.head_dim), n_pages, dev)
    w = m.n_kv_heads * cfg.head_dim
    kv.k.copy_(kfull[:, :, rank * w:(rank + 1) * w])
    kv.v.copy_(vfull[:, :, rank * w:(rank + 1) * w])
    heap = SymmHeap(64 << 20, dev, dist.group.WORLD, rank, world)
    nm = NativeLlamaTP(m, kv, bt, T, T, 8, status, True, heap)
    given = torch.full((T,), -1, dtype=torch.int32, device=dev)
    given[::2] = torch.randint(0, 8192, (len(given[::2]),), generator=g, dtype=torch.int32).to(dev)
    ctr = torch.tensor([5], dtype=torch.int64, device=dev)
    tok = torch.zeros(T, dtype=torch.int32, device=dev)
    lp, lz = torch.zeros(T, device=dev), torch.zeros(T, device=dev)
    times = []
    for it in range(4):                     # several passes: counters and buffers are reused across epochs
        heap.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        nm.forward(ids, pos, locs, rows, pref, bs, E)
        nm.lm_head(T)
        nm.tp_sample(rows=T, temperature=0.7, alpha=1.3, tokens_in=given, seed=42, cycle_counter=ctr, call_id=2,
                     tok_out=tok, logp_out=lp, logz_out=lz)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    shard = nm.logits[:T].clone()
    parts = [torch.empty_like(shard) for _ in range(world)]
    dist.all_gather(parts, shard)
    toks = [torch.empty_like(tok) for _ in range(world)]
    dist.all_gather(toks, tok)
    lps = [torch.empty_like(lp) for _ in range(world)]
    dist.all_gather(lps, lp)
    st = status.clone()
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    if rank == 0:
        full = LlamaModel(cfg, torch.bfloat16, dev).init_random(3)
        kv_full = KVPool(KVSpec(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim), n_pages, dev)
        kv_full.k.copy_(kfull)
        kv_full.v.copy_(vfull)
        status1 = torch.zeros(1, dtype=torch.int32, device=dev)
        ref = NativeLlama(full, kv_full, bt, T, T, 8, status1, False)
        ref.forward(ids, pos, locs, rows, pref, bs, E)
        ref_logits = ref.lm_head(T)[:T].clone()
        got = torch.cat(parts, dim=1)[:, :cfg.vocab_size].contiguous()
        scratch = torch.empty(K.sample_scratch_bytes(T, 32), dtype=torch.uint8, device=dev)
        tok1 = torch.zeros(T, dtype=torch.int32, device=dev)
        lp1, lz1 = torch.zeros(T, device=dev), torch.zeros(T, device=dev)
        K.sample_or_score(got, rows=T, V=cfg.vocab_size, splits=1, split_stride=0, row_stride=cfg.vocab_size,
                          temperature=0.7, alpha=1.3, softcap=0.0, tokens_in=given, seed=42, cycle_counter=ctr,
                          call_id=2, scratch=scratch, nchunks=32, tok_out=tok1, logp_out=lp1, logz_out=lz1)
        torch.cuda.synchronize()
        res = {
            "status": int(st), "logit_err": float((got - ref_logits).abs().max() / ref_logits.abs().max()),
            "tokens_equal": bool(torch.equal(tok1, tok)), "logp_err": float((lp1 - lp).abs().max()),
            "ranks_agree": all(torch.equal(t, toks[0]) for t in toks) and all(torch.equal(x, lps[0]) for x in lps),
            "ms": times, "world": world,
        }
        with open(out_path, "w") as f:
            json.dump(res, f)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
