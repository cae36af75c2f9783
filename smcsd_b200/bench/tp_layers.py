"""Tensor-parallel layer benchmark: the fused all-gather -> GEMM / GEMM -> reduce-scatter kernel chain against the
same layers on cuBLAS + NCCL, on real ranks (one process per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29533 \
        -m smcsd_b200.bench.tp_layers --model llama-3.1-70b --layers 8 --bs 8 --E 9

Both arms run ``--layers`` full-width decoder layers of the named architecture for ``bs * E`` token rows (a verify
pass), captured in one CUDA graph per arm and timed on the device with CUDA events; the reported time is the
maximum over ranks.  The baseline arm is the usual Megatron layout: column-parallel QKV and gate/up, row-parallel
o-proj and down with an NCCL all-reduce after each, norms and SwiGLU as PyTorch ops, the same attention kernel.
The floor printed next to the results is the slower of (weight bytes per rank / measured HBM copy bandwidth) and
(bytes that must cross NVLink per rank / 770 GB/s).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os

import torch
import torch.distributed as dist


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-70b")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--bs", type=int, default=8)
    ap.add_argument("--E", type=int, default=9)
    ap.add_argument("--ctx", type=int, default=256)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--shard-like", type=int, default=0,
                    help="shrink heads and FFN by this factor (run on one rank to see one shard's chain without peers)")
    ap.add_argument("--stage-times", action="store_true",
                    help="also time every kernel of the fused chain (eager launches with an event after each)")
    return ap


def run(ns, init_pg: bool = True) -> dict:
    """Runs both arms on the ranks of the current torchrun job and returns the result record (the same on every
    rank).  ``ns``: namespace with the fields of ``_parser()``.  With ``init_pg=False`` the caller's default process
    group (NCCL) is used and left alive."""
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from ..memory.pools import KVPool, KVSpec
    from ..models.config import preset
    from ..models.layers import rmsnorm
    from ..models.llama import LlamaModel
    from ..ops import native as K
    from ..ops.bench_kernels import peaks
    from ..ops.native_tp import NativeLlamaTP
    from ..parallel.symm import SymmHeap
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    if init_pg:
        dist.init_process_group("nccl", device_id=dev)
    K.tp_lib()
    cfg = dataclasses.replace(preset(ns.model), n_layers=ns.layers)
    if ns.shard_like > 1:
        cfg = dataclasses.replace(cfg, n_heads=cfg.n_heads // ns.shard_like, n_kv_heads=cfg.n_kv_heads // ns.shard_like,
                                  ffn_size=cfg.ffn_size // ns.shard_like, name=f"{cfg.name}/shard{ns.shard_like}")
    bs, E, P = ns.bs, ns.E, ns.ctx
    T = bs * E
    n_pages = bs * (P + E) + 8
    m = LlamaModel(cfg, torch.bfloat16, dev, tp_rank=rank, tp_size=world).init_random(3)
    kv = KVPool(KVSpec(cfg.n_layers, m.n_kv_heads, cfg.head_dim), n_pages, dev)
    kv.k.normal_(0, 0.5)
    kv.v.normal_(0, 0.5)
    bt = torch.zeros(bs, P + E, dtype=torch.int32, device=dev)
    for b in range(bs):
        bt[b] = torch.arange(1 + b * (P + E), 1 + (b + 1) * (P + E), dtype=torch.int32, device=dev)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=g, dtype=torch.int32).to(dev)
    pos = (torch.arange(E) + P).repeat(bs).to(torch.int32).to(dev)
    locs = bt[:, P:P + E].reshape(-1).contiguous()
    rows = torch.arange(bs, dtype=torch.int32, device=dev)
    pref = torch.full((bs,), P, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    heap = SymmHeap(256 << 20, dev, dist.group.WORLD, rank, world)
    nm = NativeLlamaTP(m, kv, bt, T, T, 8, status, True, heap)
    nm.set_context(P + E, bs)

    def timed(fn):
        """Capture ``fn`` in a graph (after one eager run on a side stream) and time ``reps`` replays."""
        torch.cuda.synchronize()
        dist.barrier()                     # ranks enter together: cross-rank waits in the kernels are bounded
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            fn()
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(ns.reps):
            gr.replay()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / ns.reps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    fused_ms = timed(lambda: nm.forward(ids, pos, locs, rows, pref, bs, E))
    fused_status = int(status.item())

    stage_us = None
    if ns.stage_times:
        names = ["norm+allgather (embed)"] + ["qkv GEMM (AG wait)", "attention", "o-proj GEMM -> RS", "reduce+norm+allgather",
                                             "gate/up GEMM (AG wait)", "down GEMM -> RS", "reduce+norm+allgather"] * ns.layers
        acc = [0.0] * len(names)
        for _ in range(ns.reps):
            torch.cuda.synchronize()
            dist.barrier()
            evs = [torch.cuda.Event(enable_timing=True)]
            evs[0].record()
            for _k in nm.stages(ids, pos, locs, rows, pref, bs, E):
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                evs.append(e)
            torch.cuda.synchronize()
            for i in range(len(names)):
                acc[i] += evs[i].elapsed_time(evs[i + 1]) * 1e3 / ns.reps
        t = torch.tensor(acc, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        acc = t.tolist()
        stage_us = {"norm+allgather (embed)": acc[0]}
        for j in range(7):                  # mean over layers of each of the seven per-layer kernels
            stage_us[names[1 + j]] = stage_us.get(names[1 + j], 0.0) + sum(acc[1 + j::7]) / ns.layers
    # ---- cuBLAS + NCCL arm on the same shards ---------------------------------------------------
    nq, nkv, D, d = m.n_heads, m.n_kv_heads, cfg.head_dim, cfg.hidden_size
    h = torch.zeros(T, d, dtype=torch.float32, device=dev)
    attn = torch.zeros(T, nq * D, dtype=torch.bfloat16, device=dev)
    dummy = torch.zeros(8, device=dev)
    scale = D ** -0.5
    ks = K.attn_kv_splits(P + E, bs, nkv, E, nq // nkv, D)

    def baseline():
        h.copy_(m.embed[ids.long()].float())
        for li, L in enumerate(m.layers):
            xn = rmsnorm(h, L.ln1, cfg.rms_eps).to(torch.bfloat16)
            qkv = (xn @ L.wqkv.t()).float()
            K.attention_fused(qkv, pos, locs, m.rope, kv.k[li], kv.v[li], bt, rows, pref, attn, dummy, dummy, bs=bs,
                              E=E, Hq=nq, Hkv=nkv, D=D, KS=ks, scale=scale, status=status)
            o = (attn @ L.wo.t()).float()
            dist.all_reduce(o)
            h.add_(o)
            xn = rmsnorm(h, L.ln2, cfg.rms_eps).to(torch.bfloat16)
            gu = xn @ L.wgu.t()
            blk = m.gu_block
            gu = gu.view(T, -1, 2, blk)
            act = (torch.nn.functional.silu(gu[:, :, 0].float()) * gu[:, :, 1].float()).to(torch.bfloat16).reshape(T, -1)
            dn = (act @ L.wdown.t()).float()
            dist.all_reduce(dn)
            h.add_(dn)

    base_ms = timed(baseline)
    per_layer_w = sum(t.numel() * 2 for t in (m.layers[0].wqkv, m.layers[0].wo, m.layers[0].wgu, m.layers[0].wdown))
    hbm, _, src = peaks()
    # reduce-scatter: (tp-1)/tp of this rank's fp32 partial rows leave twice per layer; all-gather: (tp-1)/tp of the
    # bf16 rows arrive twice per layer
    link_bytes = 2 * (world - 1) / world * T * d * 4 + 2 * (world - 1) / world * T * d * 2
    floor_us = max(per_layer_w / (hbm * 1e3), link_bytes / (770.0 * 1e3))
    res = ({
            "bench": "tp_layers", "model": cfg.name, "layers": ns.layers, "tp": world, "tokens": T, "context": P,
            "fused_us_per_layer": fused_ms * 1e3 / ns.layers, "cublas_nccl_us_per_layer": base_ms * 1e3 / ns.layers,
            "speedup": base_ms / fused_ms, "floor_us_per_layer": floor_us,
            "fused_fraction_of_floor": floor_us / (fused_ms * 1e3 / ns.layers),
            "weight_MB_per_rank_per_layer": per_layer_w / 1e6, "nvlink_MB_per_rank_per_layer": link_bytes / 1e6,
            "peaks": src, "device_status": fused_status, "fused_stage_us_eager": stage_us,
            "timing": "CUDA events around graph replays, max over ranks"})
    dist.barrier()
    del nm, heap, m, kv
    torch.cuda.empty_cache()
    return res


def main(argv=None) -> None:
    ns = _parser().parse_args(argv)
    res = run(ns, init_pg=True)
    if int(os.environ["RANK"]) == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
