"""Micro-benchmarks of the sm_100a kernels with a roofline read-out.

    python -m smcsd_b200.ops.bench_kernels                       # the standard table (graph-timed)
    python -m smcsd_b200.ops.bench_kernels --only gemm --N 16384 --K 2048 --M 8 --epi swiglu --iters 3 --plain
    python -m smcsd_b200.ops.bench_kernels --only attn --ctx 4096 --bs 8 --E 9 --model 8b

Kernels are timed with CUDA events around CUDA-graph replays of many launches that rotate through
enough distinct weight copies to exceed L2, so reads come from HBM.  ``--plain`` launches a few
iterations eagerly instead (small footprint; the form to put under ``ncu``).  Fractions are of the
measured peaks in ``MEASURED_PEAKS.json`` when present.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import native as K

EPIS = {"store": K.EPI_STORE_F32, "resid": K.EPI_RESID_F32, "swiglu": K.EPI_SWIGLU_BF16, "bf16": K.EPI_BF16}


def peaks():
    """(HBM copy GB/s, bf16 TFLOP/s, "measured" | "fallback"): the machine's measured-peaks record, else the fallback."""
    from ..utils.roofline import measured_peaks
    return measured_peaks()


def time_graph(fn, inner: int, reps: int = 20) -> float:
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())      # the inputs are still being written on the current stream
    with torch.cuda.stream(side):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(inner):
            fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1000.0 / reps / inner


def gemm_case(N, Kd, M, epi, splits, pdl=True, plain=False, iters=3, copies=None):
    dev = "cuda"
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    mb = N * Kd * 2 / 1e6
    copies = copies or max(2, int(400 / mb) + 1)
    if plain:
        copies = 2
    Ws = [(torch.randn(N, Kd, device=dev) * 0.02).bfloat16() for _ in range(copies)]
    X = torch.randn(M, Kd, device=dev).bfloat16()
    if epi == K.EPI_SWIGLU_BF16:
        out, ldo = torch.zeros(M, N // 2, device=dev, dtype=torch.bfloat16), N // 2
    elif epi == K.EPI_BF16:
        out, ldo = torch.zeros(M, N, device=dev, dtype=torch.bfloat16), N
    else:
        out, ldo = torch.zeros(M, N, device=dev), N
    if splits:
        s = splits
    elif epi in (K.EPI_STORE_F32, K.EPI_RESID_F32):
        s = K.gemm_cluster_splits(N, Kd, M)
    elif epi == K.EPI_SWIGLU_BF16:
        s = K.gemm_swiglu_splits(N, Kd, M)
    else:
        s = 1
    idx = [0]

    def fn():
        K.gemm_skinny(Ws[idx[0] % copies], X, out, M=M, splits=s, epi=epi, ldo=ldo, status=st, pdl=pdl)
        idx[0] += 1
    if plain:
        for _ in range(iters):
            fn()
        torch.cuda.synchronize()
        return None
    us = time_graph(fn, copies * 4)
    assert int(st) == 0
    return us, mb, s


def attention_case(ctx, bs, E, Hq, Hkv, D, shared_prefix=True, plain=False, iters=3, layers=8, ks=0):
    """Fused attention step at context ``ctx``: ``bs`` particles, ``E`` new tokens each.  With ``shared_prefix`` the
    particles point at the same prompt pages (one request's group after fan-out); otherwise every row owns its
    pages.  ``layers`` distinct K/V pools are rotated so the pages come from HBM, not L2."""
    dev = "cuda"
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    n_pages = (ctx + E) * bs + 8
    kd = Hkv * D
    pools = [(torch.randn(n_pages + 1, kd, device=dev).bfloat16(), torch.randn(n_pages + 1, kd, device=dev).bfloat16())
             for _ in range(1 if plain else layers)]
    bt = torch.zeros(bs, ctx + E, dtype=torch.int32, device=dev)
    for b in range(bs):
        base = 0 if shared_prefix else b * (ctx + E)
        bt[b, :ctx] = torch.arange(base, base + ctx, dtype=torch.int32, device=dev)
        bt[b, ctx:] = torch.arange(bs * ctx + b * E, bs * ctx + (b + 1) * E, dtype=torch.int32, device=dev) \
            if shared_prefix else torch.arange(base + ctx, base + ctx + E, dtype=torch.int32, device=dev)
    rows = torch.arange(bs, dtype=torch.int32, device=dev)
    prefix = torch.full((bs,), ctx, dtype=torch.int32, device=dev)
    T = bs * E
    pos = (ctx + torch.arange(E, device=dev)).repeat(bs).int()
    locs = torch.stack([bt[b, ctx:ctx + E] for b in range(bs)]).reshape(-1).int().contiguous()
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev)
    rope = torch.randn(ctx + E + 8, D, device=dev)
    out = torch.zeros(T, Hq * D, device=dev, dtype=torch.bfloat16)
    ks = ks or K.attn_kv_splits(ctx, bs, Hkv, E, Hq // Hkv, D)
    pa = torch.zeros(T * Hq * ks * D, device=dev)
    pm = torch.zeros(T * Hq * ks * 2, device=dev)
    idx = [0]

    def fn():
        kp, vp = pools[idx[0] % len(pools)]
        K.attention_fused(qkv, pos, locs, rope, kp, vp, bt, rows, prefix, out, pa, pm, bs=bs, E=E, Hq=Hq,
                          Hkv=Hkv, D=D, KS=ks, scale=D ** -0.5, status=st, pdl=True)
        idx[0] += 1
    if plain:
        for _ in range(iters):
            fn()
        torch.cuda.synchronize()
        return None
    us = time_graph(fn, len(pools) * 4)
    assert int(st) == 0, f"device status {int(st)}"
    uniq = (ctx if shared_prefix else ctx * bs) * kd * 2 * 2 / 1e6       # distinct K+V bytes
    touched = ctx * bs * kd * 2 * 2 / 1e6                                 # bytes requested by all particles
    return us, uniq, touched, ks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, choices=[None, "gemm", "attn"])
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--bs", type=int, default=8)
    ap.add_argument("--E", type=int, default=9)
    ap.add_argument("--model", default="8b", choices=["8b", "1b"])
    ap.add_argument("--private-prefix", action="store_true")
    ap.add_argument("--ks", type=int, default=0, help="attention key-range splits (0 = the engine's choice)")
    ap.add_argument("--N", type=int, default=16384)
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--M", type=int, default=8)
    ap.add_argument("--epi", default="swiglu", choices=list(EPIS))
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--plain", action="store_true")
    args = ap.parse_args()
    K.lib()
    hbm, tf, src = peaks()
    if args.only == "gemm":
        r = gemm_case(args.N, args.K, args.M, EPIS[args.epi], args.splits, plain=args.plain, iters=args.iters)
        if r:
            us, mb, s = r
            print(json.dumps({"kernel": "gemm_skinny", "N": args.N, "K": args.K, "M": args.M, "epi": args.epi,
                              "splits": s, "us": us, "GBps": mb / us * 1e3, f"frac_of_{src}_hbm": mb / us * 1e3 / hbm}))
        return
    if args.only == "attn":
        Hq, Hkv, D = (32, 8, 128) if args.model == "8b" else (32, 8, 64)
        r = attention_case(args.ctx, args.bs, args.E, Hq, Hkv, D, shared_prefix=not args.private_prefix,
                           plain=args.plain, iters=args.iters, ks=args.ks)
        if r:
            us, uniq, touched, ks = r
            print(json.dumps({"kernel": "attn_fused", "model": args.model, "ctx": args.ctx, "bs": args.bs, "E": args.E,
                              "kv_splits": ks,
                              "shared_prefix": not args.private_prefix, "us": us, "unique_kv_MB": uniq,
                              "requested_kv_MB": touched, "requested_GBps": touched / us * 1e3,
                              f"requested_frac_of_{src}_hbm": touched / us * 1e3 / hbm}))
        return
    table = [("1B qkv", 3072, 2048, 8, "store"), ("1B o_proj", 2048, 2048, 8, "resid"),
             ("1B gate_up+swiglu", 16384, 2048, 8, "swiglu"), ("1B down", 2048, 8192, 8, "resid"),
             ("1B lm_head", 128256, 2048, 8, "store"), ("8B qkv", 6144, 4096, 72, "store"),
             ("8B o_proj", 4096, 4096, 72, "resid"), ("8B gate_up+swiglu", 28672, 4096, 72, "swiglu"),
             ("8B down", 4096, 14336, 72, "resid"), ("8B lm_head", 128256, 4096, 72, "store"),
             # batched serving: 8 and 16 requests x 8 particles x 9 verify tokens
             ("8B gate_up M=576", 28672, 4096, 576, "swiglu"), ("8B down M=576", 4096, 14336, 576, "resid"),
             ("8B gate_up M=1152", 28672, 4096, 1152, "swiglu"), ("8B down M=1152", 4096, 14336, 1152, "resid"),
             ("1B gate_up M=128", 16384, 2048, 128, "swiglu"), ("1B down M=128", 2048, 8192, 128, "resid")]
    print(f"peaks ({src}): HBM {hbm:.0f} GB/s, bf16 {tf:.0f} TFLOP/s")
    print(f"{'case':22s} {'MB':>7s} {'splits':>6s} {'us':>8s} {'GB/s':>8s} {'of HBM':>7s} {'TFLOP/s':>8s}")
    for name, N, Kd, M, epi in table:
        us, mb, s = gemm_case(N, Kd, M, EPIS[epi], 0)
        flops = 2.0 * N * Kd * M
        print(f"{name:22s} {mb:7.1f} {s:6d} {us:8.2f} {mb / us * 1e3:8.0f} {mb / us * 1e3 / hbm:7.2f} "
              f"{flops / us / 1e6:8.1f}")
    print(f"{'attention case':34s} {'splits':>6s} {'us':>8s} {'req MB':>8s} {'req GB/s':>9s}")
    cases = []
    for ctx in (256, 512, 1024, 2048, 4096):
        cases.append((f"8B verify E=9 ctx {ctx}", ctx, 8, 9, (32, 8, 128), True))
    for ctx in (256, 1024, 2048, 4096):
        cases.append((f"1B decode E=1 ctx {ctx}", ctx, 8, 1, (32, 8, 64), True))
    cases.append(("8B verify E=9 ctx 4096 private", 4096, 8, 9, (32, 8, 128), False))
    cases.append(("1B decode E=1 ctx 384 bs=128", 384, 128, 1, (32, 8, 64), False))      # 16 requests x 8 particles
    cases.append(("8B verify E=9 ctx 384 bs=128", 384, 128, 9, (32, 8, 128), False))
    for name, ctx, bs, E, dims, shared in cases:
        auto = K.attn_kv_splits(ctx, bs, dims[1], E, dims[0] // dims[1], dims[2])
        for ks in sorted({1, 2, 4, auto} if ctx >= 512 else {1, auto}):
            us, uniq, touched, k2 = attention_case(ctx, bs, E, *dims, shared_prefix=shared, ks=ks)
            print(f"{name:34s} {k2:5d}{'*' if ks == auto else ' '} {us:8.2f} {touched:8.1f} {touched / us * 1e3:9.0f}")
    print("(* = the split count the engine picks for that shape)")


if __name__ == "__main__":
    main()
