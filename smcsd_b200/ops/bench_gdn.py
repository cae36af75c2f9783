"""Gated-DeltaNet prompt pass of one layer: token-by-token kernel against the chunk-parallel tcgen05 kernel.

    python -m smcsd_b200.ops.bench_gdn --rows 32 --tokens 512

Shapes of the hybrid target (16 key / 16 value heads of 128 x 128, conv width 4); CUDA events over ``--reps``
launches after warm-up, conv + SiLU pass included in both arms.
"""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--reps", type=int, default=5)
    ns = ap.parse_args(argv)
    from . import native as K
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Hk = Hv = ns.heads
    dk = dv = 128
    W, eps = 4, 1e-6
    conv_dim = 2 * Hk * dk + Hv * dv
    ldp = conv_dim + Hv * dv + 2 * Hv
    ldp += (-ldp) % 8
    bs, n = ns.rows, ns.tokens
    T = bs * n
    proj = torch.randn(T, ldp, device=dev)
    conv_w = (torch.randn(conv_dim, W, device=dev) * 0.3).bfloat16()
    dt_bias = torch.ones(Hv, device=dev)
    A_log = torch.log(torch.empty(Hv, device=dev).uniform_(0.5, 8.0))
    gnorm_w = torch.ones(dv, device=dev, dtype=torch.bfloat16)
    rows = torch.arange(bs, dtype=torch.int32, device=dev)
    off = (torch.arange(bs, device=dev) * n).to(torch.int32)
    ln = torch.full((bs,), n, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    conv_s = torch.zeros(bs, conv_dim, W - 1, device=dev)
    temp = torch.zeros(bs, Hv, dk, dv, device=dev)
    conv_out = torch.zeros(T, conv_dim, device=dev)
    out = torch.zeros(T, Hv * dv, device=dev, dtype=torch.bfloat16)
    res = {"rows": bs, "tokens_per_row": n, "heads": Hv}
    outs = {}
    for name, chunked in (("token_serial_us", False), ("chunked_tcgen05_us", True)):
        def run():
            K.gdn_step(proj, conv_s, temp, rows, conv_w, dt_bias, A_log, gnorm_w, conv_out, out, bs=bs, E=0, Hk=Hk, Hv=Hv,
                       dk=dk, dv=dv, W=W, eps=eps, tok_off=off, tok_len=ln, chunked=chunked, status=status, max_len=n)
        temp.zero_(); conv_s.zero_()
        run()
        torch.cuda.synchronize()
        outs[name] = out.float().clone()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(ns.reps):
            run()
        b.record()
        torch.cuda.synchronize()
        res[name] = a.elapsed_time(b) / ns.reps * 1e3
    L = K.lib()

    def conv_only():
        K._check(L.smc_gdn_conv(K._p(proj), proj.stride(0), K._p(conv_s), K._p(rows), K._p(conv_w), K._p(conv_out), bs, 0,
                                K._p(off), K._p(ln), conv_dim, W, n, 0, K._stream()), "smc_gdn_conv")
    conv_only()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(ns.reps):
        conv_only()
    b.record()
    torch.cuda.synchronize()
    res["conv_pass_us"] = a.elapsed_time(b) / ns.reps * 1e3
    trace = torch.zeros(10, dtype=torch.int64, device=dev)
    K.gdn_step(proj, conv_s, temp, rows, conv_w, dt_bias, A_log, gnorm_w, conv_out, out, bs=bs, E=0, Hk=Hk, Hv=Hv, dk=dk,
               dv=dv, W=W, eps=eps, tok_off=off, tok_len=ln, chunked=True, status=status, max_len=n, trace=trace)
    torch.cuda.synchronize()
    tot = max(1, int(trace.sum()))
    names = ["operands", "mma_G", "L_local_tiles", "solve", "mma_vw_kc", "kcum_scatter", "mma_D1_out", "vnew_decay",
             "mma_out_state", "outputs"]
    res["chunk_phase_share"] = {k: round(int(v) / tot, 3) for k, v in zip(names, trace.tolist())}
    res["chunk_cycles"] = tot // max(1, (n + 63) // 64)
    res["speedup"] = res["token_serial_us"] / res["chunked_tcgen05_us"]
    res["max_abs_diff_first_pass"] = float((outs["token_serial_us"] - outs["chunked_tcgen05_us"]).abs().max())
    res["status"] = int(status.item())
    print(json.dumps(res))


if __name__ == "__main__":
    main()
