"""Attention step of one layer against context length: the single fused launch and the shared-prefix passes
(rope + KV write, one pass over the prompt keys per group of particles, per-particle pass over the rest).

    python -m smcsd_b200.ops.bench_attention --shape verify --contexts 256,1024,4096,8192,16384,32768
    python -m smcsd_b200.ops.bench_attention --shape decode

Eight particles share a prompt of ``context`` tokens and own ``--suffix`` further tokens each.  Every replay runs
``--layers`` layers with separate K/V pools (so the working set is the layers' K/V, not one pool resident in L2);
times are CUDA events over graph replays, per layer.
"""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="verify", choices=["verify", "decode", "head"])
    ap.add_argument("--contexts", default="256,1024,4096,8192,16384,32768")
    ap.add_argument("--suffix", type=int, default=256)
    ap.add_argument("--particles", type=int, default=8)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--contiguous", action="store_true",
                    help="the prompt sits in consecutive pages (a fresh pool) instead of randomly scattered ones")
    ns = ap.parse_args(argv)
    from ..ops import native as K
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if ns.shape == "verify":
        E, Hq, Hkv, D, NP = 9, 32, 8, 128, 2
    elif ns.shape == "decode":
        E, Hq, Hkv, D, NP = 1, 32, 8, 64, 8
    else:
        E, Hq, Hkv, D, NP = 2, 32, 8, 64, 8
    N, G = ns.particles, Hq // Hkv
    bs, T = N, N * E
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rows_out = []
    for P in [int(x) for x in ns.contexts.split(",")]:
        S = ns.suffix
        n_pages = P + N * (S + E) + 8
        pools = [(torch.randn(n_pages + 1, Hkv * D, device=dev).bfloat16(), torch.randn(n_pages + 1, Hkv * D, device=dev).bfloat16())
                 for _ in range(ns.layers)]
        bt = torch.zeros(bs + 1, P + S + E + 8, dtype=torch.int32, device=dev)
        perm = (torch.randperm(n_pages, device=dev) + 1).to(torch.int32)
        if ns.contiguous:
            perm = (torch.arange(n_pages, device=dev) + 1).to(torch.int32)
        for b in range(bs):
            bt[b, :P] = perm[:P]
            bt[b, P:P + S + E] = perm[P + b * (S + E): P + (b + 1) * (S + E)]
        rows = torch.arange(bs, dtype=torch.int32, device=dev)
        prefix = torch.full((bs,), P + S, dtype=torch.int32, device=dev)
        pos = (torch.arange(E, device=dev) + P + S).repeat(bs).to(torch.int32)
        locs = torch.cat([bt[b, P + S:P + S + E] for b in range(bs)]).contiguous()
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev)
        from ..models.layers import rope_table
        rope = rope_table(D, 10000.0, None, P + S + E + 8, dev)
        out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=dev)
        q = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=dev)
        state = torch.zeros(T, Hq, D + 2, device=dev)
        shared = torch.full((bs,), P, dtype=torch.int32, device=dev)
        rows_g, shared_g = rows[::NP].contiguous(), shared[::NP].contiguous()
        ks1 = K.attn_kv_splits(P + S, bs, Hkv, E, G, D)
        n_mt = (NP * E * G + 15) // 16
        n_kw = max(1, 8 // n_mt)
        ksg = 1
        while ksg < 8 and (bs // NP) * Hkv * ksg * 2 <= 148 and P // (ksg * 2 * 32 * n_kw) >= 2:
            ksg *= 2
        kss = K.attn_kv_splits(S, bs, Hkv, E, G, D)

        def single():
            for k, v in pools:
                K.attention_fused(qkv, pos, locs, rope, k, v, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D,
                                  KS=ks1, scale=D ** -0.5, status=status, pdl=True)

        def cascade():
            for k, v in pools:
                K.rope_kv_write(qkv, 1, 0, pos, locs, rope, q, k, v, M=T, Hq=Hq, Hkv=Hkv, D=D, status=status, pdl=True)
                K.attention_fused(qkv, pos, locs, rope, k, v, bt, rows_g, shared_g, None, bs=bs // NP, E=NP * E, Hq=Hq,
                                  Hkv=Hkv, D=D, KS=ksg, scale=D ** -0.5, status=status, pdl=True, q_in=q, part_out=state,
                                  causal=False)
                K.attention_fused(qkv, pos, locs, rope, k, v, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D,
                                  KS=kss, scale=D ** -0.5, status=status, pdl=True, q_in=q, key_begin=shared, part_in=state)

        # the tcgen05 pass takes all particles of the group at once (its query rows are tiled by 128)
        rows_t, shared_t = rows[::N].contiguous(), shared[::N].contiguous()
        kst = K.attention_tc_splits(bs // N, Hkv, P, N * E * G)
        state_tc = torch.zeros(kst, T, Hq, D + 2, device=dev)

        def cascade_tc():
            # two launches: the group pass rotates the queries itself, the per-particle pass is the ordinary step
            for k, v in pools:
                K.attention_prefix_tc(None, k, v, bt, rows_t, shared_t, state_tc, n_seq=bs // N, E=N * E, T=T, Hq=Hq,
                                      Hkv=Hkv, D=D, KS=kst, scale=D ** -0.5, status=status, qkv=qkv, q_off=0,
                                      positions=pos, rope=rope, pdl=True)
                K.attention_fused(qkv, pos, locs, rope, k, v, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D,
                                  KS=kss, scale=D ** -0.5, status=status, pdl=True, key_begin=shared,
                                  part_in=state_tc, part_in_n=kst, part_in_stride=state_tc.stride(0))

        def group_mma():
            for k, v in pools:
                K.attention_fused(qkv, pos, locs, rope, k, v, bt, rows_g, shared_g, None, bs=bs // NP, E=NP * E, Hq=Hq,
                                  Hkv=Hkv, D=D, KS=ksg, scale=D ** -0.5, status=status, pdl=False, q_in=q, part_out=state,
                                  causal=False)

        def group_tc():
            for k, v in pools:
                K.attention_prefix_tc(q, k, v, bt, rows_t, shared_t, state_tc, n_seq=bs // N, E=N * E, T=T, Hq=Hq,
                                      Hkv=Hkv, D=D, KS=kst, scale=D ** -0.5, status=status)

        def suffix_only():
            for k, v in pools:
                K.attention_fused(qkv, pos, locs, rope, k, v, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D,
                                  KS=kss, scale=D ** -0.5, status=status, pdl=False, q_in=q, key_begin=shared, part_in=state)

        def suffix_self():
            for k, v in pools:
                K.attention_fused(qkv, pos, locs, rope, k, v, bt, rows, prefix, out, bs=bs, E=E, Hq=Hq, Hkv=Hkv, D=D,
                                  KS=kss, scale=D ** -0.5, status=status, pdl=False, key_begin=shared, part_in=state)

        def rope_only():
            for k, v in pools:
                K.rope_kv_write(qkv, 1, 0, pos, locs, rope, q, k, v, M=T, Hq=Hq, Hkv=Hkv, D=D, status=status, pdl=False)

        def timed(fn):
            fn()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            for _ in range(2):
                gr.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(ns.reps):
                gr.replay()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / ns.reps / ns.layers * 1e3

        t1 = timed(single)
        o1 = out.float().clone()
        t2 = timed(cascade)
        err = float((out.float() - o1).abs().max())
        t3 = timed(cascade_tc)
        err_tc = float((out.float() - o1).abs().max())
        t4, t5 = timed(group_mma), timed(group_tc)
        t6, t7, t8 = timed(suffix_only), timed(suffix_self), timed(rope_only)
        trace = torch.zeros(4096, 12, dtype=torch.int64, device=dev)
        k0, v0 = pools[0]
        K.attention_prefix_tc(q, k0, v0, bt, rows_t, shared_t, state_tc, n_seq=bs // N, E=N * E, T=T, Hq=Hq, Hkv=Hkv, D=D,
                              KS=kst, scale=D ** -0.5, status=status, trace=trace)
        torch.cuda.synchronize()
        used = trace[trace[:, 4] > 0].double()
        wait_share = (used[:, [0, 1, 2, 3, 5, 6, 7]] / used[:, 4:5]).mean(0).tolist() if used.numel() else []
        wait_share += (used[:, 8:11] / used[:, 11:12].clamp(min=1)).mean(0).tolist() if used.numel() else []
        wait_share += [float(used[:, 4].mean())] if used.numel() else []
        kv_bytes = (P + N * S) * Hkv * D * 2 * 2
        rows_out.append({"shape": ns.shape, "pages": "consecutive" if ns.contiguous else "scattered", "prompt": P, "suffix": S, "particles": N, "E": E, "single_us": t1,
                         "shared_prefix_us": t2, "speedup": t1 / t2, "shared_prefix_tcgen05_us": t3, "speedup_tcgen05": t1 / t3,
                         "splits_group_tcgen05": kst, "group_pass_us": t4,
                         "group_pass_tcgen05_us": t5, "suffix_pass_us": t6, "suffix_pass_own_rope_us": t7, "rope_kv_write_us": t8,
                         "tcgen05_wait_shares": dict(zip(["scores_ready", "score_load", "p_buffer", "exp_store", "mma_kv",
                                                          "mma_score_buffer", "mma_p", "load_stage_free", "load_issue", "load_landing",
                                                          "softmax_total_cycles"], [round(x, 3) for x in wait_share])), "max_abs_diff_tcgen05": err_tc, "splits_single": ks1, "splits_group": ksg,
                         "splits_suffix": kss, "particles_per_group_pass": NP, "max_abs_diff": err,
                         "unique_kv_MB_per_layer": kv_bytes / 1e6, "status": int(status.item())})
        print(json.dumps(rows_out[-1]))
        del pools


if __name__ == "__main__":
    main()
