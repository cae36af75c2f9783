"""Times one model forward (+ lm_head and sampling) of the persistent kernel against the one-kernel-per-step chain,
and prints the persistent kernel's phase timeline.

    python -m smcsd_b200.ops.bench_forward --model llama-3.2-1b --bs 8 --E 1 --ctx 700
    python -m smcsd_b200.ops.bench_forward --model llama-3.1-8b --bs 8 --E 9 --ctx 700 --layers 8

Both arms run inside CUDA graphs and are timed with CUDA events over ``--reps`` replays; weights are larger than L2
(full models) so every replay streams them from HBM.  ``--layers`` shrinks the model for profiler captures.
"""
from __future__ import annotations

import argparse
import dataclasses
import json

import torch


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.2-1b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--bs", type=int, default=8)
    ap.add_argument("--E", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=700)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--no-chain", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly (for profiler captures of single launches)")
    ap.add_argument("--detail", type=int, default=-1, help="with --trace: per-CTA stamps of this phase index")
    ap.add_argument("--trace", action="store_true", help="print the per-phase timeline of the last persistent launch")
    ns = ap.parse_args(argv)
    from ..memory.pools import KVPool, KVSpec
    from ..models.config import preset
    from ..models.llama import LlamaModel
    from ..ops import native as K
    from ..ops.bench_kernels import peaks
    from ..ops.native_backend import NativeLlama
    from ..ops.native_forward import PersistentLlama
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = preset(ns.model)
    if ns.layers:
        cfg = dataclasses.replace(cfg, n_layers=ns.layers)
    bs, E, P = ns.bs, ns.E, ns.ctx
    T = bs * E
    m = LlamaModel(cfg, torch.bfloat16, dev).init_random(3)
    n_pages = bs * (P + E) + 8
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
    counters = torch.zeros(4, dtype=torch.int64, device=dev)
    tok = torch.zeros(T, dtype=torch.int32, device=dev)
    lp = torch.zeros(T, dtype=torch.float32, device=dev)
    lz = torch.zeros(T, dtype=torch.float32, device=dev)
    given = torch.full((T,), -1, dtype=torch.int32, device=dev)
    if E > 2:          # verify shape: score the drafted tokens, sample the bonus row
        given.view(bs, E)[:, :-1] = 17
    lm_rows, lm_off, lm_step = (bs, E - 1, E) if E <= 2 else (T, 0, 1)
    tin = given[:lm_rows] if E > 2 else None

    def timed(fn):
        torch.cuda.synchronize()
        fn()
        torch.cuda.synchronize()
        if ns.no_graph:
            runner = fn
        else:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            runner = gr.replay
        for _ in range(3):
            runner()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(ns.reps):
            runner()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / ns.reps * 1e3

    pf = PersistentLlama(m, kv, bt, 128, status)
    pf.set_context(P + E, bs, (E,))
    if ns.trace:
        pf.enable_trace()
    pf_us = timed(lambda: pf.run(ids, pos, locs, rows, pref, bs, E, lm_rows=lm_rows, lm_off=lm_off, lm_step=lm_step,
                                 temperature=0.7, alpha=1.0, tokens_in=tin, seed=5, cycle_counter=counters, call_id=1,
                                 tok_out=tok, logp_out=lp, logz_out=lz))
    chain_us = None
    if not ns.no_chain:
        nm = NativeLlama(m, kv, bt, T, T, 8, status, True)
        nm.set_context(P + E, bs, (E,))
        scratch = torch.empty(K.sample_scratch_bytes(T, 32), dtype=torch.uint8, device=dev)

        def chain():
            nm.forward(ids, pos, locs, rows, pref, bs, E)
            nm.lm_head(lm_rows, row_offset=lm_off, row_step=lm_step)
            K.sample_or_score(nm.logits, rows=lm_rows, V=cfg.vocab_size, splits=1, split_stride=0,
                              row_stride=nm.logits.stride(0), temperature=0.7, alpha=1.0, softcap=0.0, tokens_in=tin,
                              seed=5, cycle_counter=counters, call_id=1, scratch=scratch, nchunks=32, tok_out=tok,
                              logp_out=lp, logz_out=lz, pdl=True)
        chain_us = timed(chain)
    wbytes = sum(t.numel() * 2 for L in m.layers for t in (L.wqkv, L.wo, L.wgu, L.wdown)) + m.lm_head.numel() * 2
    hbm, _, src = peaks()
    res = {"bench": "forward", "model": cfg.name, "layers": cfg.n_layers, "bs": bs, "E": E, "ctx": P,
           "persistent_us": pf_us, "chain_us": chain_us, "weight_MB": wbytes / 1e6,
           "floor_us": wbytes / (hbm * 1e3), "persistent_fraction_of_floor": wbytes / (hbm * 1e3) / pf_us,
           "peaks": src, "device_status": int(status.item()), "stages": pf.plan(E, pf.bn_for(T))[4],
           "kv_splits": pf.kv_splits(bs, E, P + E)}
    print(json.dumps(res))
    if ns.trace:
        tr = pf.trace.cpu()[: pf.n_phases(lm_rows)].double()
        t0 = tr[0, :, 0].min()
        names = ["embed"] + ["qkv", "attn", "o", "gu", "down"] * cfg.n_layers + ["lm_head", "merge"]
        rows_out = []
        prev_done = None
        for ph in range(tr.shape[0]):
            op, dn = tr[ph, :, 0], tr[ph, :, 1]
            rows_out.append({"ph": ph, "name": names[ph], "open_first_us": float((op.min() - t0) / 1e3),
                             "open_last_us": float((op.max() - t0) / 1e3), "done_first_us": float((dn.min() - t0) / 1e3),
                             "done_last_us": float((dn.max() - t0) / 1e3),
                             "gap_after_prev_us": None if prev_done is None else float((op.min() - prev_done) / 1e3)})
            prev_done = dn.max()
        show = rows_out[:12] + rows_out[-8:] if len(rows_out) > 22 else rows_out
        for r in show:
            print(json.dumps(r))
        import collections
        agg = collections.defaultdict(list)
        for r in rows_out:
            agg[r["name"]].append(r["done_last_us"] - r["open_first_us"])
        if ns.detail >= 0:
            ph = ns.detail
            t_open = tr[ph, :, 0].min()
            for c in range(tr.shape[1]):
                print(json.dumps({"cta": c, **{k: (float((tr[ph, c, i] - t_open) / 1e3) if tr[ph, c, i] > 0 else None)
                                               for i, k in enumerate(["open", "done", "acc_full", "pre_atomic",
                                                                      "post_atomic", "fix_loaded", "fix_done"])}}))
        print(json.dumps({"mean_phase_span_us": {k: sum(v) / len(v) for k, v in agg.items()},
                          "total_us": rows_out[-1]["done_last_us"]}))


if __name__ == "__main__":
    main()
