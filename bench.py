#!/usr/bin/env python
"""Headline benchmark: output tokens/s of SMC speculative decoding, Llama-3.1-8B target +
Llama-3.2-1B draft, N=8 particles, gamma=8, T=0.7, one request per GPU (data-parallel replicas),
bf16 random-init weights, synthetic prompts (uniform token ids).

A "step" is one decode cycle: every particle advances gamma+1 = 9 tokens, so each request emits
9 output tokens per step.  ``value`` brackets exactly K replays of the cycle with CUDA events (max
over ranks); ``repeats`` re-times the same K cycles a few more times (median and spread);
``e2e`` times whole ``SMCEngine.generate`` calls in the published shape (256-token prompts, 1024
new tokens: prompt upload from pinned memory, prefill, all cycles, token download) and ``config2``
does the same with log-normal prompt lengths (median 200) and 512 new tokens.  On two or more GPUs
the same job then measures the fused collective paths: a 70B-shaped tensor-parallel layer chain
(kernel-issued all-gather / reduce-scatter against cuBLAS + NCCL) and a particle-parallel decode
cycle with forced cross-GPU resampling, reported under ``fused``.

    python bench.py --gpus 1 --steps 40 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 40 --warmup 5
    python bench.py --impl reference        # prints why the reference cannot run here
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import sys
import time

PUBLISHED_TOKS = 677.0     # reference docs/smc/performance.md:14-16 (1x B200, 256-token prompts, 1024 outputs)


def reference_arm(args) -> int:
    """The reference is a thin layer over a patched SGLang fork that is absent from its tree
    (empty submodule) and from this image, so its stock code path cannot start."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
    why = None
    try:
        import smcsd  # noqa: F401
        why = "reference imported but no runner is wired"
    except Exception as e:  # ModuleNotFoundError: sglang
        why = f"{type(e).__name__}: {e} (smcsd installs, but its SGLang fork submodule is empty and sglang is not on this image)"
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")}))
    return 0


def _e2e(eng, sched, lens, new_tokens, vocab, rank, world, dist, torch, seed):
    """Wall-clock tokens/s of ``generate`` over the given prompts (one untimed request of the same shape first)."""
    from smcsd_b200.utils.prompts import random_prompts
    prompts = random_prompts(lens, vocab, seed=seed + rank)
    sp = {"max_new_tokens": new_tokens, "ignore_eos": True}
    # cycle graphs are captured lazily per (batch, attention split plan): warm them up outside the timed region
    eng.generate(input_ids=random_prompts([max(lens)], vocab, seed=seed + 991 + rank)[0], sampling_params=sp)
    b0 = dict(sched.io_bytes)
    c0 = sched.stats["cycles"]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    n_out = 0
    for p in prompts:
        o = eng.generate(input_ids=p, sampling_params=sp)
        n_out += o["completion_tokens"]
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    tt = torch.tensor([dt], device="cuda", dtype=torch.float64)
    nn = torch.tensor([float(n_out)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dist.all_reduce(nn, op=dist.ReduceOp.SUM)
    cyc = max(sched.stats["cycles"] - c0, 1)
    return {"value": float(nn.item()) / float(tt.item()), "unit": "output tokens/s",
            "h2d_bytes_per_step": (sched.io_bytes["h2d"] - b0["h2d"]) / cyc,
            "d2h_bytes_per_step": (sched.io_bytes["d2h"] - b0["d2h"]) / cyc,
            "requests_per_gpu": len(lens), "new_tokens": new_tokens, "prompt_lens": list(lens),
            "warmup": "one untimed request of the same shape",
            "timing": "wall clock around generate() calls, cuda-synchronized, max over ranks"}


def _run_fused_children(rank: int, steps: int, warm: int, dry_run: bool = False, limit_s: int = 420):
    """Start ``smcsd_b200.bench.fused_section`` for this rank (same RANK / WORLD_SIZE / LOCAL_RANK, next-door port, its
    own store), wait at most ``limit_s`` seconds, stop it by pid on overrun; rank 0 returns the record it wrote."""
    import subprocess
    import tempfile
    env = dict(os.environ)
    env["MASTER_PORT"] = str(int(env.get("MASTER_PORT", "29500")) + 17)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    for k in [k for k in env if k.startswith("TORCHELASTIC_")]:
        env.pop(k)                                   # the child hosts its own rendezvous store
    out = os.path.join(tempfile.gettempdir(), f"smc_fused_{env['MASTER_PORT']}_{os.getppid()}.json")
    if rank == 0 and os.path.exists(out):
        os.remove(out)
    cmd = [sys.executable, "-m", "smcsd_b200.bench.fused_section", "--steps", str(steps), "--warmup", str(warm),
           "--out", out] + (["--dry-run"] if dry_run else [])
    proc = subprocess.Popen(cmd, env=env, cwd=os.path.dirname(os.path.abspath(__file__)),
                            stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    timed_out = False
    try:
        proc.wait(timeout=limit_s)
    except subprocess.TimeoutExpired:
        timed_out = True
        proc.kill()
        proc.wait()
    if rank != 0:
        return None
    if os.path.exists(out):
        with open(out) as f:
            rec = json.load(f)
        os.remove(out)
        return rec
    return {"status": -2, "error": "the fused-collective job " + ("ran past its time limit" if timed_out else
                                                                 f"ended with code {proc.returncode} without a record")}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "torch", "reference"])
    ap.add_argument("--target", default="llama-3.1-8b")
    ap.add_argument("--draft", default="llama-3.2-1b")
    ap.add_argument("-N", "--n-particles", type=int, default=8)
    ap.add_argument("-g", "--gamma", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256,
                    help="prompt length in tokens (the published headline uses 256; 0 = log-normal, median 200)")
    ap.add_argument("--repeats", type=int, default=4, help="extra timed repeats of the K cycles (median / spread)")
    ap.add_argument("--e2e-requests", type=int, default=2)
    ap.add_argument("--e2e-new-tokens", type=int, default=1024, help="the published headline generates 1024")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-config2", action="store_true")
    ap.add_argument("--no-fused", action="store_true", help="skip the multi-GPU fused-collective measurements")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--quantization", default=None, choices=[None, "fp8"],
                    help="run the MAIN measurement with W8A8 projections (the line's dtype says so; not the headline)")
    ap.add_argument("--kv-cache-dtype", default="auto", choices=["auto", "fp8_e4m3"],
                    help="run the MAIN measurement with the e4m3 KV cache (the line's dtype says so; not the headline)")
    ap.add_argument("--no-fp8", action="store_true",
                    help="skip the extra W8A8 (e4m3) measurement reported under the 'fp8' key (one GPU only)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from smcsd_b200 import SMCEngine
    from smcsd_b200.io_types import GenerateRequest, SamplingParams
    from smcsd_b200.ops import native as K
    from smcsd_b200.utils.profiling import ClockSampler
    from smcsd_b200.utils.prompts import lognormal_lengths, random_prompts

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    G = args.gamma + 1
    steps, warm = args.steps, max(args.warmup, 3)
    reps = max(0, args.repeats)
    need_tokens = (steps * (1 + reps) + warm + 4) * G + 1
    new_tokens = max(512, need_tokens)
    sampler = ClockSampler(local).start() if rank == 0 else None      # clocks over the whole benchmark
    eng = SMCEngine(f"preset:{args.target}", f"preset:{args.draft}", n_particles=args.n_particles, gamma=args.gamma,
                    draft_temperature=0.7, target_temperature=0.7, resample_threshold=0.5, max_running_requests=1,
                    base_gpu_id=local, context_length=max(4096, args.prompt_len) + max(new_tokens, args.e2e_new_tokens) + 4 * G,
                    random_seed=rank,
                    backend="native" if args.impl == "native" else "torch", in_process=True,
                    cycle_graph=not args.no_graph, mem_fraction_static=0.6, quantization=args.quantization,
                    kv_cache_dtype=args.kv_cache_dtype)
    sched = eng._sched
    vocab = sched.target.cfg.vocab_size
    lens = [args.prompt_len] if args.prompt_len else lognormal_lengths(1, seed=1000 + rank)
    # bytes a decode cycle cannot avoid reading (weights once per pass, cached keys and values) over the measured copy
    # bandwidth; the context is taken at the middle of the timed region
    try:
        from smcsd_b200.utils.roofline import decode_cycle_floor
        floor = decode_cycle_floor(sched.target.cfg, sched.draft.cfg, args.gamma,
                                   defer_bonus=bool(sched.args.defer_bonus), rows=args.n_particles,
                                   context=lens[0] + (warm + steps // 2) * G, shared_prompt=lens[0])
    except Exception:                 # an explanatory key must never cost the measurement
        floor = None
    prompt = random_prompts(lens, vocab, seed=rank)[0]

    # ---- device-timed region: K decode cycles of one live request ------------------------------
    sched.add_request(GenerateRequest("bench", prompt, SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)))
    sched.step()                      # prefill + fan-out
    if not sched.running:
        raise SystemExit(f"the benchmark request was not admitted: {[getattr(o, 'error', None) for o in sched.outbox]}")
    for _ in range(warm):
        sched.step()

    def timed_cycles() -> float:
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            sched.step()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    l0 = K.launch_count
    ms_max = timed_cycles()
    per_cycle_launches = getattr(sched.native_runner, "launches_per_cycle", 0) if sched.native_runner else 0
    launches = per_cycle_launches * steps if per_cycle_launches else K.launch_count - l0
    more = [timed_cycles() / steps for _ in range(reps)]
    status = sched.native_runner.check_status() if sched.native_runner else 0
    sched.abort("bench")
    sched.step()
    toks = steps * G * world
    value = toks / (ms_max / 1e3)
    all_ms = [ms_max / steps] + more
    repeats = {"ms_per_step": all_ms, "median_ms_per_step": statistics.median(all_ms),
               "min_ms_per_step": min(all_ms), "max_ms_per_step": max(all_ms),
               "note": "first entry is the headline region; the others re-time the same K cycles later in the request"}

    # ---- end to end through SMCEngine.generate ---------------------------------------------------
    e2e = config2 = None
    if not args.no_e2e:
        n_req = args.e2e_requests
        lens2 = [args.prompt_len] * n_req if args.prompt_len else lognormal_lengths(n_req, seed=2000 + rank)
        e2e = _e2e(eng, sched, lens2, args.e2e_new_tokens, vocab, rank, world, dist, torch, seed=77)
    if not args.no_config2 and not args.no_e2e:
        lens3 = lognormal_lengths(max(2, args.e2e_requests), seed=3000 + rank)
        config2 = _e2e(eng, sched, lens3, 512, vocab, rank, world, dist, torch, seed=177)
        config2["shape"] = "log-normal prompt lengths (median 200, sigma 1, clipped 4..2048), 512 new tokens"
    status |= sched.native_runner.check_status() if sched.native_runner else 0

    # ---- the same K cycles with quantization='fp8' (labelled, next to the bf16 headline; one GPU only) -------------
    fp8 = None
    if world == 1 and not args.no_fp8 and args.impl == "native" and not args.quantization and args.kv_cache_dtype == "auto":
        try:
            eng.shutdown()
            del eng, sched
            gc.collect()
            torch.cuda.empty_cache()
            eng = SMCEngine(f"preset:{args.target}", f"preset:{args.draft}", n_particles=args.n_particles,
                            gamma=args.gamma, draft_temperature=0.7, target_temperature=0.7, resample_threshold=0.5,
                            max_running_requests=1, base_gpu_id=local,
                            context_length=max(4096, args.prompt_len) + new_tokens + 4 * G, random_seed=rank,
                            backend="native", in_process=True, cycle_graph=not args.no_graph, mem_fraction_static=0.6,
                            quantization="fp8")
            sched = eng._sched
            sched.add_request(GenerateRequest("bench8", prompt, SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)))
            sched.step()
            for _ in range(warm):
                sched.step()
            ms8 = [timed_cycles() / steps for _ in range(3)]
            st8 = sched.native_runner.check_status()
            sched.abort("bench8")
            sched.step()
            fp8 = {"dtype": "fp8 e4m3 weights + per-token e4m3 activations in every projection (W8A8, fp32 accumulate); "
                            "attention, norms, residual stream and lm_head as in the bf16 run",
                   "ms_per_step": ms8[0], "value": G / (ms8[0] / 1e3),
                   "unit": "tokens/s", "all_ms_per_step": ms8, "device_status": int(st8),
                   "note": "not the headline: reduced-precision variant of the same K device-timed cycles (first region, as the "
                           "headline; the target's projections are quantised, the draft stays bf16)"}
        except Exception as e:       # the headline line must still be printed
            fp8 = {"error": f"{type(e).__name__}: {e}"[:300]}

    # ---- fused collective paths (two or more GPUs) ----------------------------------------------------
    # Run as child processes with a process group of their own and a time limit: a failure there cannot take this
    # job's line down or leave its ranks waiting for one another.
    fused = None
    if world > 1 and not args.no_fused and args.impl == "native":
        eng.shutdown()
        del eng, sched
        gc.collect()
        torch.cuda.empty_cache()
        fused = _run_fused_children(rank, steps, warm)
        dist.barrier()
    clocks = sampler.stop() if sampler else None

    if rank == 0:
        e2e_ratio = (e2e["value"] / (PUBLISHED_TOKS * world)) if e2e else None
        line = {
            "metric": "output tokens/s (Llama-3.1-8B target + Llama-3.2-1B draft, SMC N=8 gamma=8)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": ms_max / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": e2e_ratio if e2e_ratio is not None else value / (PUBLISHED_TOKS * world),
            "vs_baseline_device_timed": value / (PUBLISHED_TOKS * world),
            "dtype": "bf16" + (" + e4m3 W8A8 projections of the target" if args.quantization else "") +
                     (" + e4m3 KV cache" if args.kv_cache_dtype != "auto" else ""),
            "data": "synthetic", "impl": args.impl,
            "config": {"model": f"{args.target}+{args.draft}", "global_batch": world, "seq_len": lens[0],
                       "parallelism": f"dp{world}", "n_particles": args.n_particles, "gamma": args.gamma,
                       "tokens_per_step_per_request": G, "cycle_graph": not args.no_graph,
                       "l2": "inputs larger than L2: every step streams 16 GB of target and 8 x 2.5 GB of draft weights",
                       "weights": "random-init bf16 from a seed", "vs_baseline_note":
                       "vs_baseline = end-to-end tokens/s (e2e.value) over the published 677 tok/s per GPU (wall clock, "
                       "same 256-in / 1024-out shape); vs_baseline_device_timed divides the device-timed decode rate "
                       "by the same figure"},
            "clocks": clocks, "repeats": repeats, "e2e": e2e, "config2": config2, "fused": fused, "fp8": fp8,
            "gpu_launches": int(launches), "device_status": int(status),
        }
        if floor is not None and not args.quantization and args.kv_cache_dtype == "auto":
            line["roofline"] = {"floor_ms": floor["floor_ms"], "fraction_of_floor": floor["floor_ms"] / (ms_max / steps),
                                "weight_gb_per_cycle": floor["weight_bytes"] / 1e9, "kv_gb_per_cycle": floor["kv_bytes"] / 1e9,
                                "hbm_gbs": floor["hbm_gbs"], "peaks": floor["peaks"],
                                "note": "floor = bytes one cycle must read from HBM / copy bandwidth (of " +
                                        floor["peaks"] + "); fraction = floor / device-timed ms per cycle"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
