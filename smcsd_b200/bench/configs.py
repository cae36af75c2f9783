"""Benchmarks of the multi-GPU serving configurations (synthetic prompts, random-init bf16 weights).

    python -m smcsd_b200.bench.configs --config pp      --gpus 8 --batch 8       # 8B+1B, N=12, particles sharded over ranks
    python -m smcsd_b200.bench.configs --config tp70b   --gpus 8 --batch 16      # 70B target tensor-parallel, 1B draft replicated
    python -m smcsd_b200.bench.configs --config hybrid  --gpus 4 --batch 32      # hybrid GDN target + dense draft, particle-parallel
    python -m smcsd_b200.bench.configs --config dp      --gpus 2 --batch 2       # independent replicas

Each run goes through ``SMCEngine.generate`` with one scheduler process per GPU.  It reports end-to-end output
tokens/s (wall clock around ``generate``, the API process waits for every result) and the device-timed decode
cycle (CUDA events inside every scheduler, ``SMC_TIME_CYCLES=1``; the slowest rank is reported).  ``--layers``
shrinks the models for smoke runs; such a run is labelled ``reduced`` and is not a benchmark number.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import time

from ..models.config import preset
from ..utils.prompts import lognormal_lengths, random_prompts, uniform_lengths


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["pp", "tp70b", "hybrid", "dp"])
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--new-tokens", type=int, default=None)
    ap.add_argument("--layers", type=int, default=0, help="override the target's layer count (smoke runs only)")
    ap.add_argument("--impl", default="native", choices=["native", "torch"])
    ns = ap.parse_args(argv)
    os.environ["SMC_TIME_CYCLES"] = "1"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from ..engine import SMCEngine
    kw = dict(draft_temperature=0.7, target_temperature=0.7, resample_threshold=0.5, backend=ns.impl,
              max_running_requests=ns.batch, mem_fraction_static=0.7)
    if ns.config == "pp":
        tgt, drf = preset("llama-3.1-8b"), preset("llama-3.2-1b")
        n_part = 12 if 12 % ns.gpus == 0 else 2 * ns.gpus
        kw.update(n_particles=n_part, gamma=8, pp_size=ns.gpus)
        lens, new = uniform_lengths(ns.batch, 700, 900, seed=1), ns.new_tokens or 256
    elif ns.config == "tp70b":
        tgt, drf = preset("llama-3.1-70b"), preset("llama-3.2-1b")
        kw.update(n_particles=8, gamma=8, tp_size=ns.gpus)
        lens, new = lognormal_lengths(ns.batch, seed=1), ns.new_tokens or 512
    elif ns.config == "hybrid":
        tgt, drf = preset("hybrid-gdn-target"), preset("hybrid-gdn-draft")
        kw.update(n_particles=8, gamma=8, pp_size=ns.gpus)
        lens, new = [512] * ns.batch, ns.new_tokens or 512
    else:
        tgt, drf = preset("llama-3.1-8b"), preset("llama-3.2-1b")
        kw.update(n_particles=8, gamma=8, dp_size=ns.gpus, max_running_requests=max(1, ns.batch // ns.gpus))
        lens, new = lognormal_lengths(ns.batch, seed=1), ns.new_tokens or 512
    reduced = False
    if ns.layers:
        reduced = True
        tgt = dataclasses.replace(tgt, n_layers=ns.layers,
                                  layer_types=tgt.layer_types[:ns.layers] if tgt.layer_types else None)
    kw["context_length"] = max(lens) + new + 64
    eng = SMCEngine(tgt, drf, **kw)
    prompts = random_prompts(lens, tgt.vocab_size, seed=3)
    sp = {"max_new_tokens": new, "ignore_eos": True}
    eng.generate(input_ids=[p[:32] for p in prompts[:max(1, min(len(prompts), ns.batch))]],
                 sampling_params={"max_new_tokens": 3 * (kw["gamma"] + 1), "ignore_eos": True})
    eng.collective_rpc("cycle_timing", reset=True)
    t0 = time.perf_counter()
    outs = eng.generate(input_ids=prompts, sampling_params=sp)
    dt = time.perf_counter() - t0
    timing = [r.value for r in eng.collective_rpc("cycle_timing")]
    n_out = sum(o["completion_tokens"] for o in outs)
    res = {"config": ns.config, "impl": ns.impl, "n_gpus": ns.gpus, "batch": ns.batch, "n_particles": kw["n_particles"],
           "gamma": kw["gamma"], "target": tgt.name, "target_layers": tgt.n_layers, "draft": drf.name,
           "prompt_len_mean": sum(lens) / len(lens), "new_tokens": new, "reduced": reduced,
           "e2e_output_tok_per_s": n_out / dt, "e2e_seconds": dt, "cycle_timing_leader_ranks": timing,
           "data": "synthetic", "dtype": "bf16", "weights": "random-init"}
    print(json.dumps(res))
    eng.shutdown()


if __name__ == "__main__":
    main()
