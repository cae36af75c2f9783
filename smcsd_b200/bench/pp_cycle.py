"""Particle-parallel decode cycle on the ranks of a torchrun job: the particles of one request are sharded over the
GPUs, every rank runs full draft + target forwards for its share, and resampling moves ancestors' KV rows across
NVLink inside the cycle (in-kernel peer loads).  Resampling is forced every cycle (threshold 1.0), so the number
reported includes the cross-GPU copies.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29541 \
        -m smcsd_b200.bench.pp_cycle --steps 20 --warmup 5

The time is CUDA events around ``--steps`` decode cycles on every rank, maximum over ranks.  The reference has no
counterpart (all particles of a group live on one GPU: smcsd/core/kernels/fused_resample_kv.py:98-105).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def run(steps: int = 20, warmup: int = 5, particles_per_rank: int = 2, gamma: int = 8, prompt_len: int = 256,
        target: str = "llama-3.1-8b", draft: str = "llama-3.2-1b", layers: int = 0) -> dict:
    """Needs an initialised NCCL default group (one rank per GPU).  Returns the same record on every rank."""
    import dataclasses

    from ..config import EngineArgs
    from ..io_types import GenerateRequest, SamplingParams
    from ..models.config import preset
    from ..parallel.bootstrap import Comm
    from ..runtime.scheduler import SMCScheduler
    from ..utils.prompts import random_prompts
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    G = gamma + 1
    new_tokens = (steps + max(warmup, 3) + 6) * G
    tgt, drf = preset(target), preset(draft)
    if layers:
        tgt = dataclasses.replace(tgt, n_layers=layers)
    args = EngineArgs(model_path=tgt, draft_model_path=drf, n_particles=particles_per_rank * world, gamma=gamma,
                      draft_temperature=0.7, target_temperature=0.7, resample_threshold=1.0, max_running_requests=1,
                      pp_size=world, base_gpu_id=0, context_length=prompt_len + new_tokens + 4 * G, backend="native",
                      mem_fraction_static=0.3, random_seed=11).finalize()
    comm = Comm.from_env(args, group_size=world)
    sched = SMCScheduler(args, pp_rank=rank, pp_size=world, comm=comm, local_rank=local)
    prompt = random_prompts([prompt_len], sched.target.cfg.vocab_size, seed=5)[0]
    sched.add_request(GenerateRequest("pp", prompt, SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)))
    sched.step()
    for _ in range(max(warmup, 3)):
        sched.step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        sched.step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    st = sched.state
    remote_jobs = int(st.counters[3].item())          # cross-GPU ancestor copies of the last cycle on this rank
    suffix = (steps + max(warmup, 3) + 1) * G          # rows past the (replicated) prompt that such a copy moves
    row_bytes = sum(kv.k.shape[0] * kv.k.shape[2] * kv.k.element_size() * 2 for kv in (sched.kv_t, sched.kv_d))
    status = sched.native_runner.check_status() if sched.native_runner else 0
    t = torch.tensor([ms, float(remote_jobs), float(status)], device="cuda", dtype=torch.float64)
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    tsum = t.clone()
    dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    sched.abort("pp")
    sched.step()
    torch.cuda.synchronize()
    dist.barrier()
    res = {"bench": "pp_cycle", "ranks": world, "n_particles": particles_per_rank * world, "gamma": gamma,
           "model": f"{tgt.name}+{drf.name}", "target_layers": tgt.n_layers, "pp_cycle_ms": float(tmax[0].item()),
           "tokens_per_s": G / (float(tmax[0].item()) / 1e3),
           "remote_copies_last_cycle": int(tsum[1].item()),
           "pp_nvlink_bytes_per_cycle": int(tsum[1].item()) * suffix * row_bytes,
           "status": int(tmax[2].item()), "timing": "CUDA events around the decode cycles, max over ranks"}
    del sched
    torch.cuda.empty_cache()
    return res


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--particles-per-rank", type=int, default=2)
    ap.add_argument("--layers", type=int, default=0, help="shrink the target (smoke runs only)")
    ns = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    res = run(ns.steps, ns.warmup, ns.particles_per_rank, layers=ns.layers)
    if int(os.environ["RANK"]) == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
