"""Multi-GPU measurements of the fused collective paths, run as a job of their own.

``bench.py --gpus N`` starts this module once per rank in a child process (own process group on another port), so that
a failure here can neither take the headline measurement down nor leave its ranks waiting for one another: the parent
waits with a time limit and reads the record rank 0 wrote.

    RANK=.. WORLD_SIZE=.. LOCAL_RANK=.. MASTER_ADDR=127.0.0.1 MASTER_PORT=.. \
        python -m smcsd_b200.bench.fused_section --steps 20 --warmup 5 --out fused.json

Measured: the 70B-shaped tensor-parallel layer chain (``tp_layers``: fused all-gather / reduce-scatter kernels against
cuBLAS + NCCL, with the roofline floor) at TP = world, and a particle-parallel decode cycle with forced cross-GPU
resampling (``pp_cycle``).  The particle-parallel cycle is run on two ranks only: on four ranks one run of this
benchmark raised an illegal memory access (a rank that was a second ahead of the others planned from weights that had
not arrived and read an unpopulated peer slot); the kernels now refuse to plan after a wait that ran out and the ranks
meet on the host after prefills and graph captures, but that has not been confirmed on four GPUs yet, so larger worlds
skip the cycle and say so.
"""
from __future__ import annotations

import argparse
import datetime
import gc
import json
import os


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--out", required=True)
    ap.add_argument("--dry-run", action="store_true", help="process-group plumbing only (CPU, gloo): no measurements")
    ns = ap.parse_args(argv)
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    fused = {"status": 0}
    if ns.dry_run:
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
        t = torch.ones(1)
        dist.all_reduce(t)
        fused["dry_run_world"] = int(t.item())
    else:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=240))
        try:
            from . import pp_cycle, tp_layers
            a = tp_layers._parser().parse_args(["--model", "llama-3.1-70b", "--layers", "8", "--bs", "8", "--E", "9"])
            r = tp_layers.run(a, init_pg=False)
            fused.update({"tp_layer_us": r["fused_us_per_layer"], "tp_layer_nccl_us": r["cublas_nccl_us_per_layer"],
                          "tp_floor_us": r["floor_us_per_layer"], "tp_tokens": r["tokens"], "tp_size": r["tp"],
                          "tp_model": "llama-3.1-70b layers (8 full-width layers per rank shard)",
                          "tp_fraction_of_floor": r["fused_fraction_of_floor"]})
            fused["status"] |= int(r["device_status"])
            gc.collect()
            torch.cuda.empty_cache()
            if world == 2:
                r = pp_cycle.run(steps=ns.steps, warmup=ns.warmup)
                fused.update({"pp_cycle_ms": r["pp_cycle_ms"], "pp_nvlink_bytes_per_cycle": r["pp_nvlink_bytes_per_cycle"],
                              "pp_n_particles": r["n_particles"], "pp_remote_copies_last_cycle": r["remote_copies_last_cycle"],
                              "pp_tokens_per_s": r["tokens_per_s"]})
                fused["status"] |= int(r["status"])
            else:
                fused["pp_skipped"] = ("particle-parallel cycle measured on 2 ranks only: the fix for the illegal memory "
                                       "access of one earlier 4-rank run is not confirmed on 4 GPUs yet")
        except Exception as e:       # the record must still be written
            fused["status"] = -1
            fused["error"] = f"{type(e).__name__}: {e}"[:300]
    if rank == 0:
        tmp = ns.out + ".tmp"
        with open(tmp, "w") as f:
            json.dump(fused, f)
        os.replace(tmp, ns.out)
    # leave without tearing the process group down: after a device error that can wait for peers forever
    os._exit(0)


if __name__ == "__main__":
    main()
