"""Throughput sweep over batch sizes and (gamma, n_particles) pairs; writes ``method,gamma,n,tps,b`` CSV rows.

    python -m smcsd_b200.bench.sweep --model preset:llama-3.1-8b --draft-model preset:llama-3.2-1b --out smc_1b_8b.csv
    python -m smcsd_b200.bench.sweep --model preset:llama-3.1-70b --draft-model preset:llama-3.2-1b --tp-size 4 --out smc_1b_70b.csv

Grid of the reference sweeps (scripts/tps_benchmark_scripts/smc_1b_8b_triton.sh:9-39, BENCHMARK_CONFIGS.md):
b in {1,4,8,16}; (gamma,n) in {(8,8),(10,8),(10,6),(12,8),(16,8),(8,6),(8,4),(12,6)}; random 256-token inputs,
512-token outputs, T=0.7, memory fraction 0.60.  Each point runs the offline-throughput harness in a fresh process
and parses its ``Output token throughput`` line.  ``--merge a.csv b.csv`` concatenates result files; ``--method sd``
sweeps the classic speculative-decoding comparison arm (``bench/spec_decode_baseline.py``) over the batch sizes.
"""
from __future__ import annotations

import argparse
import csv
import re
import subprocess
import sys

GRID = [(8, 8), (10, 8), (10, 6), (12, 8), (16, 8), (8, 6), (8, 4), (12, 6)]
BATCHES = [1, 4, 8, 16]


def main(argv=None) -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--model")
    p.add_argument("--draft-model")
    p.add_argument("--tp-size", type=int, default=1)
    p.add_argument("--out", default="sweep.csv")
    p.add_argument("--batches", type=int, nargs="*", default=BATCHES)
    p.add_argument("--input-len", type=int, default=256)
    p.add_argument("--output-len", type=int, default=512)
    p.add_argument("--grid", nargs="*", default=None, help="subset of the (gamma,n) grid, e.g. --grid 8,8 12,8")
    p.add_argument("--merge", nargs="*")
    p.add_argument("--method", default="smc", choices=["smc", "sd"],
                   help="sd: the classic speculative-decoding comparison arm (PyTorch forwards, one draft chain)")
    p.add_argument("--sd-steps", type=int, default=4, help="draft tokens per step of the sd arm")
    ns = p.parse_args(argv)
    if ns.merge:
        rows = []
        for fn in ns.merge:
            with open(fn) as f:
                rows += [r for r in csv.reader(f) if r and r[0] != "method"]
        with open(ns.out, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["method", "gamma", "n", "tps", "b"])
            w.writerows(rows)
        return
    with open(ns.out, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["method", "gamma", "n", "tps", "b"])
        grid = [tuple(int(x) for x in g.split(",")) for g in ns.grid] if ns.grid else GRID
        if ns.method == "sd":
            # rows of the reference's baseline sweep (scripts/tps_benchmark_scripts/sglang_sd_1b_8b_triton_v2.sh:26-40):
            # one configuration per batch size; gamma holds the draft tokens per step, n is 1
            for b in ns.batches:
                cmd = [sys.executable, "-O", "-m", "smcsd_b200.bench.spec_decode_baseline", "--model", ns.model,
                       "--draft-model", ns.draft_model, "--num-prompts", str(b), "--max-running-requests", str(b),
                       "--random-input-len", str(ns.input_len), "--random-output-len", str(ns.output_len),
                       "--num-steps", str(ns.sd_steps), "--temperature", "0.7"]
                r = subprocess.run(cmd, capture_output=True, text=True)
                m = re.search(r"Output token throughput \(tok/s\):\s+([0-9.]+)", r.stdout)
                tps = float(m.group(1)) if m else float("nan")
                w.writerow(["sd", ns.sd_steps, 1, tps, b])
                f.flush()
                print(f"b={b} sd steps={ns.sd_steps}: {tps} tok/s", flush=True)
            return
        for b in ns.batches:
            for gamma, n in grid:
                cmd = [sys.executable, "-O", "-m", "smcsd_b200.bench.offline_throughput", "--model", ns.model,
                       "--draft-model", ns.draft_model, "-N", str(n), "-g", str(gamma), "--smc-draft-temperature", "0.7",
                       "--smc-target-temperature", "0.7", "--num-prompts", str(b), "--max-running-requests", str(b),
                       "--random-input-len", str(ns.input_len), "--random-output-len", str(ns.output_len),
                       "--mem-fraction-static", "0.60", "--tp-size", str(ns.tp_size), "--cuda-graph-max-bs", str(b * n)]
                r = subprocess.run(cmd, capture_output=True, text=True)
                m = re.search(r"Output token throughput \(tok/s\):\s+([0-9.]+)", r.stdout)
                tps = float(m.group(1)) if m else float("nan")
                w.writerow(["smc", gamma, n, tps, b])
                f.flush()
                print(f"b={b} gamma={gamma} n={n}: {tps} tok/s", flush=True)


if __name__ == "__main__":
    main()
