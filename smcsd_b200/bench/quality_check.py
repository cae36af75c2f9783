"""Side-by-side quality check: a handful of fixed prompts through SMC decoding and through plain target sampling
(SMC with one particle and gamma=1 degenerates to sampling from the target), printed for eyeballing
(the reference's scripts/quick_quality_check.py).

    python -m smcsd_b200.bench.quality_check --model M --draft-model D -N 8 -g 8
"""
from __future__ import annotations

import argparse

from ..config import EngineArgs

PROMPTS = [
    "Explain why the sky is blue in two sentences.",
    "Write a Python function that returns the n-th Fibonacci number.",
    "What is 17 * 23? Show the steps.",
    "Summarize the plot of Romeo and Juliet in one paragraph.",
    "List three differences between TCP and UDP.",
]


def main(argv=None) -> None:
    p = argparse.ArgumentParser("quality_check")
    EngineArgs.add_cli_args(p)
    p.add_argument("--max-new-tokens", type=int, default=128)
    ns = p.parse_args(argv)
    from ..http_server import build_engine_from_args
    sp = {"max_new_tokens": ns.max_new_tokens}
    smc = build_engine_from_args(ns)
    smc_out = smc.generate(prompt=PROMPTS, sampling_params=sp)
    smc.shutdown()
    ns.n_particles, ns.gamma, ns.resample_threshold = 1, 1, 0.0
    base = build_engine_from_args(ns)
    base_out = base.generate(prompt=PROMPTS, sampling_params=sp)
    base.shutdown()
    for q, a, b in zip(PROMPTS, base_out, smc_out):
        print("=" * 100)
        print("PROMPT :", q)
        print("-" * 100)
        print("TARGET :", a["text"])
        print("-" * 100)
        print(f"SMC    : {b['text']}\n         (log Z_hat = {b.get('smc_log_Z_hat')})")


if __name__ == "__main__":
    main()
