"""Profiler harness: runs a workload under ``engine.start_profile`` and waits for the Chrome trace
(``*.trace.json.gz``), like the reference's scripts/smc_profile_engine.py:283-303.

    python -m smcsd_b200.bench.profile_engine --model M --draft-model D -N 8 -g 8 --output-dir /tmp/prof --num-steps 20
"""
from __future__ import annotations

import argparse
import glob
import os
import time

from ..config import EngineArgs
from ..utils.prompts import random_prompts


def main(argv=None) -> None:
    p = argparse.ArgumentParser("profile_engine")
    EngineArgs.add_cli_args(p)
    p.add_argument("--output-dir", default="/tmp/smcsd_b200_profile")
    p.add_argument("--num-steps", type=int, default=None)
    p.add_argument("--activities", nargs="*", default=["CPU", "GPU"])
    p.add_argument("--with-stack", action="store_true")
    p.add_argument("--record-shapes", action="store_true")
    p.add_argument("--num-prompts", type=int, default=2)
    p.add_argument("--input-len", type=int, default=128)
    p.add_argument("--output-len", type=int, default=64)
    ns = p.parse_args(argv)
    from ..http_server import build_engine_from_args
    eng = build_engine_from_args(ns)
    vocab = eng._sched.target.cfg.vocab_size if eng._sched is not None else 32000
    prompts = random_prompts([ns.input_len] * ns.num_prompts, vocab, 3)
    sp = {"max_new_tokens": ns.output_len, "ignore_eos": True}
    eng.generate(input_ids=prompts[:1], sampling_params={"max_new_tokens": 8, "ignore_eos": True})
    before = set(glob.glob(os.path.join(ns.output_dir, "*.trace.json.gz")))
    eng.start_profile(output_dir=ns.output_dir, num_steps=ns.num_steps, activities=ns.activities,
                      with_stack=ns.with_stack, record_shapes=ns.record_shapes)
    eng.generate(input_ids=prompts, sampling_params=sp)
    eng.stop_profile()
    deadline = time.time() + 120
    new = set()
    while time.time() < deadline and not new:
        new = set(glob.glob(os.path.join(ns.output_dir, "*.trace.json.gz"))) - before
        time.sleep(0.5)
    print("traces:", sorted(new))
    eng.shutdown()


if __name__ == "__main__":
    main()
