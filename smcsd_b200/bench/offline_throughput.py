"""Offline throughput benchmark: one timed ``generate`` over a set of prompts.

    python -m smcsd_b200.bench.offline_throughput --model preset:llama-3.1-8b --draft-model preset:llama-3.2-1b \
        -N 8 -g 8 --smc-draft-temperature 0.7 --smc-target-temperature 0.7 \
        --dataset-name random --num-prompts 8 --random-input-len 256 --random-output-len 512 --result-file out.jsonl

Datasets: ``random`` (uniform token ids, fixed or ranged lengths), ``lognormal`` (median 200, sigma 1,
clipped to 4..2048), ``generated-shared-prefix`` (groups of prompts sharing a long prefix), ``file`` (one JSON
list of token ids, or one text prompt with a tokenizer, per line), ``sharegpt`` (a ShareGPT conversation dump given
with ``--dataset-path``: the first human turn is the prompt and the length of the first reply the output budget of
that request, as in the reference harness; without a tokenizer, words are hashed into the vocabulary).  Warm-up: 16 short requests.  Prints
request / input / output / total throughput with the ``Output token throughput (tok/s):`` line that sweep
scripts parse, and appends a JSON line to ``--result-file``.  Timing is wall clock around the whole
``generate`` call (tokenization and prefill included), like the reference harness
(scripts/tps_benchmark_scripts/bench_offline_throughput.py:332-337,390-440); the device-timed number is
``bench.py`` at the repository root.  ``--backend-name engine`` runs the vanilla arm (plain target sampling at
``--temperature`` through the same kernels) for side-by-side numbers.
"""
from __future__ import annotations

import argparse
import json
import time
from typing import List

import torch

from ..config import EngineArgs
from ..utils.prompts import lognormal_lengths, random_prompts


def load_sharegpt(path: str, n: int, vocab: int, tokenizer=None, max_in: int = 2048, max_out: int = 2048):
    """(prompts as token ids, per-request output lengths) from a ShareGPT JSON dump: a list of records with a
    ``conversations`` list of ``{"from": "human" | "gpt", "value": text}`` turns.  Conversations that do not start with
    a human turn followed by a reply, or whose prompt is shorter than 4 tokens, are skipped."""
    import zlib
    with open(path) as f:
        data = json.load(f)

    def encode(text: str) -> List[int]:
        if tokenizer is not None:
            return list(tokenizer.encode(text))
        return [zlib.crc32(w.encode()) % vocab for w in text.split()]      # stable stand-in for preset (random) models
    prompts, outs = [], []
    for rec in data:
        conv = rec.get("conversations") or rec.get("conversation") or []
        if len(conv) < 2 or conv[0].get("from") not in ("human", "user") or not conv[1].get("value"):
            continue
        ids, reply = encode(conv[0].get("value", "")), encode(conv[1]["value"])
        if len(ids) < 4 or len(reply) < 4:
            continue
        prompts.append(ids[:max_in])
        outs.append(min(len(reply), max_out))
        if len(prompts) == n:
            break
    return prompts, outs


def build_prompts(ns, vocab: int) -> List[List[int]]:
    n = ns.num_prompts
    if ns.dataset_name == "random":
        lo = max(1, int(ns.random_input_len * ns.random_range_ratio)) if ns.random_range_ratio < 1 else ns.random_input_len
        g = torch.Generator().manual_seed(ns.seed)
        lens = torch.randint(lo, ns.random_input_len + 1, (n,), generator=g).tolist()
        return random_prompts(lens, vocab, ns.seed)
    if ns.dataset_name == "lognormal":
        return random_prompts(lognormal_lengths(n, seed=ns.seed), vocab, ns.seed)
    if ns.dataset_name == "generated-shared-prefix":
        g = torch.Generator().manual_seed(ns.seed)
        out = []
        per = max(1, n // ns.gsp_num_groups)
        for _ in range(ns.gsp_num_groups):
            prefix = torch.randint(0, vocab, (ns.gsp_system_prompt_len,), generator=g).tolist()
            for _ in range(per):
                out.append(prefix + torch.randint(0, vocab, (ns.gsp_question_len,), generator=g).tolist())
        return out[:n]
    if ns.dataset_name == "file":
        out = []
        with open(ns.dataset_path) as f:
            for line in f:
                line = line.strip()
                if line:
                    out.append(json.loads(line) if line.startswith("[") else line)
        return out[:n]
    raise ValueError(ns.dataset_name)


def main(argv=None) -> None:
    p = argparse.ArgumentParser("offline_throughput")
    EngineArgs.add_cli_args(p)
    p.add_argument("--backend-name", "--bench-backend", dest="backend_name", default="smc_engine",
                   choices=["smc_engine", "engine"],
                   help="smc_engine: SMC speculative decoding; engine: plain sampling from the target (vanilla arm)")
    p.add_argument("--dataset-name", default="random",
                   choices=["random", "lognormal", "generated-shared-prefix", "file", "sharegpt"])
    p.add_argument("--dataset-path", default=None)
    p.add_argument("--num-prompts", type=int, default=8)
    p.add_argument("--random-input-len", type=int, default=256)
    p.add_argument("--random-output-len", type=int, default=512)
    p.add_argument("--random-range-ratio", type=float, default=1.0)
    p.add_argument("--gsp-num-groups", type=int, default=4)
    p.add_argument("--gsp-system-prompt-len", type=int, default=1024)
    p.add_argument("--gsp-question-len", type=int, default=128)
    p.add_argument("--seed", type=int, default=1)
    p.add_argument("--skip-warmup", action="store_true")
    p.add_argument("--result-file", default=None)
    p.add_argument("--temperature", type=float, default=0.7, help="accepted for parity; SMC uses the engine temperatures")
    ns = p.parse_args(argv)
    from ..http_server import build_baseline_engine_from_args, build_engine_from_args
    eng = build_engine_from_args(ns) if ns.backend_name == "smc_engine" else \
        build_baseline_engine_from_args(ns, ns.temperature)
    vocab = eng._sched.target.cfg.vocab_size if eng._sched is not None else 32000
    if ns.dataset_name == "sharegpt":
        if not ns.dataset_path:
            raise SystemExit("--dataset-name sharegpt needs --dataset-path (a ShareGPT JSON dump)")
        prompts, out_lens = load_sharegpt(ns.dataset_path, ns.num_prompts, vocab, getattr(eng, "tokenizer", None))
        sp = [{"max_new_tokens": n, "ignore_eos": True, "temperature": ns.temperature} for n in out_lens]
    else:
        prompts = build_prompts(ns, vocab)
        sp = {"max_new_tokens": ns.random_output_len, "ignore_eos": True, "temperature": ns.temperature}
    key = "prompt" if prompts and isinstance(prompts[0], str) else "input_ids"
    if not ns.skip_warmup:
        warm = random_prompts([min(256, ns.random_input_len)] * min(16, max(1, ns.max_running_requests)), vocab, 99)
        eng.generate(input_ids=warm, sampling_params={"max_new_tokens": 16, "ignore_eos": True})
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate(**{key: prompts}, sampling_params=sp)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_in = sum(o["prompt_tokens"] for o in outs)
    n_out = sum(o["completion_tokens"] for o in outs)
    res = {"backend": ns.backend_name, "num_prompts": len(prompts), "total_latency_s": dt,
           "request_throughput": len(prompts) / dt, "input_throughput": n_in / dt, "output_throughput": n_out / dt,
           "total_throughput": (n_in + n_out) / dt, "n_particles": ns.n_particles, "gamma": ns.gamma,
           "tp_size": ns.tp_size, "dataset": ns.dataset_name}
    print("\n====== Offline Throughput Benchmark Result =======")
    print(f"{'Backend:':40s}{ns.backend_name}")
    print(f"{'Successful requests:':40s}{len(prompts)}")
    print(f"{'Benchmark duration (s):':40s}{dt:.2f}")
    print(f"{'Total input tokens:':40s}{n_in}")
    print(f"{'Total generated tokens:':40s}{n_out}")
    print(f"{'Request throughput (req/s):':40s}{res['request_throughput']:.2f}")
    print(f"{'Input token throughput (tok/s):':40s}{res['input_throughput']:.2f}")
    print(f"{'Output token throughput (tok/s):':40s}{res['output_throughput']:.2f}")
    print(f"{'Total token throughput (tok/s):':40s}{res['total_throughput']:.2f}")
    if ns.result_file:
        with open(ns.result_file, "a") as f:
            f.write(json.dumps(res) + "\n")
    eng.shutdown()


if __name__ == "__main__":
    main()
