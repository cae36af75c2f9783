"""GSM8K accuracy, offline engine: zero-shot ``#### <number>`` prompts through the chat template.

    python -m smcsd_b200.bench.accuracy_gsm8k --model /path/to/Llama-3.1-8B-Instruct --draft-model /path/to/Llama-3.2-1B-Instruct \
        --data /path/to/gsm8k_test.jsonl --num-questions 200 -N 8 -g 8

Reports accuracy, invalid-answer rate and output tok/s (the reference's scripts/accuracy_test_gsm8k.py:101-174,
242-294); ``--mode baseline`` runs plain sampling from the target model instead of SMC.  The dataset is a local JSONL with ``question`` / ``answer`` fields; nothing is downloaded.
"""
from __future__ import annotations

import argparse
import json
import re
import time
from typing import List, Optional

from ..config import EngineArgs

INSTRUCTION = ("Solve the following grade-school math problem. Think step by step, then give the final answer on its "
               "own line in the form '#### <number>'.\n\n")
_NUM = re.compile(r"####\s*\$?(-?[\d,]*\.?\d+)")


def load_questions(path: str, n: int):
    qs = []
    with open(path) as f:
        for line in f:
            if line.strip():
                qs.append(json.loads(line))
            if len(qs) >= n:
                break
    return qs


def gold_answer(ans: str) -> Optional[float]:
    m = _NUM.search(ans)
    return float(m.group(1).replace(",", "")) if m else None


def parse_answer(text: str) -> Optional[float]:
    m = _NUM.findall(text)
    if m:
        try:
            return float(m[-1].replace(",", ""))
        except ValueError:
            return None
    nums = re.findall(r"-?[\d,]*\.?\d+", text)
    try:
        return float(nums[-1].replace(",", "")) if nums else None
    except ValueError:
        return None


def build_prompt(tokenizer, question: str) -> str:
    msg = [{"role": "user", "content": INSTRUCTION + question}]
    if getattr(tokenizer, "chat_template", None):
        return tokenizer.apply_chat_template(msg, tokenize=False, add_generation_prompt=True)
    return INSTRUCTION + question + "\n"


def score(outputs: List[str], golds: List[Optional[float]]):
    correct = invalid = 0
    for text, gold in zip(outputs, golds):
        pred = parse_answer(text)
        if pred is None:
            invalid += 1
        elif gold is not None and abs(pred - gold) < 1e-4:
            correct += 1
    n = max(len(outputs), 1)
    return correct / n, invalid / n


def main(argv=None) -> None:
    p = argparse.ArgumentParser("accuracy_gsm8k")
    EngineArgs.add_cli_args(p)
    p.add_argument("--data", required=True)
    p.add_argument("--num-questions", type=int, default=200)
    p.add_argument("--max-new-tokens", type=int, default=512)
    p.add_argument("--min-accuracy", type=float, default=None)
    p.add_argument("--mode", default="smc_engine", choices=["smc_engine", "baseline"],
                   help="baseline: plain sampling from the target model at --temperature (vanilla arm)")
    p.add_argument("--temperature", type=float, default=0.7, help="sampling temperature of the baseline arm")
    ns = p.parse_args(argv)
    from ..http_server import build_baseline_engine_from_args, build_engine_from_args
    eng = build_engine_from_args(ns) if ns.mode == "smc_engine" else build_baseline_engine_from_args(ns, ns.temperature)
    qs = load_questions(ns.data, ns.num_questions)
    prompts = [build_prompt(eng.tokenizer, q["question"]) for q in qs]
    golds = [gold_answer(q["answer"]) for q in qs]
    t0 = time.perf_counter()
    outs = eng.generate(prompt=prompts, sampling_params={"max_new_tokens": ns.max_new_tokens})
    dt = time.perf_counter() - t0
    acc, inv = score([o["text"] for o in outs], golds)
    toks = sum(o["completion_tokens"] for o in outs)
    print(json.dumps({"mode": ns.mode, "accuracy": acc, "invalid": inv, "num_questions": len(qs), "output_tok_per_s": toks / dt,
                      "latency_s": dt}))
    eng.shutdown()
    if ns.min_accuracy is not None and acc < ns.min_accuracy:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
