"""GSM8K accuracy through the HTTP server: launches ``python -m smcsd_b200.http_server``, polls ``/health``,
sends concurrent ``/generate`` requests, reads ``/server_info`` and applies optional thresholds to the exit code
(the reference's scripts/accuracy_test_gsm8k_http.py:129-166,208-278,380-391).

    python -m smcsd_b200.bench.accuracy_gsm8k_http --model M --draft-model D --data gsm8k_test.jsonl --parallel 16
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import json
import subprocess
import sys
import time

import requests

from .accuracy_gsm8k import INSTRUCTION, gold_answer, load_questions, score


def wait_healthy(base: str, proc, timeout: float) -> None:
    t0 = time.time()
    while time.time() - t0 < timeout:
        if proc.poll() is not None:
            raise RuntimeError(f"server exited with code {proc.returncode}")
        try:
            if requests.get(base + "/health", timeout=2).status_code == 200:
                return
        except requests.RequestException:
            pass
        time.sleep(1.0)
    raise TimeoutError("server did not become healthy")


def main(argv=None) -> None:
    p = argparse.ArgumentParser("accuracy_gsm8k_http")
    p.add_argument("--model", required=True)
    p.add_argument("--draft-model", required=True)
    p.add_argument("--data", required=True)
    p.add_argument("--num-questions", type=int, default=200)
    p.add_argument("--max-new-tokens", type=int, default=512)
    p.add_argument("--parallel", type=int, default=16)
    p.add_argument("--port", type=int, default=30000)
    p.add_argument("-N", "--smc-n-particles", type=int, default=8)
    p.add_argument("-g", "--smc-gamma", type=int, default=8)
    p.add_argument("--server-timeout", type=float, default=1800)
    p.add_argument("--min-accuracy", type=float, default=None)
    p.add_argument("--min-throughput", type=float, default=None)
    p.add_argument("server_args", nargs="*", help="extra flags passed to the server after --")
    ns = p.parse_args(argv)
    base = f"http://127.0.0.1:{ns.port}"
    cmd = [sys.executable, "-m", "smcsd_b200.http_server", "--model", ns.model, "--draft-model", ns.draft_model,
           "-N", str(ns.smc_n_particles), "-g", str(ns.smc_gamma), "--port", str(ns.port),
           "--max-running-requests", str(ns.parallel)] + list(ns.server_args)
    proc = subprocess.Popen(cmd)
    try:
        wait_healthy(base, proc, ns.server_timeout)
        qs = load_questions(ns.data, ns.num_questions)
        golds = [gold_answer(q["answer"]) for q in qs]

        def ask(q):
            r = requests.post(base + "/generate", json={"text": INSTRUCTION + q["question"] + "\n",
                                                        "sampling_params": {"max_new_tokens": ns.max_new_tokens}},
                              timeout=3600)
            r.raise_for_status()
            j = r.json()
            return j["text"], j["meta_info"]["completion_tokens"]
        t0 = time.perf_counter()
        with cf.ThreadPoolExecutor(ns.parallel) as ex:
            res = list(ex.map(ask, qs))
        dt = time.perf_counter() - t0
        acc, inv = score([t for t, _ in res], golds)
        tps = sum(n for _, n in res) / dt
        info = requests.get(base + "/server_info", timeout=10).json()
        print(json.dumps({"accuracy": acc, "invalid": inv, "output_tok_per_s": tps, "latency_s": dt,
                          "server": {"smc": info.get("smc"), "stats": info.get("stats")}}))
        bad = (ns.min_accuracy is not None and acc < ns.min_accuracy) or \
              (ns.min_throughput is not None and tps < ns.min_throughput)
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
    if bad:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
