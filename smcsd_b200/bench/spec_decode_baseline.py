"""Classic speculative decoding (draft k tokens, verify, accept by rejection sampling): the comparison arm of the
reference's sweeps, which run it through SGLang's ``STANDALONE`` mode with one draft chain
(scripts/tps_benchmark_scripts/sglang_sd_1b_8b_triton_v2.sh:26-40: ``--speculative-num-steps 4
--speculative-eagle-topk 1 --speculative-num-draft-tokens 5``).

    python -m smcsd_b200.bench.spec_decode_baseline --model preset:llama-3.1-8b --draft-model preset:llama-3.2-1b \
        --num-prompts 8 --num-steps 4 --temperature 0.7

Every step drafts ``k`` tokens with the small model, scores the ``k + 1`` positions with the target in one pass and
accepts the longest prefix by the standard rule (accept d with probability min(1, p(d) / q(d)); the first refused
position is redrawn from the normalised positive part of p - q; a fully accepted chain earns a bonus token from the
target), so the output law is exactly the target's.  It runs on the PyTorch forwards of the two models (dense models
only: a rejected chain would have to roll a recurrent state back) over the same paged KV pools and block table as
the engine; pages are token-granular, so a rejected suffix is simply overwritten by the next step.  It is a
baseline for accept-rate and quality comparisons, not a tuned kernel path.
"""
from __future__ import annotations

import argparse
import json
import time
from typing import Dict, List, Optional, Sequence

import torch

from ..config import EngineArgs
from ..models.layers import ExtendBatch


def accept_chain(p: torch.Tensor, q: torch.Tensor, drafts: Sequence[int], gen: Optional[torch.Generator] = None,
                 greedy: bool = False) -> List[int]:
    """One sequence's accept / redraw step.  ``p`` [k+1, V] target probabilities of the k drafted positions and the
    bonus position, ``q`` [k, V] draft probabilities, ``drafts`` the k drafted tokens.  Returns the tokens to commit
    (accepted prefix plus one redrawn or bonus token)."""
    k = len(drafts)
    out: List[int] = []
    for i in range(k):
        d = int(drafts[i])
        if greedy:
            ok = int(p[i].argmax()) == d
        else:
            u = float(torch.rand((), generator=gen, device=p.device))
            ok = u * float(q[i, d]) < float(p[i, d])         # u < p/q without the division
        if ok:
            out.append(d)
            continue
        if greedy:
            out.append(int(p[i].argmax()))
        else:
            resid = (p[i] - q[i]).clamp_(min=0)
            tot = float(resid.sum())
            resid = resid / tot if tot > 0 else p[i]           # p == q: any draw from p is right
            out.append(int(torch.multinomial(resid, 1, generator=gen)))
        return out
    out.append(int(p[k].argmax()) if greedy else int(torch.multinomial(p[k], 1, generator=gen)))
    return out


class SpecDecodeBaseline:
    """Holds the two models and their pools (built by the engine's scheduler on the PyTorch backend) and decodes
    batches of prompts with draft-and-verify steps."""

    def __init__(self, model, draft_model, num_steps: int = 4, temperature: float = 1.0, max_running_requests: int = 8,
                 **engine_kw):
        from ..runtime.scheduler import SMCScheduler
        t = max(float(temperature), 0.0)
        kw = dict(engine_kw)
        kw.update(n_particles=1, gamma=int(num_steps), draft_temperature=max(t, 1e-5), target_temperature=max(t, 1e-5),
                  backend="torch", max_running_requests=int(max_running_requests), resample_threshold=0.0)
        self.args = EngineArgs(model_path=model, draft_model_path=draft_model, **kw).finalize()
        s = SMCScheduler(self.args)
        if getattr(s.target, "has_state", False) or getattr(s.draft, "has_state", False):
            raise ValueError("the speculative-decoding baseline supports dense models only")
        self.s = s
        self.k = int(num_steps)
        self.T = t
        self.greedy = t < 1e-4
        self.dev = s.device
        self.gen = torch.Generator(device=self.dev)
        self.gen.manual_seed(int(self.args.random_seed) * 7919 + 23)
        self.stats = dict(steps=0, seq_steps=0, drafted=0, accepted=0, committed=0)

    # ------------------------------------------------------------------ model passes
    def _probs(self, logits: torch.Tensor) -> torch.Tensor:
        if self.greedy:
            return torch.nn.functional.one_hot(logits.argmax(-1), logits.shape[-1]).to(torch.float32)
        return torch.softmax(logits.float() / self.T, dim=-1)

    def _extend(self, model, kv, rows: List[int], tokens: List[List[int]], prefix: List[int]) -> torch.Tensor:
        """Run ``E`` new tokens per row at positions prefix..prefix+E-1; returns probabilities [bs, E, V]."""
        bs, E = len(rows), len(tokens[0])
        bt = self.s.bt.table
        ids = torch.tensor(tokens, dtype=torch.int64, device=self.dev).reshape(-1)
        pre = torch.tensor(prefix, dtype=torch.int64, device=self.dev)
        pos = (pre.view(bs, 1) + torch.arange(E, device=self.dev).view(1, E)).reshape(-1)
        r = torch.tensor(rows, dtype=torch.int64, device=self.dev)
        locs = bt[r.view(bs, 1), pos.view(bs, E)].reshape(-1).long()
        b = ExtendBatch(ids, pos, locs, r.to(torch.int32), pre.to(torch.int32), extend_len=E, prefix_lens_host=list(prefix))
        hid = model.forward_torch(b, kv, bt, None)
        return self._probs(model.logits_torch(hid)).view(bs, E, -1)

    def _prefill(self, rows: List[int], prompts: List[List[int]]) -> torch.Tensor:
        s = self.s
        lens = [len(p) for p in prompts]
        ids = torch.tensor([t for p in prompts for t in p], dtype=torch.int64, device=self.dev)
        pos = torch.cat([torch.arange(L, device=self.dev) for L in lens])
        locs = torch.cat([s.bt.table[r, :L] for r, L in zip(rows, lens)])
        r = torch.tensor(rows, dtype=torch.int32, device=self.dev)
        zeros = torch.zeros(len(rows), dtype=torch.int32, device=self.dev)
        b = ExtendBatch(ids, pos, locs, r, zeros, extend_len=0, extend_lens=lens, prefix_lens_host=[0] * len(rows))
        hid = s.target.forward_torch(b, s.kv_t, s.bt.table, None)
        s.draft.forward_torch(b, s.kv_d, s.bt.table, None)
        last = torch.tensor(lens, device=self.dev).cumsum(0) - 1
        return self._probs(s.target.logits_torch(hid[last]))

    # ------------------------------------------------------------------ decoding
    def generate(self, input_ids: List[List[int]], max_new_tokens: int = 64, ignore_eos: bool = True,
                 eos_ids: Sequence[int] = ()) -> List[Dict]:
        outs: List[Optional[Dict]] = [None] * len(input_ids)
        B = int(self.args.max_running_requests)
        for lo in range(0, len(input_ids), B):
            for i, o in enumerate(self._wave(input_ids[lo:lo + B], max_new_tokens, ignore_eos, set(eos_ids))):
                outs[lo + i] = o
        return outs

    def _wave(self, prompts: List[List[int]], max_new: int, ignore_eos: bool, eos: set) -> List[Dict]:
        s, k = self.s, self.k
        need = [len(p) + max_new + k + 2 for p in prompts]
        if max(need) > s.bt.max_context:
            raise ValueError(f"prompt + output of {max(need)} tokens exceeds the context length {s.bt.max_context}")
        rows = list(range(len(prompts)))                       # one block-table row per sequence of the wave
        pages = []
        for r, n in zip(rows, need):
            pg = s.alloc.alloc(n)
            if pg is None:
                for q_ in pages:
                    s.alloc.free(q_)
                raise RuntimeError("KV page pool exhausted")
            s.bt.table[r, :n] = pg
            pages.append(pg)
        try:
            p0 = self._prefill(rows, prompts)
            seqs = [list(p) for p in prompts]
            for i in range(len(prompts)):
                tok = int(p0[i].argmax()) if self.greedy else int(torch.multinomial(p0[i], 1, generator=self.gen))
                seqs[i].append(tok)
            plen = [len(p) for p in prompts]
            done = [False] * len(prompts)
            reason: List[Optional[dict]] = [None] * len(prompts)

            def check(i: int) -> None:
                new = seqs[i][plen[i]:]
                if not ignore_eos and eos:
                    for j, t in enumerate(new):
                        if t in eos:
                            del seqs[i][plen[i] + j + 1:]
                            done[i], reason[i] = True, {"type": "stop", "matched": t}
                            return
                if len(new) >= max_new:
                    del seqs[i][plen[i] + max_new:]
                    done[i], reason[i] = True, {"type": "length", "length": max_new}
            for i in range(len(prompts)):
                check(i)
            while not all(done):
                act = [i for i in range(len(prompts)) if not done[i]]
                ar = [rows[i] for i in act]
                n = [len(seqs[i]) for i in act]                # committed tokens; both caches hold at least n-2 of them
                # draft: the last two committed tokens (the first of them may be cached already; it is rewritten with
                # the same values), then k-1 single tokens
                q = self._extend(s.draft, s.kv_d, ar, [seqs[i][-2:] for i in act], [x - 2 for x in n])[:, 1]
                qs, drafts = [q], []
                for step in range(k):
                    d = q.argmax(-1) if self.greedy else torch.multinomial(q, 1, generator=self.gen).view(-1)
                    drafts.append(d)
                    if step == k - 1:
                        break
                    q = self._extend(s.draft, s.kv_d, ar, [[int(t)] for t in d], [x + step for x in n])[:, 0]
                    qs.append(q)
                D = torch.stack(drafts, dim=1)                 # [bs, k]
                Q = torch.stack(qs, dim=1)                     # [bs, k, V]
                # target: the last committed token and the k drafts in one pass
                P = self._extend(s.target, s.kv_t, ar, [[seqs[i][-1]] + D[j].tolist() for j, i in enumerate(act)],
                                 [x - 1 for x in n])           # [bs, k+1, V]
                self.stats["steps"] += 1
                self.stats["seq_steps"] += len(act)
                for j, i in enumerate(act):
                    new = accept_chain(P[j], Q[j], D[j].tolist(), self.gen, self.greedy)
                    self.stats["drafted"] += k
                    self.stats["accepted"] += len(new) - 1
                    seqs[i].extend(new)
                    check(i)
            out = []
            for i in range(len(prompts)):
                ids = seqs[i][plen[i]:]
                self.stats["committed"] += len(ids)
                out.append(dict(output_ids=ids, completion_tokens=len(ids), prompt_tokens=plen[i],
                                finish_reason=reason[i]))
            return out
        finally:
            for pg in pages:
                s.alloc.free(pg)

    def accept_rate(self) -> float:
        return self.stats["accepted"] / max(1, self.stats["drafted"])

    def tokens_per_step(self) -> float:
        """Committed tokens per sequence and draft-and-verify step (accepted drafts plus the redrawn / bonus token)."""
        return (self.stats["accepted"] + self.stats["seq_steps"]) / max(1, self.stats["seq_steps"])


def main(argv=None) -> None:
    from ..utils.prompts import random_prompts
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--draft-model", required=True)
    ap.add_argument("--num-prompts", type=int, default=8)
    ap.add_argument("--random-input-len", type=int, default=256)
    ap.add_argument("--random-output-len", type=int, default=512)
    ap.add_argument("--num-steps", type=int, default=4, help="draft tokens per step")
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--max-running-requests", type=int, default=8)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--random-seed", type=int, default=0)
    ns = ap.parse_args(argv)
    eng = SpecDecodeBaseline(ns.model, ns.draft_model, ns.num_steps, ns.temperature, ns.max_running_requests,
                             dtype=ns.dtype, device=ns.device, random_seed=ns.random_seed,
                             context_length=ns.random_input_len + ns.random_output_len + ns.num_steps + 8)
    prompts = random_prompts([ns.random_input_len] * ns.num_prompts, eng.s.target.cfg.vocab_size, seed=ns.random_seed)
    t0 = time.perf_counter()
    outs = eng.generate(prompts, ns.random_output_len)
    if eng.dev.type == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_out = sum(o["completion_tokens"] for o in outs)
    print(f"Output token throughput (tok/s): {n_out / dt:.2f}")
    print(json.dumps({"method": "sd", "num_steps": ns.num_steps, "accept_rate": eng.accept_rate(),
                      "tokens_per_step": eng.tokens_per_step(), "output_tokens": n_out, "seconds": dt}))


if __name__ == "__main__":
    main()
