"""Randomised operation sequences against the scheduler on the tiny CPU models: requests of random shapes, aborts of
waiting / running / finished / unknown ids, pauses, and steps in random order.  Whatever the order, every request
ends exactly once (finished or aborted), nothing leaks (pages, slots, parent rows) and the allocator's reference
counts add up."""
import random

import pytest
import torch

from smcsd_b200.config import EngineArgs
from smcsd_b200.io_types import GenerateRequest, RequestOutput, SamplingParams
from smcsd_b200.runtime.scheduler import SMCScheduler


def _sched(overlap: bool, **kw):
    base = dict(model_path="preset:tiny-target", draft_model_path="preset:tiny-draft", n_particles=3, gamma=2,
                dtype="float32", device="cpu", max_running_requests=3, draft_temperature=0.8, target_temperature=0.8,
                max_total_tokens=700, context_length=96, enable_overlap=overlap, resample_threshold=0.7)
    base.update(kw)
    return SMCScheduler(EngineArgs(**base).finalize())


@pytest.mark.parametrize("seed,overlap,models", [(0, True, "dense"), (1, False, "dense"), (2, True, "dense"),
                                                 (3, True, "hybrid"), (4, False, "hybrid")])
def test_random_operation_sequences_leave_nothing_behind(seed, overlap, models):
    rnd = random.Random(seed)
    # hybrid: recurrent-state rows are forked, copied by resampling and released next to the KV pages
    kw = dict(model_path="preset:tiny-hybrid", draft_model_path="preset:tiny-hybrid") if models == "hybrid" else {}
    s = _sched(overlap, **kw)
    g = torch.Generator().manual_seed(seed)
    sent, ended = {}, {}

    def absorb(outs):
        for o in outs:
            if isinstance(o, RequestOutput) and o.finished:
                assert o.rid in sent and o.rid not in ended, f"{o.rid} ended twice or was never sent"
                ended[o.rid] = o

    for op in range(220):
        r = rnd.random()
        if r < 0.22:
            rid = f"r{len(sent)}"
            n = rnd.randint(3, 24)
            eos = rnd.random() < 0.4
            sp = SamplingParams(max_new_tokens=rnd.randint(1, 30), ignore_eos=not eos)
            req = GenerateRequest(rid, torch.randint(0, 4096, (n,), generator=g).tolist(), sp,
                                  eos_token_ids=list(range(0, 4096, 11)) if eos else [])
            sent[rid] = req
            s.add_request(req)
        elif r < 0.32 and sent:
            s.abort(rnd.choice(list(sent)))             # waiting, running, finished long ago: all must be fine
        elif r < 0.34:
            s.abort("nobody")
        elif r < 0.38:
            s.pause_generation()
        elif r < 0.44:
            s.continue_generation()
        else:
            absorb(s.step())
    s.continue_generation()
    absorb(s.run_until_idle())
    assert set(ended) == set(sent)
    for rid, o in ended.items():
        sp = sent[rid].sampling_params
        if o.aborted:
            continue
        assert 1 <= o.completion_tokens <= sp.max_new_tokens
        if o.finish_reason["type"] == "length":
            assert o.completion_tokens == sp.max_new_tokens
        else:
            assert not sp.ignore_eos and o.finish_reason["matched"] % 11 == 0
    s.check_idle_invariants()
    s.alloc.check_conservation()
    assert s.alloc.available() == s.alloc.size and not s.running and not s.waiting and s.reserved_pages == 0
