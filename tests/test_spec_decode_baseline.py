"""Speculative-decoding baseline arm (draft, verify, accept by rejection sampling) on the tiny CPU models."""
import torch

from smcsd_b200.bench.spec_decode_baseline import SpecDecodeBaseline, accept_chain


def _prompts(n, L=11, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 4096, (L + i,), generator=g).tolist() for i in range(n)]


def test_accept_rule_reproduces_the_target_law():
    """First committed token of many chains drafted from q is distributed as p (exactness of the accept / redraw
    rule), and a chain whose drafts all pass earns the bonus token."""
    g = torch.Generator().manual_seed(1)
    V, k, n = 6, 2, 30000
    p = torch.softmax(torch.randn(k + 1, V, generator=g) * 1.5, -1)
    q = torch.softmax(torch.randn(k, V, generator=g) * 1.5, -1)
    counts = torch.zeros(V)
    lengths = torch.zeros(k + 2)
    for _ in range(n):
        d = [int(torch.multinomial(q[i], 1, generator=g)) for i in range(k)]
        out = accept_chain(p, q, d, g)
        counts[out[0]] += 1
        lengths[len(out)] += 1
    tv = 0.5 * float((counts / n - p[0]).abs().sum())
    assert tv < 0.02
    assert lengths[0] == 0 and lengths[k + 1] > 0 and float(lengths.sum()) == n
    # identical distributions accept everything
    assert len(accept_chain(p, p[:k].clone(), [1, 2], g)) == k + 1


def test_greedy_output_equals_plain_greedy_decoding_of_the_target():
    """With temperature 0 the accepted text must be exactly the target's greedy continuation, whatever the draft
    proposes; checked by scoring prompt + output in one fresh pass (no cache reuse) and comparing the arg-max of
    every position with the next token."""
    eng = SpecDecodeBaseline("preset:tiny-target", "preset:tiny-draft", num_steps=3, temperature=0.0,
                             max_running_requests=3, dtype="float32", device="cpu", context_length=128)
    prompts = _prompts(4)
    outs = eng.generate(prompts, max_new_tokens=17)
    assert [o["completion_tokens"] for o in outs] == [17] * 4
    assert eng.stats["steps"] > 0 and 0.0 <= eng.accept_rate() <= 1.0 and eng.tokens_per_step() >= 1.0
    s = eng.s
    for pr, o in zip(prompts, outs):
        full = pr + o["output_ids"]
        pages = s.alloc.alloc(len(full))
        s.bt.table[0, :len(full)] = pages
        probs = eng._extend(s.target, s.kv_t, [0], [full], [0])[0]          # [len, V] one pass over everything
        s.alloc.free(pages)
        nxt = probs.argmax(-1).tolist()
        for t in range(len(pr) - 1, len(full) - 1):
            assert nxt[t] == full[t + 1], t
    s.alloc.check_conservation()


def test_sampling_run_stops_on_eos_and_frees_its_pages():
    eng = SpecDecodeBaseline("preset:tiny-target", "preset:tiny-draft", num_steps=4, temperature=0.8,
                             max_running_requests=2, dtype="float32", device="cpu", context_length=128)
    free0 = eng.s.alloc.available()
    outs = eng.generate(_prompts(3, seed=2), max_new_tokens=20, ignore_eos=False, eos_ids=list(range(0, 4096, 7)))
    for o in outs:
        ids = o["output_ids"]
        if o["finish_reason"]["type"] == "stop":
            assert ids[-1] % 7 == 0 and all(t % 7 for t in ids[:-1])
        else:
            assert len(ids) == 20 and all(t % 7 for t in ids)
    assert eng.s.alloc.available() == free0
