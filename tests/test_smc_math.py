"""SMC arithmetic on CPU: sampling identities, weight-increment gating truth table, ESS, systematic
resampling invariants, logZ unbiasedness on an enumerable toy model."""
import math

import pytest
import torch

from smcsd_b200.smc import math as M


def test_logprob_identity_and_extreme_logits():
    torch.manual_seed(0)
    for T in (0.5, 0.7, 1.0, 1.3):
        logits = torch.randn(6, 8, 32000) * 3
        idx = torch.randint(0, 32000, (6, 8))
        ref = torch.log_softmax(logits / T, -1).gather(-1, idx.unsqueeze(-1)).squeeze(-1)
        assert (M.chosen_logprob(logits, idx, T) - ref).abs().max() < 1e-4
    logits = torch.randn(4, 4, 1000) * 50
    idx = torch.randint(0, 1000, (4, 4))
    out = M.chosen_logprob(logits, idx, 0.7)
    assert torch.isfinite(out).all()


def test_gumbel_max_matches_softmax_distribution():
    g = torch.Generator().manual_seed(1)
    base = torch.randn(16) * 1.5
    logits = base.unsqueeze(0).expand(200000, 16)
    tok, logp, logz = M.gumbel_sample(logits, 0.7, 1.0, generator=g)
    emp = torch.bincount(tok, minlength=16).float() / tok.numel()
    p = torch.softmax(base / 0.7, -1)
    assert 0.5 * (emp - p).abs().sum() < 0.01
    assert logz.abs().max() == 0
    assert (logp - torch.log_softmax(base / 0.7, -1)[tok]).abs().max() < 1e-5


def test_greedy_limit_and_power_target():
    logits = torch.tensor([[0.1, 2.0, -1.0, 1.9]])
    tok, _, _ = M.gumbel_sample(logits, 0.0)
    assert int(tok) == 1
    g = torch.Generator().manual_seed(2)
    base = torch.randn(8)
    alpha, T = 1.7, 0.9
    tok, _, logz = M.gumbel_sample(base.unsqueeze(0).expand(100000, 8), T, alpha, generator=g)
    emp = torch.bincount(tok, minlength=8).float() / tok.numel()
    assert 0.5 * (emp - torch.softmax(alpha * base / T, -1)).abs().sum() < 0.01
    explicit = torch.logsumexp(alpha * base / T, -1) - alpha * torch.logsumexp(base / T, -1)
    assert abs(float(logz[0]) - float(explicit)) < 1e-5
    assert float(M.bonus_logz(base.unsqueeze(0), 1.0, T)) == pytest.approx(0.0, abs=1e-6)


def _wb(tokens, diff, logz, counts, finished, max_new, ignore, eos):
    t = lambda x, dt: torch.tensor(x, dtype=dt)
    return M.write_back_reference(t(tokens, torch.int32), t(diff, torch.float32),
                                  None if logz is None else t(logz, torch.float32), t(counts, torch.int32),
                                  t(finished, torch.bool), t(max_new, torch.int32), t(ignore, torch.bool),
                                  t(eos, torch.int32))


def test_weight_increment_gating_truth_table():
    eos = [[9, -1, -1, -1, -1, -1, -1, -1]]
    d = [[1.0, 2.0, 4.0]]
    # 1. nothing special: all gamma diffs + bonus
    r = _wb([[1, 2, 3, 4]], d, [0.5], [1], [False], [100], [False], eos)
    assert float(r["weight_inc"]) == 7.5 and not bool(r["newly_finished"])
    # 2. previously finished: absorbing, zero increment
    r = _wb([[1, 2, 3, 4]], d, [0.5], [1], [True], [100], [False], eos)
    assert float(r["weight_inc"]) == 0.0
    # 3. EOS at draft column 1: cutoff includes that column, bonus dropped
    r = _wb([[1, 9, 3, 4]], d, [0.5], [1], [False], [100], [False], eos)
    assert float(r["weight_inc"]) == 3.0 and int(r["finish_code"]) == M.FINISH_EOS and int(r["finished_len"]) == 3
    assert int(r["matched_eos"]) == 9
    # 4. EOS in the bonus column: all diffs and the bonus count
    r = _wb([[1, 2, 3, 9]], d, [0.5], [1], [False], [100], [False], eos)
    assert float(r["weight_inc"]) == 7.5 and int(r["finished_len"]) == 5
    # 5. length hit together with an EOS: length is the reason, EOS still sets the cutoff
    r = _wb([[9, 2, 3, 4]], d, [0.5], [1], [False], [5], [False], eos)
    assert int(r["finish_code"]) == M.FINISH_LENGTH and int(r["finished_len"]) == 5 and float(r["weight_inc"]) == 1.0
    # 6. ignore_eos: the EOS id is an ordinary token
    r = _wb([[9, 2, 3, 4]], d, None, [1], [False], [100], [True], eos)
    assert float(r["weight_inc"]) == 7.0 and not bool(r["newly_finished"])


def test_ess_and_threshold():
    assert float(M.effective_sample_size(torch.zeros(8))) == pytest.approx(8.0)
    w = torch.tensor([0.0, -50.0, -50.0, -50.0])
    assert float(M.effective_sample_size(w)) == pytest.approx(1.0, abs=1e-6)
    assert bool(M.should_resample(w, 0.5)) and not bool(M.should_resample(torch.zeros(4), 0.5))
    assert not bool(M.should_resample(w, 0.0)) and not bool(M.should_resample(torch.zeros(1), 0.5))


@pytest.mark.parametrize("n", [2, 4, 8, 16])
def test_systematic_resampling_invariants(n):
    g = torch.Generator().manual_seed(n)
    for trial in range(50):
        w = torch.softmax(torch.randn(n, generator=g) * 3, -1)
        u = float(torch.rand(1, generator=g))
        dst, src = M.resample_plan(w, u)
        assert len(dst) == len(src) and len(set(dst)) == len(dst) and not set(dst) & set(src)
        counts = torch.bincount(M.systematic_ancestors(w, u), minlength=n)
        # systematic resampling keeps floor(n w) <= count <= ceil(n w)
        assert ((counts.float() - n * w.float()).abs() < 1.0 + 1e-6).all()
        assert int(counts.sum()) == n
    dst, src = M.resample_plan(torch.full((n,), 1.0 / n), 0.37)
    assert dst == []
    w = torch.zeros(n)
    w[1] = 1.0
    dst, src = M.resample_plan(w, 0.5)
    assert sorted(dst) == [i for i in range(n) if i != 1] and set(src) == {1}


def test_philox_is_deterministic_and_uniform():
    a = M.philox_uniform(7, 3, 1)
    assert a == M.philox_uniform(7, 3, 1) and a != M.philox_uniform(7, 4, 1) and 0.0 < a < 1.0
    xs = [M.philox_uniform(1, s, r) for s in range(200) for r in range(5)]
    assert abs(sum(xs) / len(xs) - 0.5) < 0.03


def test_logz_estimator_is_unbiased_on_a_toy_model():
    """One-token toy: proposal q, target p over 6 symbols.  E[mean_i p(x_i)/q(x_i)] = 1, so exp(logZ_hat)
    averaged over many independent SMC groups must be 1."""
    g = torch.Generator().manual_seed(0)
    q = torch.softmax(torch.randn(6, generator=g), -1)
    p = torch.softmax(torch.randn(6, generator=g), -1)
    N, trials = 8, 20000
    x = torch.multinomial(q, N * trials, replacement=True, generator=g).view(trials, N)
    lw = torch.log(p[x]) - torch.log(q[x])
    z = torch.exp(M.logz_increment(lw))
    assert abs(float(z.mean()) - 1.0) < 0.02
