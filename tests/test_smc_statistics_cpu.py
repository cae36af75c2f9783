"""End-to-end statistics of the engine on a toy vocabulary where the target law can be enumerated: the returned
sequence follows the target (not the draft), and exp(log_Z_hat) averages to one (both models are normalised, so the
true normalising constant is 1) for the two fixed resampling schedules (never, every cycle)."""
import pytest
import torch

from smcsd_b200 import SMCEngine
from smcsd_b200.bench.spec_decode_baseline import SpecDecodeBaseline
from smcsd_b200.models.config import ModelConfig

V = 8
T = 0.1           # random-init logits are small; a low temperature makes the two laws peaked and different


def _cfgs():
    tgt = ModelConfig(arch="llama", vocab_size=V, hidden_size=32, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=16,
                      ffn_size=64, max_position=64, name="toy-t")
    drf = ModelConfig(arch="llama", vocab_size=V, hidden_size=16, n_layers=1, n_heads=1, n_kv_heads=1, head_dim=16,
                      ffn_size=32, max_position=64, name="toy-d")
    return tgt, drf


def _kw(**kw):
    base = dict(dtype="float32", device="cpu", random_seed=3, context_length=48)
    base.update(kw)
    return base


def _marginals(prompt):
    """Exact law of the first drafted position (the token after x0) under the target and under the draft, by
    enumerating x0: sum over x0 of p(x0 | prompt) * model(. | prompt, x0)."""
    tgt, drf = _cfgs()
    o = SpecDecodeBaseline(tgt, drf, num_steps=2, temperature=T, max_running_requests=1, **_kw())
    s = o.s
    pages = s.alloc.alloc(len(prompt) + 1)
    s.bt.table[0, :len(prompt) + 1] = pages
    out = {}
    for name, model, kv in (("target", s.target, s.kv_t), ("draft", s.draft, s.kv_d)):
        p0 = o._extend(s.target, s.kv_t, [0], [prompt], [0])[0, -1]             # x0 always comes from the target
        m = torch.zeros(V)
        for x0 in range(V):
            m += p0[x0] * o._extend(model, kv, [0], [prompt + [x0]], [0])[0, -1]
        out[name] = m
    s.alloc.free(pages)
    return out["target"], out["draft"]


@pytest.mark.parametrize("threshold", [0.0, 1.0])
def test_output_law_and_normalising_constant(threshold):
    """Two cycles of three tokens after x0, 32 particles.  With threshold 1.0 every group is resampled after the first
    cycle, so the second cycle's weights start from the resampled set; with 0.0 it is plain importance sampling.  Both
    are fixed schedules, for which exp(log_Z_hat) is unbiased.  The law of the first drafted position of the returned
    sequence is the target's up to the O(1/N) bias of self-normalised weights, and far from the draft's."""
    tgt, drf = _cfgs()
    prompt = [1, 5, 2, 7, 3]
    p_t, p_d = _marginals(prompt)
    assert 0.5 * float((p_t - p_d).abs().sum()) > 0.2            # the two laws differ, so the test can tell them apart
    eng = SMCEngine(tgt, drf, n_particles=32, gamma=2, draft_temperature=T, target_temperature=T,
                    resample_threshold=threshold, max_running_requests=16, **_kw())
    n, counts, z = 0, torch.zeros(V), []
    for _ in range(8):
        outs = eng.generate(input_ids=[prompt] * 96, sampling_params={"max_new_tokens": 7, "ignore_eos": True})
        for o in outs:
            assert o["completion_tokens"] == 7
            counts[o["output_ids"][1]] += 1
            z.append(o["smc_log_Z_hat"])
            n += 1
    emp = counts / n
    tv_target = 0.5 * float((emp - p_t).abs().sum())
    tv_draft = 0.5 * float((emp - p_d).abs().sum())
    assert tv_target < 0.16 and tv_target < tv_draft - 0.04, (tv_target, tv_draft)
    zhat = torch.tensor(z, dtype=torch.float64).exp()
    se = float(zhat.std()) / n ** 0.5
    assert abs(float(zhat.mean()) - 1.0) < max(4 * se, 0.03), (float(zhat.mean()), se)
    if threshold == 1.0:
        assert eng._sched.stats["resampled_groups"] >= n           # every group was resampled after its first cycle


def test_particle_parallel_groups_keep_the_same_statistics():
    """The 32 particles of every request sharded over two gloo ranks, resampling after every cycle: weights are
    exchanged, every rank derives the same global plan and ancestors cross ranks.  The returned sequences must still
    follow the target law and exp(log_Z_hat) must still average to one."""
    tgt, drf = _cfgs()
    prompt = [1, 5, 2, 7, 3]
    p_t, p_d = _marginals(prompt)
    n, counts, z = 0, torch.zeros(V), []
    with SMCEngine(tgt, drf, n_particles=32, gamma=2, draft_temperature=T, target_temperature=T,
                   resample_threshold=1.0, max_running_requests=16, pp_size=2, **_kw()) as eng:
        for _ in range(5):
            outs = eng.generate(input_ids=[prompt] * 96, sampling_params={"max_new_tokens": 7, "ignore_eos": True})
            for o in outs:
                assert len(o["smc_particle_output_ids"]) == 32
                counts[o["output_ids"][1]] += 1
                z.append(o["smc_log_Z_hat"])
                n += 1
        info = eng.get_server_info()
    assert info["stats"]["resampled_groups"] >= n
    emp = counts / n
    tv_target = 0.5 * float((emp - p_t).abs().sum())
    tv_draft = 0.5 * float((emp - p_d).abs().sum())
    assert tv_target < 0.16 and tv_target < tv_draft - 0.04, (tv_target, tv_draft)
    zhat = torch.tensor(z, dtype=torch.float64).exp()
    se = float(zhat.std()) / n ** 0.5
    assert abs(float(zhat.mean()) - 1.0) < max(4 * se, 0.04), (float(zhat.mean()), se)
