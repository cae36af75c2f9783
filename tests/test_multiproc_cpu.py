"""Process-per-rank plumbing on CPU (gloo): launcher handshake, ZMQ request path, tensor-parallel
sharding through torch.distributed, data-parallel replicas, and host-side fault injection
(a rank that raises during start-up, a rank that never reports ready, a rank that dies mid-run)."""
import pytest
import torch

from smcsd_b200 import SMCEngine


def _prompts(n, L=12, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 4096, (L,), generator=g).tolist() for _ in range(n)]


def _kw(**kw):
    base = dict(n_particles=4, gamma=3, dtype="float32", device="cpu", max_running_requests=4,
                draft_temperature=0.7, target_temperature=0.7, random_seed=5)
    base.update(kw)
    return base


def test_subprocess_scheduler_matches_in_process():
    sp = {"max_new_tokens": 10, "ignore_eos": True}
    a = SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(in_process=True)).generate(input_ids=_prompts(2), sampling_params=sp)
    with SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(in_process=False)) as eng:
        b = eng.generate(input_ids=_prompts(2), sampling_params=sp)
        info = eng.get_server_info()
        assert info["backend"] == "torch"
    assert [x["output_ids"] for x in a] == [x["output_ids"] for x in b]


def test_tensor_parallel_two_ranks_match_single_rank():
    """Two gloo ranks each hold half of the heads / ffn channels / vocabulary; the sharded run must
    reproduce the unsharded tokens (fp32, same seeds)."""
    sp = {"max_new_tokens": 9, "ignore_eos": True}
    ref = SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(in_process=True)).generate(input_ids=_prompts(2), sampling_params=sp)
    with SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(tp_size=2)) as eng:
        out = eng.generate(input_ids=_prompts(2), sampling_params=sp)
    for r, o in zip(ref, out):
        assert o["completion_tokens"] == 9
        agree = sum(int(x == y) for x, y in zip(r["output_ids"], o["output_ids"])) / 9
        assert agree >= 0.8      # summation order differs between sharded and unsharded fp32 matmuls


def test_tensor_parallel_hybrid_two_ranks_match_single_rank():
    """Hybrid Gated-DeltaNet target on two gloo ranks: attention heads, KV heads, Gated-DeltaNet key / value heads (with
    their conv channels and recurrent state), FFN channels and vocabulary rows are split over the ranks; the sharded
    run must reproduce the unsharded tokens (fp32, same seeds)."""
    sp = {"max_new_tokens": 9, "ignore_eos": True}
    ref = SMCEngine("preset:tiny-hybrid", "preset:tiny-draft", **_kw(in_process=True)).generate(input_ids=_prompts(2), sampling_params=sp)
    with SMCEngine("preset:tiny-hybrid", "preset:tiny-draft", **_kw(tp_size=2)) as eng:
        out = eng.generate(input_ids=_prompts(2), sampling_params=sp)
    for r, o in zip(ref, out):
        assert o["completion_tokens"] == 9
        agree = sum(int(x == y) for x, y in zip(r["output_ids"], o["output_ids"])) / 9
        assert agree >= 0.8      # summation order differs between sharded and unsharded fp32 matmuls


def test_data_parallel_replicas_round_robin():
    with SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(dp_size=2)) as eng:
        out = eng.generate(input_ids=_prompts(4), sampling_params={"max_new_tokens": 6, "ignore_eos": True})
        assert [o["completion_tokens"] for o in out] == [6] * 4
        assert len(eng.scheduler_info) == 2


def test_rank_failure_at_startup_is_reported():
    with pytest.raises(RuntimeError, match="injected init failure|exited before"):
        SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(in_process=False), _fault={"raise_in_init": 0})


def test_rank_that_never_joins_times_out():
    from smcsd_b200.config import EngineArgs
    from smcsd_b200.runtime.launcher import PortArgs, launch_schedulers
    args = EngineArgs(model_path="preset:tiny-target", draft_model_path="preset:tiny-draft", **_kw()).finalize()
    with pytest.raises(TimeoutError):
        launch_schedulers(args, PortArgs.init_new(1), fault={"never_ready": 0}, timeout=3.0)


def test_rank_death_mid_run_is_detected():
    eng = SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(in_process=False),
                    _fault={"die_after": 3, "die_rank": 0})
    with pytest.raises(RuntimeError, match="scheduler process died"):
        eng.generate(input_ids=_prompts(1), sampling_params={"max_new_tokens": 200, "ignore_eos": True})


@pytest.mark.parametrize("ranks,particles", [(2, 4), (4, 8)])
def test_particle_parallel_ranks_cpu(ranks, particles):
    """Particles of every group sharded over gloo ranks (two particles per rank): global resampling with cross-rank
    ancestor transfer, identical drain decisions on every rank, gathered finalize."""
    sp = {"max_new_tokens": 14, "ignore_eos": True}
    with SMCEngine("preset:tiny-target", "preset:tiny-draft",
                   **_kw(pp_size=ranks, n_particles=particles, resample_threshold=0.9)) as eng:
        out = eng.generate(input_ids=_prompts(3), sampling_params=sp)
        info = eng.collective_rpc("server_info")[0].value
    for o in out:
        assert o["completion_tokens"] == 14
        assert len(o["smc_particle_output_ids"]) == particles and len(o["smc_log_w_tilde"]) == particles
    assert info["stats"]["resampled_groups"] > 0


def test_lost_request_message_is_reported_not_waited_for():
    """One request message is dropped on its way to the scheduler (injected on the host): with a time limit the caller
    gets that request back as aborted, the others complete, and the engine keeps serving."""
    sp = {"max_new_tokens": 8, "ignore_eos": True}
    with SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(in_process=False),
                   _fault={"drop_request": 0}) as eng:
        out = eng.generate(input_ids=_prompts(2), sampling_params=sp, timeout=6.0)
        assert out[0].get("aborted") and "no answer" in out[0]["error"] and out[0]["completion_tokens"] == 0
        assert not out[1].get("aborted") and out[1]["completion_tokens"] == 8
        again = eng.generate(input_ids=_prompts(1, seed=3), sampling_params=sp, timeout=60.0)
        assert again[0]["completion_tokens"] == 8 and not again[0].get("aborted")


def test_pause_and_continue_reach_the_scheduler_process():
    sp = {"max_new_tokens": 6, "ignore_eos": True}
    with SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(in_process=False)) as eng:
        eng.pause_generation()
        assert eng.get_server_info()["paused"] is True
        out = eng.generate(input_ids=_prompts(1), sampling_params=sp, timeout=2.0)     # nothing is served while paused
        assert out[0].get("aborted")
        eng.continue_generation()
        assert eng.get_server_info()["paused"] is False
        out = eng.generate(input_ids=_prompts(1), sampling_params=sp, timeout=60.0)
        assert out[0]["completion_tokens"] == 6 and not out[0].get("aborted")


def test_a_group_rank_that_exits_mid_run_is_detected():
    """Two ranks share every request (particle-parallel).  The second rank exits between steps (host-injected); the
    first would wait for it in its next collective, but the engine sees the dead process, stops the others and raises
    instead of hanging."""
    eng = SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(pp_size=2, resample_threshold=0.9),
                    _fault={"die_after": 4, "die_rank": 1})
    with pytest.raises(RuntimeError, match="scheduler process died"):
        eng.generate(input_ids=_prompts(2), sampling_params={"max_new_tokens": 400, "ignore_eos": True})
    assert all(not p.is_alive() for p in eng._procs)


def test_bench_child_process_section_plumbing(tmp_path):
    """``bench.py --gpus N`` measures its fused-collective paths in child processes with a process group of their own
    and reads back the record rank 0 wrote; the plumbing-only mode runs the same path on two CPU ranks."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "children.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29637", os.path.join(root, "tests", "mp_bench_children_check.py"), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert json.loads(out.read_text()) == {"status": 0, "dry_run_world": 2}


def test_particle_parallel_hybrid_models_cpu():
    """Gated-DeltaNet models with the particles sharded over two ranks: a cross-rank ancestor brings its recurrent
    state (conv window and temporal state of every linear-attention layer) along with its KV rows."""
    sp = {"max_new_tokens": 14, "ignore_eos": True}
    kw = _kw(pp_size=2, resample_threshold=0.9, draft_temperature=1.0, target_temperature=0.5)
    with SMCEngine("preset:tiny-hybrid", "preset:tiny-hybrid", **kw) as eng:
        out = eng.generate(input_ids=_prompts(3), sampling_params=sp)
        info = eng.collective_rpc("server_info")[0].value
    assert [o["completion_tokens"] for o in out] == [14] * 3
    assert all(len(o["smc_particle_output_ids"]) == 4 for o in out)
    assert info["stats"]["resampled_groups"] > 0


def test_a_group_rank_that_stalls_ends_the_others_wait(monkeypatch):
    """One of two particle-parallel ranks never reaches the step (host-injected stall).  Its peer's host rendezvous
    after the prefill is time-limited: it fails naming the missing rank, the engine sees the crash and raises, well
    before any default collective timeout."""
    import time
    monkeypatch.setenv("SMC_PP_ALIGN_TIMEOUT_S", "4")
    eng = SMCEngine("preset:tiny-target", "preset:tiny-draft", **_kw(pp_size=2), _fault={"stall_rank": 1})
    t0 = time.time()
    with pytest.raises(RuntimeError, match="scheduler process died"):
        eng.generate(input_ids=_prompts(1), sampling_params={"max_new_tokens": 20, "ignore_eos": True})
    assert time.time() - t0 < 60
    assert all(not p.is_alive() for p in eng._procs)
