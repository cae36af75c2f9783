"""End-to-end CPU plumbing run on the tiny Llama pair (fp32, random init, no GPU)."""
import torch

from smcsd_b200 import SMCEngine


def _prompts(n=8, length=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 4096, (length,), generator=g).tolist() for _ in range(n)]


def _engine(**kw):
    base = dict(n_particles=4, gamma=4, draft_temperature=0.7, target_temperature=0.7, dtype="float32",
                device="cpu", max_running_requests=8, resample_threshold=0.5)
    base.update(kw)
    return SMCEngine("preset:tiny-target", "preset:tiny-draft", **base)


def test_plumbing_run_tiny_llama():
    eng = _engine()
    outs = eng.generate(input_ids=_prompts(), sampling_params={"max_new_tokens": 64, "ignore_eos": True})
    assert len(outs) == 8
    for o in outs:
        assert o["completion_tokens"] == 64 and len(o["output_ids"]) == 64
        ts = o["time_stats"]
        assert 0.0 <= ts["queue_s"] <= ts["ttft_s"] <= ts["e2e_s"] and ts["decode_cycles"] >= 1
        assert o["finish_reason"]["type"] == "length"
        assert len(o["smc_particle_output_ids"]) == 4
        assert len(o["smc_log_w_tilde"]) == 4
        assert all(0 <= t < 4096 for t in o["output_ids"])
    sched = eng._sched
    sched.check_idle_invariants()
    sched.alloc.check_conservation()
    assert sched.stats["finished"] == 8


def test_seed_determinism_and_single_input():
    a = _engine(random_seed=3).generate(input_ids=_prompts(1)[0], sampling_params={"max_new_tokens": 20, "ignore_eos": True})
    b = _engine(random_seed=3).generate(input_ids=_prompts(1)[0], sampling_params={"max_new_tokens": 20, "ignore_eos": True})
    assert isinstance(a, dict)
    assert a["output_ids"] == b["output_ids"]
    assert a["smc_log_Z_hat"] == b["smc_log_Z_hat"]


def test_legacy_schedule_and_more_requests_than_slots():
    eng = _engine(defer_bonus=False, max_running_requests=2)
    outs = eng.generate(input_ids=_prompts(5, 16), sampling_params={"max_new_tokens": 12, "ignore_eos": True})
    assert [o["completion_tokens"] for o in outs] == [12] * 5
    eng._sched.check_idle_invariants()


def test_eos_stops_and_prefill_finish():
    eng = _engine()
    p = _prompts(1)[0]
    # every token is a stop token: the request ends at x0, before any fan-out
    o = eng.generate(input_ids=p, sampling_params={"max_new_tokens": 30, "stop_token_ids": list(range(4096))[:8]})
    assert o["completion_tokens"] >= 1
    o2 = eng.generate(input_ids=p, sampling_params={"max_new_tokens": 1, "ignore_eos": True})
    assert o2["completion_tokens"] == 1 and o2["finish_reason"]["type"] == "length"
    eng._sched.check_idle_invariants()


def test_rejected_features_abort():
    eng = _engine()
    o = eng.generate(input_ids=_prompts(1)[0], sampling_params={"max_new_tokens": 8, "stop": ["abc"]})
    assert o.get("aborted") and "stop strings" in o["error"]


def test_profiler_traces_whole_run_and_by_stage(tmp_path):
    """start_profile / stop_profile write Chrome traces; a by-stage capture writes one file per prefill / decode
    stretch and honours the stage filter."""
    import glob
    eng = _engine()
    ids = [list(range(3, 20))]
    sp = {"max_new_tokens": 9, "ignore_eos": True}
    eng.start_profile(output_dir=str(tmp_path / "whole"), activities=["CPU"])
    eng.generate(input_ids=ids, sampling_params=sp)
    eng.stop_profile()
    assert len(glob.glob(str(tmp_path / "whole" / "*.trace.json.gz"))) == 1
    eng.start_profile(output_dir=str(tmp_path / "staged"), activities=["CPU"], profile_by_stage=True)
    eng.generate(input_ids=ids, sampling_params=sp)
    eng.stop_profile()
    names = sorted(glob.glob(str(tmp_path / "staged" / "*.trace.json.gz")))
    assert any(n.endswith("-prefill.trace.json.gz") for n in names) and any(n.endswith("-decode.trace.json.gz") for n in names)
    eng.start_profile(output_dir=str(tmp_path / "decode_only"), activities=["CPU"], profile_by_stage=True,
                      profile_stages=["decode"])
    eng.generate(input_ids=ids, sampling_params=sp)
    eng.stop_profile()
    names = glob.glob(str(tmp_path / "decode_only" / "*.trace.json.gz"))
    assert names and all(n.endswith("-decode.trace.json.gz") for n in names)


def test_vanilla_arm_is_plain_target_sampling():
    """The baseline arm of the harnesses: one particle, gamma 1, the target as its own proposal.  Weights stay at
    zero (proposal == target), nothing resamples and the requested number of tokens comes out."""
    import argparse

    from smcsd_b200.config import EngineArgs
    from smcsd_b200.http_server import build_baseline_engine_from_args
    p = argparse.ArgumentParser()
    EngineArgs.add_cli_args(p)
    ns = p.parse_args(["--model", "preset:tiny-target", "--draft-model", "preset:tiny-draft", "--dtype", "float32",
                       "--device", "cpu", "--max-running-requests", "2"])
    eng = build_baseline_engine_from_args(ns, temperature=0.8)
    assert eng.args.n_particles == 1 and eng.args.gamma == 1
    outs = eng.generate(input_ids=[[5, 6, 7, 8], [9, 10, 11]], sampling_params={"max_new_tokens": 12, "ignore_eos": True})
    assert [o["completion_tokens"] for o in outs] == [12, 12]
    for o in outs:
        assert abs(o["smc_log_Z_hat"]) < 1e-4 and all(abs(w) < 1e-4 for w in o["smc_log_w_tilde"])
    assert eng._sched.stats["resampled_groups"] == 0
    eng.shutdown()


def test_e4m3_kv_cache_on_the_pytorch_path():
    """kv_cache_dtype='fp8_e4m3' on CPU: page rows hold e4m3 bytes and per-(token, head) scales; the PyTorch attention
    dequantises them.  The run completes, frees every page, and its tokens mostly agree with the bf16-cache run."""
    from smcsd_b200 import SMCEngine
    import torch
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 4096, (20,), generator=g).tolist() for _ in range(2)]
    kw = dict(n_particles=4, gamma=3, dtype="float32", device="cpu", max_running_requests=2, draft_temperature=0.7,
              target_temperature=0.7, random_seed=5)
    sp = {"max_new_tokens": 12, "ignore_eos": True}
    ref = SMCEngine("preset:tiny-target", "preset:tiny-draft", **kw).generate(input_ids=prompts, sampling_params=sp)
    eng = SMCEngine("preset:tiny-target", "preset:tiny-draft", kv_cache_dtype="fp8_e4m3", **kw)
    out = eng.generate(input_ids=prompts, sampling_params=sp)
    assert eng._sched.kv_t.k.dtype == torch.uint8
    assert [o["completion_tokens"] for o in out] == [12, 12]
    eng._sched.check_idle_invariants()
    agree = sum(int(a == b) for r, o in zip(ref, out) for a, b in zip(r["output_ids"], o["output_ids"])) / 24
    assert agree >= 0.5


def test_offline_throughput_sharegpt_dataset(tmp_path, capsys):
    """The offline throughput harness on a ShareGPT-style dump: first human turn = prompt, first reply length = that
    request's output budget; records without a reply are skipped; the sweep-parsable throughput line is printed."""
    import json
    from smcsd_b200.bench import offline_throughput as ot
    data = [
        {"conversations": [{"from": "human", "value": "tell me about the weather in the north of the country today"},
                           {"from": "gpt", "value": "it is going to rain a little in the morning and clear up later"}]},
        {"conversations": [{"from": "gpt", "value": "no human turn first"}]},
        {"conversations": [{"from": "human", "value": "how do i sort a list of numbers in python please"},
                           {"from": "gpt", "value": "call sorted on the list or use the sort method of the list"}]},
    ]
    path = tmp_path / "sharegpt.json"
    path.write_text(json.dumps(data))
    prompts, outs = ot.load_sharegpt(str(path), 8, 4096)
    assert len(prompts) == 2 and outs == [14, 13] and all(0 <= t < 4096 for p in prompts for t in p)
    res = tmp_path / "res.jsonl"
    ot.main(["--model", "preset:tiny-target", "--draft-model", "preset:tiny-draft", "-N", "4", "-g", "3",
             "--dataset-name", "sharegpt", "--dataset-path", str(path), "--num-prompts", "2", "--device", "cpu",
             "--dtype", "float32", "--max-running-requests", "2", "--skip-warmup", "--result-file", str(res)])
    out = capsys.readouterr().out
    assert "Output token throughput (tok/s):" in out
    rec = json.loads(res.read_text().strip())
    assert rec["dataset"] == "sharegpt" and rec["num_prompts"] == 2


def test_device_status_in_the_cycle_snapshot_raises():
    """A non-zero status word of the kernels (a wait on another rank that ran out, a failed range check) reaches the
    host with the cycle snapshot and stops the scheduler instead of letting it serve from a damaged state."""
    import pytest
    eng = _engine()
    sched = eng._sched
    from smcsd_b200.io_types import GenerateRequest, SamplingParams
    sched.add_request(GenerateRequest("r0", _prompts(1)[0], SamplingParams(max_new_tokens=32, ignore_eos=True)))
    sched.step()                         # prefill
    sched._run_decode()
    snap, rids = sched.pending.popleft()
    assert snap.device_status == 0
    snap.scalars[2] = 2                  # what a timed-out wait on a peer's weights leaves behind
    with pytest.raises(RuntimeError, match="device status 2"):
        sched._process_snapshot(snap, rids)
