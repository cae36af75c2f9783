"""HTTP server on the CPU path: real uvicorn server in a thread, queried with ``requests``."""
import socket
import threading
import time

import pytest
import requests
import torch


_ENGINE = []


def server_app_engine():
    return _ENGINE[-1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module")
def server():
    import uvicorn

    from smcsd_b200 import SMCEngine
    from smcsd_b200.http_server import build_app
    eng = SMCEngine("preset:tiny-target", "preset:tiny-draft", n_particles=4, gamma=4, dtype="float32", device="cpu",
                    max_running_requests=4, draft_temperature=0.7, target_temperature=0.7)
    app = build_app(eng, "tiny")
    _ENGINE.append(eng)
    port = _free_port()
    cfg = uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning")
    srv = uvicorn.Server(cfg)
    t = threading.Thread(target=srv.run, daemon=True)
    t.start()
    base = f"http://127.0.0.1:{port}"
    for _ in range(100):
        try:
            if requests.get(base + "/health", timeout=1).status_code == 200:
                break
        except Exception:
            time.sleep(0.1)
    yield base
    srv.should_exit = True
    t.join(timeout=10)


def test_generate_and_info(server):
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 4096, (20,), generator=g).tolist()
    r = requests.post(server + "/generate", json={"input_ids": ids, "sampling_params": {"max_new_tokens": 12, "ignore_eos": True}}, timeout=120)
    assert r.status_code == 200
    j = r.json()
    assert j["meta_info"]["completion_tokens"] == 12 and len(j["output_ids"]) == 12
    assert j["meta_info"]["finish_reason"]["type"] == "length"
    info = requests.get(server + "/server_info", timeout=10).json()
    assert info["smc"]["n_particles"] == 4 and info["n_served"] >= 1
    assert requests.get(server + "/get_model_info", timeout=10).status_code == 200
    assert requests.post(server + "/flush_cache", timeout=10).status_code == 200


def test_concurrent_requests_and_batch(server):
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 4096, (10 + i,), generator=g).tolist() for i in range(6)]
    results = [None] * 6

    def call(i):
        results[i] = requests.post(server + "/generate", json={"input_ids": prompts[i], "sampling_params": {"max_new_tokens": 9 + i, "ignore_eos": True}}, timeout=300).json()
    ts = [threading.Thread(target=call, args=(i,)) for i in range(6)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for i, r in enumerate(results):
        assert r["meta_info"]["completion_tokens"] == 9 + i
    r = requests.post(server + "/generate", json={"input_ids": prompts[:2], "sampling_params": {"max_new_tokens": 5, "ignore_eos": True}}, timeout=120).json()
    assert isinstance(r, list) and len(r) == 2


def test_openai_completions_and_errors(server):
    r = requests.post(server + "/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 7, "ignore_eos": True}, timeout=120)
    j = r.json()
    assert j["object"] == "text_completion" and j["usage"]["completion_tokens"] == 7
    assert requests.get(server + "/v1/models", timeout=10).json()["data"][0]["id"] == "tiny"
    bad = requests.post(server + "/generate", json={"input_ids": [1, 2], "sampling_params": {"max_new_tokens": 4, "stop": ["x"]}}, timeout=60)
    assert bad.status_code == 400
    assert requests.post(server + "/generate", json={}, timeout=10).status_code == 400


def test_streaming_routes_answer_as_server_sent_events(server):
    import json
    for path, body in (("/generate", {"input_ids": [3, 4, 5, 6, 7], "stream": True,
                                      "sampling_params": {"max_new_tokens": 6, "ignore_eos": True}}),
                       ("/v1/completions", {"prompt": [5, 6, 7, 8], "max_tokens": 6, "ignore_eos": True, "stream": True})):
        r = requests.post(server + path, json=body, timeout=120, stream=True)
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
        events = [ln[len("data: "):] for ln in r.iter_lines(decode_unicode=True) if ln and ln.startswith("data: ")]
        assert events[-1] == "[DONE]" and len(events) == 2
        payload = json.loads(events[0])
        n = payload["meta_info"]["completion_tokens"] if path == "/generate" else payload["usage"]["completion_tokens"]
        assert n == 6
    m = requests.get(server + "/server_info", timeout=10).json()["metrics"]
    assert 0.0 <= m["kv_occupancy"] <= 1.0 and m["decode_cycles"] >= 1


class _StubTokenizer:
    """Byte-level stand-in: enough of the tokenizer surface for the text routes."""
    chat_template = None

    def encode(self, text):
        return [ord(c) % 4096 for c in text]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(97 + int(t) % 26) for t in ids)


def test_abort_request_by_rid(server):
    out = {}

    def call():
        out["r"] = requests.post(server + "/generate", json={
            "input_ids": [9, 8, 7, 6, 5], "rid": "long-1",
            "sampling_params": {"max_new_tokens": 1900, "ignore_eos": True}}, timeout=300)
    t = threading.Thread(target=call)
    t.start()
    for _ in range(100):                      # until the request is in flight (a loaded machine may take a while)
        a = requests.post(server + "/abort_request", json={"rid": "long-1"}, timeout=10)
        assert a.status_code == 200
        if a.json()["aborted"] == ["long-1"]:
            break
        time.sleep(0.1)
    assert a.json()["aborted"] == ["long-1"]
    t.join(timeout=60)
    assert not t.is_alive() and out["r"].status_code == 400
    # an id that is not in flight aborts nothing; the server keeps serving
    assert requests.post(server + "/abort_request", json={"rid": "nobody"}, timeout=10).json()["aborted"] == []
    assert requests.post(server + "/abort_request", json={}, timeout=10).status_code == 400
    ok = requests.post(server + "/generate", json={"input_ids": [1, 2, 3], "rid": "short-1",
                                                   "sampling_params": {"max_new_tokens": 5, "ignore_eos": True}}, timeout=120)
    assert ok.status_code == 200 and ok.json()["meta_info"]["id"] == "short-1"


def test_chat_completions_and_profile_routes(server, tmp_path):
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    assert requests.post(server + "/v1/chat/completions", json={"messages": msgs}, timeout=10).status_code == 400
    server_app_engine().tokenizer = _StubTokenizer()
    try:
        r = requests.post(server + "/v1/chat/completions", json={"messages": msgs, "max_tokens": 6, "ignore_eos": True},
                          timeout=120)
        j = r.json()
        assert r.status_code == 200 and j["object"] == "chat.completion"
        assert j["choices"][0]["message"]["role"] == "assistant" and len(j["choices"][0]["message"]["content"]) == 6
        assert j["usage"]["completion_tokens"] == 6 and j["usage"]["prompt_tokens"] > 10
        assert requests.post(server + "/v1/chat/completions", json={"messages": "hi"}, timeout=10).status_code == 400
    finally:
        server_app_engine().tokenizer = None
    s = requests.post(server + "/start_profile", json={"output_dir": str(tmp_path), "activities": ["CPU"]}, timeout=30)
    assert s.status_code == 200 and s.json()["result"][0]["ok"]
    requests.post(server + "/generate", json={"input_ids": [4, 5, 6], "sampling_params": {"max_new_tokens": 6, "ignore_eos": True}}, timeout=120)
    e = requests.post(server + "/stop_profile", timeout=60)
    assert e.status_code == 200 and e.json()["result"][0]["ok"]


def test_pause_continue_and_priority_over_http(server):
    assert requests.post(server + "/pause_generation", timeout=30).json() == {"paused": True}
    out = {}

    def call():
        out["r"] = requests.post(server + "/generate", json={
            "input_ids": [2, 3, 4], "sampling_params": {"max_new_tokens": 5, "ignore_eos": True}}, timeout=120)
    t = threading.Thread(target=call)
    t.start()
    time.sleep(1.0)
    assert t.is_alive()                       # queued, not served, while paused
    assert requests.post(server + "/continue_generation", timeout=30).json() == {"paused": False}
    t.join(timeout=60)
    assert not t.is_alive() and out["r"].status_code == 200 and out["r"].json()["meta_info"]["completion_tokens"] == 5
    # this server runs without priority scheduling: a request that carries a priority is refused with a message
    bad = requests.post(server + "/generate", json={"input_ids": [2, 3, 4], "priority": 2,
                                                    "sampling_params": {"max_new_tokens": 5}}, timeout=60)
    assert bad.status_code == 400 and "priority" in bad.json()["detail"]


def test_client_that_hangs_up_frees_its_group(server):
    with pytest.raises(requests.exceptions.ReadTimeout):
        requests.post(server + "/generate", json={"input_ids": [7, 7, 7, 7], "sampling_params": {
            "max_new_tokens": 1900, "ignore_eos": True}}, timeout=0.6)
    for _ in range(150):                      # the disconnect is noticed within a poll interval, then the group goes
        info = requests.get(server + "/server_info", timeout=10).json()
        if info["n_running"] == 0 and info["n_waiting"] == 0:
            break
        time.sleep(0.1)
    assert info["n_running"] == 0 and info["n_waiting"] == 0
    assert info["stats"]["aborted"] >= 1


def test_metrics_route_is_prometheus_text(server):
    requests.post(server + "/generate", json={"input_ids": [5, 6, 7], "sampling_params": {"max_new_tokens": 6, "ignore_eos": True}}, timeout=120)
    r = requests.get(server + "/metrics", timeout=10)
    assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain")
    vals = {ln.split()[0]: float(ln.split()[1]) for ln in r.text.splitlines() if ln and not ln.startswith("#")}
    assert vals["smcsd:decode_cycles_total"] >= 1 and vals["smcsd:requests_finished_total"] >= 1
    assert 0.0 <= vals["smcsd:kv_occupancy"] <= 1.0 and vals["smcsd:num_running_reqs"] == 0
    assert "# TYPE smcsd:decode_tokens_total counter" in r.text


def test_health_reports_a_failed_engine_loop():
    """A scheduler step that raises (here injected on the host) answers the waiting client with the error and turns
    /health to 503 from then on."""
    from fastapi.testclient import TestClient

    from smcsd_b200 import SMCEngine
    from smcsd_b200.http_server import build_app
    eng = SMCEngine("preset:tiny-target", "preset:tiny-draft", n_particles=2, gamma=2, dtype="float32", device="cpu",
                    max_running_requests=2)
    real_step, calls = eng._sched.step, {"n": 0}

    def step():
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("the kernels reported device status 2 in a decode cycle")
        return real_step()
    eng._sched.step = step
    with TestClient(build_app(eng, "tiny")) as c:
        assert c.get("/health").status_code == 200
        r = c.post("/generate", json={"input_ids": [1, 2, 3], "sampling_params": {"max_new_tokens": 40, "ignore_eos": True}})
        assert r.status_code == 400 and "device status" in r.json()["detail"]
        h = c.get("/health")
        assert h.status_code == 503 and "device status" in h.json()["message"]


def test_unsupported_request_features_are_refused_with_a_message(server):
    base = {"input_ids": [1, 2, 3], "sampling_params": {"max_new_tokens": 4}}
    for extra, word in (({"return_logprob": True}, "return_logprob"), ({"return_hidden_states": True}, "hidden_states"),
                        ({"image_data": "x"}, "multimodal"), ({"input_embeds": [[0.1]]}, "input_embeds"),
                        ({"sampling_params": {"max_new_tokens": 4, "json_schema": "{}"}}, "grammar")):
        r = requests.post(server + "/generate", json={**base, **extra}, timeout=60)
        assert r.status_code == 400 and word in r.json()["detail"], (extra, r.text)
    r = requests.post(server + "/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 4, "logprobs": 2}, timeout=60)
    assert r.status_code == 400 and "return_logprob" in r.json()["detail"]
    r = requests.post(server + "/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 4, "n": 3}, timeout=60)
    assert r.status_code == 400 and "not supported" in r.json()["detail"]
