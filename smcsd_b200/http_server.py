"""HTTP serving: ``python -m smcsd_b200.http_server --model ... --draft-model ... -N 8 -g 8``.

Routes: ``/generate`` (native; an optional ``rid`` names the request), ``/abort_request`` (by ``rid`` or
``abort_all``), ``/v1/completions``, ``/v1/chat/completions`` (the tokenizer's chat template) and ``/v1/models``
(OpenAI style), ``/health``, ``/health_generate``, ``/server_info`` (alias ``/get_server_info``),
``/metrics`` (Prometheus text), ``/get_model_info``, ``/flush_cache``, ``/pause_generation`` / ``/continue_generation``, ``/start_profile`` /
``/stop_profile``; ``"stream": true`` on the generation
routes answers as server-sent events.  Concurrent HTTP requests are multiplexed onto the SMC scheduler by a pump thread
that owns the engine: it feeds new requests into the scheduler between decode cycles and resolves
each request's future when its group finalizes, so many clients share the batched decode loop.
Same CLI flags and routes as the reference server (smcsd/http_server.py:140-212; the routes it
inherits from SGLang are the ones its scripts use, scripts/accuracy_test_gsm8k_http.py:121-223).
The particle side channel is not sent over HTTP (the reference drops it in this mode too,
smcsd/core/scheduler.py:987-1001); ``smc_log_Z_hat`` is included in ``meta_info``.
"""
from __future__ import annotations

import argparse
import asyncio
import logging
import queue
import threading
import time
import uuid
from typing import Any, Dict, List, Optional

try:                                     # route signatures name this type; annotations are resolved at module level
    from fastapi import Request
except ImportError:                      # the offline engine works without the HTTP stack
    Request = Any

from .config import EngineArgs
from .io_types import AbortReq, GenerateRequest, ParticleOutput, RequestOutput, SamplingParams

log = logging.getLogger("smcsd_b200.http")


class EngineBridge:
    """Thread that owns the engine and multiplexes asynchronous requests onto it."""

    def __init__(self, engine):
        self.engine = engine
        self.inbox: "queue.Queue" = queue.Queue()
        self.futures: Dict[str, Any] = {}
        self.logz: Dict[str, float] = {}
        self.partial: Dict[str, List[int]] = {}
        self.loop: Optional[asyncio.AbstractEventLoop] = None
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._pump, name="smc-engine-pump", daemon=True)
        self.n_served = 0
        self.last_step_time = time.time()
        self.failed: Optional[str] = None       # first failure of the engine loop; the server reports unhealthy from then on

    def start(self, loop: asyncio.AbstractEventLoop) -> None:
        self.loop = loop
        self.thread.start()

    def stop(self) -> None:
        self._stop.set()
        self.thread.join(timeout=10)

    async def submit(self, input_ids: List[int], sp: SamplingParams, rid: Optional[str] = None,
                     priority: Optional[int] = None, extra: Optional[Dict[str, Any]] = None) -> dict:
        rid = rid or uuid.uuid4().hex
        if rid in self.futures:
            raise ValueError(f"request id {rid!r} is already in flight")
        fut = self.loop.create_future()
        self.futures[rid] = fut
        req = GenerateRequest(rid, list(input_ids), sp, eos_token_ids=self.engine._eos_ids(), arrival_time=time.time(),
                              priority=priority, **(extra or {}))
        self.inbox.put(req)
        return await fut

    def abort(self, rid: Optional[str] = None) -> List[str]:
        """Abort one request in flight (or all of them): the scheduler drops the group and answers it as aborted."""
        rids = [rid] if rid is not None else list(self.futures)
        rids = [r for r in rids if r in self.futures]
        for r in rids:
            self.inbox.put(AbortReq(r))
        return rids

    async def control(self, fn) -> Any:
        """Run ``fn()`` on the pump thread (the only thread that may touch the engine) and return its result."""
        fut = self.loop.create_future()
        self.inbox.put((fn, fut))
        return await fut

    def _resolve(self, rid: str, result: dict) -> None:
        fut = self.futures.pop(rid, None)
        if fut is not None and not fut.done():
            fut.set_result(result)

    def _handle(self, o) -> None:
        if isinstance(o, ParticleOutput):
            self.logz[o.rid] = o.log_Z_hat
            return
        if not isinstance(o, RequestOutput):
            return
        acc = self.partial.setdefault(o.rid, [])
        acc.extend(o.output_ids)
        if o.finished:
            ids = self.partial.pop(o.rid)
            res = dict(output_ids=ids, completion_tokens=len(ids), prompt_tokens=o.prompt_tokens,
                       finish_reason=o.finish_reason, aborted=o.aborted, error=o.error,
                       smc_log_Z_hat=self.logz.pop(o.rid, None), time_stats=o.time_stats)
            self.n_served += 1
            self.loop.call_soon_threadsafe(self._resolve, o.rid, res)

    def _run_control(self, fn, fut) -> None:
        try:
            res, err = fn(), None
        except Exception as e:        # the caller gets the failure, the pump keeps serving
            res, err = None, e

        def done():
            if not fut.done():
                fut.set_exception(err) if err is not None else fut.set_result(res)
        self.loop.call_soon_threadsafe(done)

    def _pump(self) -> None:
        eng = self.engine
        sched = eng._sched
        while not self._stop.is_set():
            try:
                if sched is not None:           # scheduler in this process
                    block = not sched.has_work()
                    try:
                        while True:
                            req = self.inbox.get(timeout=0.02) if block else self.inbox.get_nowait()
                            if isinstance(req, AbortReq):
                                sched.abort(req.rid)
                            elif isinstance(req, tuple):
                                self._run_control(*req)
                            else:
                                sched.add_request(req)
                            block = False
                    except queue.Empty:
                        pass
                    if sched.has_work() or sched.outbox:
                        for o in sched.step():
                            self._handle(o)
                        self.last_step_time = time.time()
                else:                           # scheduler processes behind ZMQ
                    try:
                        while True:
                            req = self.inbox.get_nowait()
                            if isinstance(req, AbortReq):
                                for tx in eng._tx:          # the replica that holds it answers; the others ignore it
                                    tx.send_pyobj(req)
                            elif isinstance(req, tuple):
                                self._run_control(*req)
                            else:
                                eng._tx[eng._rr].send_pyobj(req)
                                eng._rr = (eng._rr + 1) % len(eng._tx)
                    except queue.Empty:
                        pass
                    if eng._rx.poll(20):
                        self._handle(eng._rx.recv_pyobj())
                        self.last_step_time = time.time()
                    else:
                        eng._check_children()
            except Exception as e:  # surface the failure to every waiting client
                log.exception("engine pump failed")
                if self.failed is None:
                    self.failed = repr(e)
                for rid in list(self.futures):
                    self.loop.call_soon_threadsafe(
                        self._resolve, rid, dict(output_ids=[], completion_tokens=0, prompt_tokens=0,
                                                 finish_reason={"type": "abort", "message": repr(e)}, aborted=True,
                                                 error=repr(e), smc_log_Z_hat=None, time_stats=None))
                time.sleep(0.1)


def build_app(engine, model_name: str = "smc"):
    import json as _json

    from fastapi import FastAPI, HTTPException
    from fastapi.responses import JSONResponse, StreamingResponse

    def _sse(coro_factory):
        """Server-sent-event framing for ``stream: true``.  SMC picks the returned particle when the group
        finishes, so the stream carries one data event with the complete result, then ``[DONE]``."""
        async def gen():
            res = await coro_factory()
            for item in (res if isinstance(res, list) else [res]):
                yield "data: " + _json.dumps(item) + "\n\n"
            yield "data: [DONE]\n\n"
        return StreamingResponse(gen(), media_type="text/event-stream")

    from contextlib import asynccontextmanager
    bridge = EngineBridge(engine)

    @asynccontextmanager
    async def lifespan(_app):
        bridge.start(asyncio.get_running_loop())      # the pump thread lives as long as the server
        yield
        bridge.stop()

    app = FastAPI(title="smcsd_b200", lifespan=lifespan)
    app.state.bridge = bridge

    def _encode(text_or_ids) -> List[int]:
        if isinstance(text_or_ids, str):
            if engine.tokenizer is None:
                raise HTTPException(400, "this server has no tokenizer; send input_ids")
            return engine.tokenizer.encode(text_or_ids)
        return list(text_or_ids)

    def _decode(ids: List[int]) -> str:
        return engine.tokenizer.decode(ids, skip_special_tokens=True) if engine.tokenizer is not None else ""

    def _unsupported(body: Dict[str, Any]) -> Dict[str, Any]:
        """Request features this engine refuses (the scheduler answers each with its message, like the reference's
        request validation, smcsd/common/utils.py:150-167): they are passed on, not dropped silently."""
        x: Dict[str, Any] = {}
        if body.get("return_logprob") or body.get("logprobs") or body.get("top_logprobs"):
            x["return_logprob"] = True
        if body.get("return_hidden_states"):
            x["return_hidden_states"] = True
        if body.get("return_routed_experts"):
            x["return_routed_experts"] = True
        if body.get("input_embeds") is not None:
            x["input_embeds"] = True
        if body.get("image_data") is not None:
            x["image_data"] = True
        sp = body.get("sampling_params") if isinstance(body.get("sampling_params"), dict) else {}
        if any(body.get(k) or sp.get(k) for k in ("json_schema", "regex", "ebnf", "structural_tag")) \
                or body.get("response_format"):
            x["grammar"] = True
        return x

    async def _one(ids: List[int], params: Optional[dict], rid: Optional[str] = None,
                   priority: Optional[int] = None, http: Optional[Request] = None,
                   extra: Optional[Dict[str, Any]] = None) -> dict:
        try:
            sp = SamplingParams.from_dict(params).normalize()
            rid = rid or uuid.uuid4().hex
            task = asyncio.ensure_future(bridge.submit(ids, sp, rid, None if priority is None else int(priority), extra))
            while http is not None and not task.done():
                # a client that hung up frees its slots and pages now, not when its generation would have ended
                await asyncio.wait([task], timeout=0.25)
                if not task.done() and await http.is_disconnected():
                    bridge.abort(rid)
                    http = None                       # aborted once; the scheduler's answer ends the wait
            r = await task
        except (TypeError, ValueError) as e:
            raise HTTPException(400, str(e))
        if r["aborted"]:
            raise HTTPException(400, r["error"] or "request aborted")
        return {"text": _decode(r["output_ids"]), "output_ids": r["output_ids"],
                "meta_info": {"id": rid, "prompt_tokens": len(ids),
                              "completion_tokens": r["completion_tokens"], "finish_reason": r["finish_reason"],
                              "smc_log_Z_hat": r["smc_log_Z_hat"], "time_stats": r.get("time_stats")}}

    @app.post("/generate")
    async def generate(body: Dict[str, Any], request: Request):
        text, ids = body.get("text"), body.get("input_ids")
        if (text is None) == (ids is None):
            raise HTTPException(400, "send exactly one of text / input_ids")
        params = body.get("sampling_params") or {}
        src = text if text is not None else ids
        many = isinstance(src, list) and len(src) > 0 and isinstance(src[0], (list, str))
        items = src if many else [src]
        plist = params if isinstance(params, list) else [params] * len(items)
        rid = body.get("rid")                                # caller-chosen id(s), usable with /abort_request
        rids = rid if isinstance(rid, list) else [rid] * len(items) if (rid is None or not many) else None
        if rids is None or len(rids) != len(items):
            raise HTTPException(400, "rid must be one id per input")
        prio = body.get("priority")                          # honoured with --enable-priority-scheduling only
        extra = _unsupported(body)
        async def run():
            outs = await asyncio.gather(*[_one(_encode(x), p, r, prio, request, extra) for x, p, r in zip(items, plist, rids)])
            return outs if many else outs[0]
        if body.get("stream"):
            encoded = [_encode(x) for x in items]          # malformed input fails before the stream opens

            async def run_stream():
                outs = await asyncio.gather(*[_one(e, p, r, prio, request, extra) for e, p, r in zip(encoded, plist, rids)])
                return outs if many else outs[0]
            return _sse(run_stream)
        return await run()

    @app.post("/abort_request")
    async def abort_request(body: Dict[str, Any]):
        """``{"rid": id}`` aborts that request, ``{"abort_all": true}`` every request in flight; the aborted calls
        answer with status 400 and the abort reason."""
        if body.get("abort_all"):
            return {"aborted": bridge.abort(None)}
        if not body.get("rid"):
            raise HTTPException(400, "send rid or abort_all")
        return {"aborted": bridge.abort(str(body["rid"]))}

    @app.post("/v1/completions")
    async def completions(body: Dict[str, Any], request: Request):
        prompt = body.get("prompt")
        if prompt is None:
            raise HTTPException(400, "prompt is required")
        prompts = prompt if isinstance(prompt, list) and prompt and isinstance(prompt[0], (str, list)) else [prompt]
        params = {"max_new_tokens": int(body.get("max_tokens", 16)), "temperature": body.get("temperature", 1.0),
                  "ignore_eos": bool(body.get("ignore_eos", False))}
        if body.get("stop"):
            params["stop"] = body["stop"]
        if body.get("stop_token_ids"):
            params["stop_token_ids"] = body["stop_token_ids"]
        if int(body.get("n") or 1) != 1 or int(body.get("best_of") or 1) != 1:
            raise HTTPException(400, "n and best_of other than 1 are not supported: the particles of a request are not "
                                     "independent samples")
        encoded = [_encode(p) for p in prompts]
        extra = _unsupported(body)

        async def run():
            outs = await asyncio.gather(*[_one(e, params, http=request, extra=extra) for e in encoded])
            choices = [{"index": i, "text": o["text"], "token_ids": o["output_ids"],
                        "finish_reason": "length" if o["meta_info"]["finish_reason"]["type"] == "length" else "stop"}
                       for i, o in enumerate(outs)]
            pt = sum(o["meta_info"]["prompt_tokens"] for o in outs)
            ct = sum(o["meta_info"]["completion_tokens"] for o in outs)
            return {"id": "cmpl-" + uuid.uuid4().hex, "object": "text_completion", "created": int(time.time()),
                    "model": body.get("model", model_name), "choices": choices,
                    "usage": {"prompt_tokens": pt, "completion_tokens": ct, "total_tokens": pt + ct}}
        if body.get("stream"):
            return _sse(run)
        return await run()

    def _chat_prompt(messages) -> List[int]:
        tok = engine.tokenizer
        if tok is None:
            raise HTTPException(400, "this server has no tokenizer; chat completions need one")
        if not isinstance(messages, list) or not messages or not all(isinstance(m, dict) for m in messages):
            raise HTTPException(400, "messages must be a non-empty list of {role, content} objects")
        if getattr(tok, "chat_template", None) and hasattr(tok, "apply_chat_template"):
            ids = tok.apply_chat_template(messages, tokenize=True, add_generation_prompt=True)
            return list(ids["input_ids"] if isinstance(ids, dict) else ids)
        text = "".join(f"{m.get('role', 'user')}: {m.get('content', '')}\n" for m in messages) + "assistant:"
        return list(tok.encode(text))

    @app.post("/v1/chat/completions")
    async def chat_completions(body: Dict[str, Any], request: Request):
        ids = _chat_prompt(body.get("messages"))
        params = {"max_new_tokens": int(body.get("max_tokens") or body.get("max_completion_tokens") or 16),
                  "temperature": body.get("temperature", 1.0), "ignore_eos": bool(body.get("ignore_eos", False))}
        if body.get("stop"):
            params["stop"] = body["stop"]
        if body.get("stop_token_ids"):
            params["stop_token_ids"] = body["stop_token_ids"]

        if int(body.get("n") or 1) != 1:
            raise HTTPException(400, "n other than 1 is not supported: the particles of a request are not independent "
                                     "samples")
        extra = _unsupported(body)

        async def run():
            o = await _one(ids, params, http=request, extra=extra)
            fr = "length" if o["meta_info"]["finish_reason"]["type"] == "length" else "stop"
            pt, ct = o["meta_info"]["prompt_tokens"], o["meta_info"]["completion_tokens"]
            return {"id": "chatcmpl-" + uuid.uuid4().hex, "object": "chat.completion", "created": int(time.time()),
                    "model": body.get("model", model_name),
                    "choices": [{"index": 0, "message": {"role": "assistant", "content": o["text"]},
                                 "finish_reason": fr}],
                    "usage": {"prompt_tokens": pt, "completion_tokens": ct, "total_tokens": pt + ct}}
        if body.get("stream"):
            return _sse(run)
        return await run()

    @app.post("/pause_generation")
    async def pause_generation():
        """The cycle in flight completes, then nothing is admitted or advanced until ``/continue_generation``;
        requests sent meanwhile wait in the queue (their HTTP calls stay open)."""
        await bridge.control(engine.pause_generation)
        return {"paused": True}

    @app.post("/continue_generation")
    async def continue_generation():
        await bridge.control(engine.continue_generation)
        return {"paused": False}

    @app.post("/start_profile")
    async def start_profile(body: Optional[Dict[str, Any]] = None):
        b = body or {}
        kw = {k: b[k] for k in ("output_dir", "num_steps", "activities", "with_stack", "record_shapes",
                                "profile_by_stage", "profile_stages") if k in b}
        return {"result": await bridge.control(lambda: engine.start_profile(**kw))}

    @app.post("/stop_profile")
    async def stop_profile():
        return {"result": await bridge.control(engine.stop_profile)}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "smcsd_b200"}]}

    @app.get("/health")
    async def health():
        # a scheduler that raised (device status, a dead scheduler process) does not recover by itself: report it,
        # so that whatever supervises the server restarts it
        if bridge.failed is not None:
            return JSONResponse({"status": "error", "message": bridge.failed}, status_code=503)
        return JSONResponse({"status": "ok"})

    @app.get("/health_generate")
    async def health_generate():
        vocab_ok = [1, 2, 3, 4]
        await _one(vocab_ok, {"max_new_tokens": 2, "ignore_eos": True})
        return JSONResponse({"status": "ok"})

    async def _info() -> dict:
        # read on the pump thread, the only one that may touch the scheduler or the control socket; with scheduler
        # processes this is a live round trip to the first replica, not the record taken at start-up
        info = dict(await bridge.control(engine.get_server_info))
        info["n_served"] = bridge.n_served
        info["smc"] = {"n_particles": engine.args.n_particles, "gamma": engine.args.gamma,
                       "draft_temperature": engine.args.draft_temperature,
                       "target_temperature": engine.args.target_temperature,
                       "resample_threshold": engine.args.resample_threshold}
        return info

    @app.get("/server_info")
    async def server_info():
        return await _info()

    @app.get("/get_server_info")
    async def get_server_info():
        return await _info()

    @app.get("/metrics")
    async def metrics():
        """Prometheus text exposition of the serving gauges and counters."""
        from fastapi.responses import PlainTextResponse
        info = await _info()
        m, st = info.get("metrics", {}), info.get("stats", {})
        rows = [("num_running_reqs", "gauge", "request groups being decoded", info.get("n_running", 0)),
                ("num_queue_reqs", "gauge", "request groups waiting for admission", info.get("n_waiting", 0)),
                ("kv_occupancy", "gauge", "fraction of KV pages in use after the last cycle", m.get("kv_occupancy", 0.0)),
                ("kv_occupancy_peak", "gauge", "highest KV page occupancy seen", m.get("kv_occupancy_peak", 0.0)),
                ("kv_pages_reserved", "gauge", "KV pages reserved for running groups", m.get("kv_pages_reserved", 0)),
                ("resample_rate", "gauge", "resampling steps per group and decode cycle", m.get("resample_rate", 0.0)),
                ("decode_cycles_total", "counter", "decode cycles run", m.get("decode_cycles", 0)),
                ("decode_tokens_total", "counter", "tokens advanced over all particles", m.get("decode_tokens", 0)),
                ("prefills_total", "counter", "prompts prefilled", st.get("prefills", 0)),
                ("requests_finished_total", "counter", "requests finished", st.get("finished", 0)),
                ("requests_aborted_total", "counter", "requests aborted", st.get("aborted", 0)),
                ("requests_served_total", "counter", "HTTP generations answered", info.get("n_served", 0))]
        cyc = m.get("cycle_ms") or {}
        if isinstance(cyc, dict) and cyc.get("ms_mean") is not None:
            rows.append(("decode_cycle_ms", "gauge", "device-timed milliseconds per decode cycle (mean)", cyc["ms_mean"]))
        text = "".join(f"# HELP smcsd:{n} {h}\n# TYPE smcsd:{n} {t}\nsmcsd:{n} {float(v):g}\n" for n, t, h, v in rows)
        return PlainTextResponse(text, media_type="text/plain; version=0.0.4")

    @app.get("/get_model_info")
    async def model_info():
        return {"model_path": str(engine.args.model_path), "draft_model_path": str(engine.args.draft_model_path),
                "is_generation": True}

    @app.post("/flush_cache")
    async def flush_cache():
        ok = engine._sched.flush_cache() if engine._sched is not None else True
        return JSONResponse({"flushed": bool(ok)}, status_code=200 if ok else 400)

    return app


def build_engine_from_args(ns: argparse.Namespace):
    from .engine import SMCEngine
    a = EngineArgs.from_cli_args(ns)
    kw = a.to_dict()
    model, draft = a.model_path, a.draft_model_path
    for k in ("model_path", "draft_model_path", "extra"):
        kw.pop(k, None)
    return SMCEngine(model, draft, **kw)


def build_baseline_engine_from_args(ns: argparse.Namespace, temperature: float = 1.0):
    """Vanilla arm of the harnesses: plain sampling from the target model through the same kernels and scheduler.
    It is the engine with one particle, gamma = 1 and the target as its own proposal at the same temperature: every
    proposed token is then an exact draw from the target distribution, the importance weights stay constant and
    nothing is ever resampled, so the output law is that of ordinary autoregressive sampling at about one weight
    pass per generated token (the reference's ``--backend engine`` / ``--mode baseline`` arms:
    scripts/tps_benchmark_scripts/bench_offline_throughput.py:144-171, scripts/accuracy_test_gsm8k.py:177)."""
    from .engine import SMCEngine
    a = EngineArgs.from_cli_args(ns)
    kw = a.to_dict()
    model = a.model_path
    for k in ("model_path", "draft_model_path", "extra"):
        kw.pop(k, None)
    t = max(float(temperature), 1e-5)
    kw.update(n_particles=1, gamma=1, draft_temperature=t, target_temperature=t, power_alpha=1.0,
              resample_threshold=0.0)
    return SMCEngine(model, model, **kw)


def launch_server(ns: argparse.Namespace) -> None:
    import uvicorn
    engine = build_engine_from_args(ns)
    app = build_app(engine, model_name=str(ns.model_path))
    uvicorn.run(app, host=ns.host, port=ns.port, log_level=ns.log_level if ns.log_level != "error" else "warning")


def main(argv=None) -> None:
    p = argparse.ArgumentParser("smcsd_b200.http_server")
    EngineArgs.add_cli_args(p)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=30000)
    ns = p.parse_args(argv)
    launch_server(ns)


if __name__ == "__main__":
    main()
