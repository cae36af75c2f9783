"""Offline engine: ``SMCEngine(model, draft, ...)`` and ``generate``.

Public surface of the reference's engine (smcsd/engine.py:60-82 constructor, :200-374
generate, :376-413 profiling, :415-463 shutdown / context manager): prompts as text or
token ids, one dict per prompt back with ``text, output_ids, prompt_tokens,
completion_tokens`` and the SMC diagnostics ``smc_log_Z_hat, smc_log_w_tilde,
smc_particle_output_ids, smc_particle_texts``.  Scheduler processes are spawned one per
GPU and reached over three ZMQ sockets; with a single rank the scheduler may also run
inside the caller's process (``in_process=True``, the default for one rank), which
removes the socket hop from the hot loop.
"""
from __future__ import annotations

import atexit
import logging
import os
import pickle
import signal
import time
import uuid
from typing import Any, Dict, List, Optional, Union

from .config import EngineArgs
from .io_types import (AbortReq, GenerateRequest, ParticleOutput, ProfileReq, RequestOutput, RpcReq, SamplingParams,
                       ShutdownReq)

log = logging.getLogger("smcsd_b200.engine")


class SMCEngine:
    def __init__(self, model_path, draft_model_path, *, n_particles: int = 4, gamma: int = 4,
                 draft_temperature: float = 0.7, target_temperature: float = 1.0, power_alpha: float = 1.0,
                 resample_threshold: float = 0.5, resample_method: str = "systematic",
                 defer_bonus: Optional[bool] = None, cycle_graph: Optional[bool] = None,
                 enable_overlap: Optional[bool] = None, tp_size: int = 1, base_gpu_id: int = 0,
                 tokenizer=None, _fault: Optional[dict] = None, **server_args):
        known = EngineArgs.__dataclass_fields__
        extra = {k: server_args.pop(k) for k in list(server_args) if k not in known}
        self.args = EngineArgs(model_path=model_path, draft_model_path=draft_model_path, n_particles=n_particles,
                               gamma=gamma, draft_temperature=draft_temperature,
                               target_temperature=target_temperature, power_alpha=power_alpha,
                               resample_threshold=resample_threshold, resample_method=resample_method,
                               defer_bonus=defer_bonus, cycle_graph=cycle_graph, enable_overlap=enable_overlap,
                               tp_size=tp_size, base_gpu_id=base_gpu_id, extra=extra, **server_args).finalize()
        logging.basicConfig(level=getattr(logging, self.args.log_level.upper(), logging.ERROR))
        self.tokenizer = tokenizer
        if tokenizer is None and not self.args.skip_tokenizer_init and isinstance(model_path, str) \
                and os.path.isdir(model_path):
            try:
                from transformers import AutoTokenizer
                self.tokenizer = AutoTokenizer.from_pretrained(model_path, trust_remote_code=self.args.trust_remote_code)
            except Exception as e:  # a directory with weights but no tokenizer files
                log.warning("no tokenizer loaded from %s: %s", model_path, e)
        world = self.args.tp_size * self.args.pp_size * self.args.dp_size
        in_proc = self.args.in_process if self.args.in_process is not None else (world == 1)
        if in_proc and world != 1:
            raise ValueError("in_process=True needs tp_size * pp_size * dp_size == 1")
        self._sched = None
        self._procs = []
        self._partials: Dict[str, List[int]] = {}
        self._rr = 0
        self._closed = False
        if in_proc:
            from .runtime.scheduler import SMCScheduler
            self._sched = SMCScheduler(self.args)
            self.scheduler_info = [self._sched.server_info()]
        else:
            import zmq
            from .runtime.launcher import PortArgs, launch_schedulers
            self._zmq = zmq.Context(2)
            self.ports = PortArgs.init_new(self.args.dp_size, self.args.nccl_port)
            self._rx = self._zmq.socket(zmq.PULL)
            self._rx.bind(f"tcp://127.0.0.1:{self.ports.result_port}")
            self._rpc = self._zmq.socket(zmq.ROUTER)
            # a ROUTER silently drops a message for a peer whose connection handshake has not finished (a call right
            # after start-up); with this option the send fails instead and is retried
            self._rpc.setsockopt(zmq.ROUTER_MANDATORY, 1)
            self._rpc.bind(f"tcp://127.0.0.1:{self.ports.rpc_port}")
            self._crashed = False
            try:
                signal.signal(signal.SIGUSR1, self._on_child_crash)
            except ValueError:
                pass  # not the main thread
            self._procs, self.scheduler_info = launch_schedulers(self.args, self.ports, fault=_fault)
            self._tx = []
            for port in self.ports.request_ports:
                s = self._zmq.socket(zmq.PUSH)
                s.connect(f"tcp://127.0.0.1:{port}")
                self._tx.append(s)
        atexit.register(self.shutdown)

    # ------------------------------------------------------------------ helpers
    def _on_child_crash(self, *_):
        self._crashed = True

    def _eos_ids(self) -> List[int]:
        ids: List[int] = []
        tok = self.tokenizer
        if tok is not None:
            if getattr(tok, "eos_token_id", None) is not None:
                ids.append(int(tok.eos_token_id))
            ids.extend(int(i) for i in (getattr(tok, "additional_stop_token_ids", None) or []))
        if self._sched is not None:
            ids.extend(self._sched.target.cfg.eos_token_ids)
        else:
            from .models.config import resolve_config
            try:
                ids.extend(resolve_config(self.args.model_path).eos_token_ids)
            except Exception:
                pass
        return list(dict.fromkeys(ids))

    # ------------------------------------------------------------------ generate
    def generate(self, prompt: Union[str, List[str], None] = None,
                 sampling_params: Union[dict, List[dict], None] = None,
                 input_ids: Union[List[int], List[List[int]], None] = None,
                 return_particles: bool = True, timeout: Optional[float] = None):
        """``timeout`` (seconds, scheduler processes only): requests without a final answer by then are aborted on
        every replica and returned as ``{"aborted": True}`` instead of blocking the caller forever (a request or
        an answer lost between the processes)."""
        if (prompt is None) == (input_ids is None):
            raise ValueError("pass exactly one of prompt / input_ids")
        single = False
        if prompt is not None:
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer; pass input_ids instead")
            if isinstance(prompt, str):
                prompt, single = [prompt], True
            ids_list = [self.tokenizer.encode(p) for p in prompt]
        else:
            if len(input_ids) > 0 and isinstance(input_ids[0], int):
                input_ids, single = [input_ids], True
            ids_list = [list(x) for x in input_ids]
        n = len(ids_list)
        if isinstance(sampling_params, (list, tuple)):
            if len(sampling_params) != n:
                raise ValueError("one sampling_params dict per prompt expected")
            sps = [SamplingParams.from_dict(d).normalize() for d in sampling_params]
        else:
            sps = [SamplingParams.from_dict(sampling_params).normalize() for _ in range(n)]
        eos = self._eos_ids()
        rids = [uuid.uuid4().hex for _ in range(n)]
        reqs = [GenerateRequest(rid, ids, sp, eos_token_ids=eos, arrival_time=time.time())
                for rid, ids, sp in zip(rids, ids_list, sps)]
        results: Dict[str, dict] = {}
        particles: Dict[str, ParticleOutput] = {}
        if self._sched is not None:
            for r in reqs:
                self._sched.add_request(r)
            pending = set(rids)
            while pending:
                if self._sched.paused:
                    raise RuntimeError("generation is paused (continue_generation() resumes it); an in-process "
                                       "scheduler cannot serve generate() meanwhile")
                for o in self._sched.step():
                    self._absorb(o, results, particles, pending)
                if not self._sched.has_work() and pending:
                    for o in self._sched.step():
                        self._absorb(o, results, particles, pending)
                    if pending and not self._sched.has_work():
                        raise RuntimeError(f"scheduler went idle with {len(pending)} requests unfinished")
        else:
            for i, r in enumerate(reqs):
                self._tx[(self._rr + i) % len(self._tx)].send_pyobj(r)
            self._rr = (self._rr + n) % len(self._tx)
            pending = set(rids)
            deadline = None if timeout is None else time.time() + float(timeout)
            while pending:
                if self._rx.poll(200) == 0:
                    self._check_children()
                    if deadline is not None and time.time() > deadline:
                        self._give_up(pending, results, float(timeout))
                    continue
                self._absorb(self._rx.recv_pyobj(), results, particles, pending)
        outs = []
        for rid, ids in zip(rids, ids_list):
            r = results[rid]
            r["prompt_tokens"] = len(ids)
            po = particles.get(rid)
            if po is not None and return_particles:
                r["smc_log_Z_hat"] = po.log_Z_hat
                r["smc_log_w_tilde"] = po.log_w_tilde
                r["smc_particle_output_ids"] = po.particle_output_ids
                if self.tokenizer is not None:
                    r["smc_particle_texts"] = [self.tokenizer.decode(p) for p in po.particle_output_ids]
            if self.tokenizer is not None and not r.get("aborted"):
                r["text"] = self.tokenizer.decode(r["output_ids"], skip_special_tokens=True)
            else:
                r.setdefault("text", "")
            outs.append(r)
        return outs[0] if single else outs

    def _absorb(self, o, results, particles, pending) -> None:
        if isinstance(o, ParticleOutput):
            particles[o.rid] = o
            return
        if not isinstance(o, RequestOutput) or o.rid not in pending and o.rid not in self._partials:
            return
        acc = self._partials.setdefault(o.rid, [])
        acc.extend(o.output_ids)
        if o.finished:
            ids = self._partials.pop(o.rid)
            d: Dict[str, Any] = dict(output_ids=ids, completion_tokens=len(ids), finish_reason=o.finish_reason)
            if o.aborted:
                d["aborted"] = True
                d["error"] = o.error
            if o.time_stats:
                d["time_stats"] = o.time_stats
            results[o.rid] = d
            pending.discard(o.rid)

    def _give_up(self, pending, results, waited: float) -> None:
        """No final answer arrived in time: abort the requests wherever they are and report them as aborted."""
        for rid in list(pending):
            for tx in self._tx:
                tx.send_pyobj(AbortReq(rid))
            ids = self._partials.pop(rid, [])
            msg = f"no answer from the scheduler within {waited:g} s"
            results[rid] = dict(output_ids=ids, completion_tokens=len(ids), aborted=True, error=msg,
                                finish_reason={"type": "abort", "message": msg})
            pending.discard(rid)

    def _check_children(self) -> None:
        dead = [p for p in self._procs if not p.is_alive()]
        if dead or getattr(self, "_crashed", False):
            self.shutdown()
            raise RuntimeError("a scheduler process died; engine shut down")

    # ------------------------------------------------------------------ control
    def _rpc_roundtrip(self, msg, timeout: float = 600.0) -> List[Any]:
        if self._sched is not None:
            if isinstance(msg, ProfileReq):
                return [self._sched.handle_profile(msg)]
            return [self._sched.handle_rpc(msg)]
        leaders = [f"sched-{r * self.args.tp_size * self.args.pp_size}".encode() for r in range(self.args.dp_size)]
        import zmq
        deadline = time.time() + timeout
        for ident in leaders:
            while True:
                try:
                    self._rpc.send_multipart([ident, pickle.dumps(msg)])
                    break
                except zmq.ZMQError as e:
                    if e.errno != zmq.EHOSTUNREACH or time.time() > deadline:
                        raise
                    self._check_children()
                    time.sleep(0.01)             # the scheduler's control socket is still connecting
        out = []
        while len(out) < len(leaders):
            if self._rpc.poll(200) == 0:
                self._check_children()
                if time.time() > deadline:
                    raise TimeoutError("scheduler RPC timed out")
                continue
            _, payload = self._rpc.recv_multipart()
            out.append(pickle.loads(payload)[1])
        return out

    def start_profile(self, output_dir: Optional[str] = None, num_steps: Optional[int] = None,
                      activities: Optional[List[str]] = None, with_stack: bool = False,
                      record_shapes: bool = False, profile_by_stage: bool = False,
                      profile_stages: Optional[List[str]] = None):
        """Start a torch.profiler capture in every scheduler (same arguments as the reference,
        smcsd/engine.py:376-413); ``profile_stages`` restricts a by-stage capture to "prefill" and / or "decode"."""
        return self._rpc_roundtrip(ProfileReq("start", output_dir, num_steps, activities, with_stack,
                                              record_shapes, profile_by_stage, profile_stages))

    def stop_profile(self):
        return self._rpc_roundtrip(ProfileReq("stop"))

    def pause_generation(self):
        """Every scheduler finishes the cycle in flight and then neither admits nor advances groups until
        ``continue_generation``; requests sent meanwhile wait in the queue."""
        return self.collective_rpc("pause_generation")

    def continue_generation(self):
        return self.collective_rpc("continue_generation")

    def collective_rpc(self, method: str, **kwargs):
        return self._rpc_roundtrip(RpcReq(method, kwargs, req_id=int(time.time_ns() & 0x7FFFFFFF)))

    def get_server_info(self) -> dict:
        r = self.collective_rpc("server_info")[0]
        return r.value if hasattr(r, "value") else r

    def shutdown(self) -> None:
        if self._closed:
            return
        self._closed = True
        if self._sched is not None:
            self._sched = None
            return
        try:
            for s in getattr(self, "_tx", []):
                s.send_pyobj(ShutdownReq(), flags=1)  # NOBLOCK
        except Exception:
            pass
        from .runtime.launcher import kill_process_tree
        time.sleep(0.05)
        kill_process_tree(self._procs)
        try:
            for s in getattr(self, "_tx", []) + [self._rx, self._rpc]:
                s.close(0)
            self._zmq.term()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.shutdown()
        return False
