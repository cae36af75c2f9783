"""Process-per-GPU launcher and the scheduler process entry point.

Topology: one API process plus one scheduler process per GPU.  The ranks of one
tensor-parallel / particle-parallel group all run the same scheduler loop on the same
request stream: the group's rank 0 owns the ZMQ sockets and broadcasts each iteration's
incoming messages to its peers over a gloo group, so every rank takes identical
decisions without further coordination.  Data-parallel replicas are independent groups
with their own request socket.  A ready handshake travels over a pipe; a crashing
scheduler logs its traceback and signals the parent, and children exit with the parent
(reference: smcsd/engine.py:158-189, smcsd/core/scheduler.py:1005-1043).
"""
from __future__ import annotations

import logging
import multiprocessing as mp
import os
import pickle
import signal
import socket
import sys
import threading
import time
import traceback
from dataclasses import dataclass
from typing import List, Optional

from ..config import EngineArgs

log = logging.getLogger("smcsd_b200.launcher")


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@dataclass
class PortArgs:
    request_ports: List[int]      # one PULL endpoint per replica group (API -> scheduler)
    result_port: int              # API PULL <- schedulers PUSH
    rpc_port: int                 # API ROUTER <-> scheduler DEALER
    dist_port: int                # torch.distributed rendezvous

    @classmethod
    def init_new(cls, n_replicas: int, dist_port: Optional[int] = None) -> "PortArgs":
        # all sockets stay bound until every port is chosen, so the ports are distinct
        socks = []
        try:
            for _ in range(n_replicas + 3):
                s = socket.socket()
                s.bind(("127.0.0.1", 0))
                socks.append(s)
            ports = [s.getsockname()[1] for s in socks]
        finally:
            for s in socks:
                s.close()
        return cls(ports[:n_replicas], ports[n_replicas], ports[n_replicas + 1], dist_port or ports[n_replicas + 2])


def _watch_parent(parent_pid: int) -> None:
    def loop():
        while True:
            if os.getppid() != parent_pid:
                os._exit(1)
            time.sleep(1.0)
    threading.Thread(target=loop, daemon=True).start()


def run_scheduler_process(args: EngineArgs, rank: int, world: int, ports: PortArgs, pipe_writer,
                          parent_pid: int, fault: Optional[dict] = None) -> None:
    """Entry point of one scheduler process.  ``fault`` injects host-side failures for the
    tests (raise during init, never report ready, die after k iterations)."""
    import zmq

    from ..io_types import AbortReq, GenerateRequest, ProfileReq, RpcReq, ShutdownReq
    from ..parallel.bootstrap import Comm
    from .scheduler import SMCScheduler

    logging.basicConfig(level=getattr(logging, args.log_level.upper(), logging.ERROR),
                        format=f"[rank {rank}] %(levelname)s %(name)s: %(message)s")
    _watch_parent(parent_pid)
    fault = fault or {}
    try:
        if fault.get("raise_in_init") == rank:
            raise RuntimeError("injected init failure")
        if fault.get("never_ready") == rank:
            time.sleep(3600)
        group = args.tp_size * args.pp_size           # ranks that cooperate on one request stream
        replica, in_group = divmod(rank, group)
        comm = None
        if world > 1:
            comm = Comm.init(rank, world, args, ports.dist_port, group_size=group)
        tp_rank = in_group % args.tp_size
        pp_rank = in_group // args.tp_size
        sched = SMCScheduler(args, tp_rank=tp_rank, tp_size=args.tp_size, dp_rank=replica, local_rank=rank, comm=comm,
                             pp_rank=pp_rank, pp_size=args.pp_size)
        ctx = zmq.Context(1)
        leader = in_group == 0
        if leader:
            rx = ctx.socket(zmq.PULL)
            rx.bind(f"tcp://127.0.0.1:{ports.request_ports[replica]}")
            tx = ctx.socket(zmq.PUSH)
            tx.connect(f"tcp://127.0.0.1:{ports.result_port}")
            rpc = ctx.socket(zmq.DEALER)
            rpc.setsockopt(zmq.IDENTITY, f"sched-{rank}".encode())
            rpc.connect(f"tcp://127.0.0.1:{ports.rpc_port}")
        pipe_writer.send({"status": "ready", "rank": rank, "kv_pages": sched.alloc.size,
                          "context_len": sched.context_len, "backend": sched.backend})
        iters = 0
        n_requests_seen = 0
        while True:
            msgs = []
            if leader:
                block = not sched.has_work()
                while True:
                    try:
                        if block and not msgs:
                            if rx.poll(50) == 0 and rpc.poll(0) == 0:
                                break
                        msgs.append(rx.recv_pyobj(zmq.NOBLOCK))
                    except zmq.Again:
                        break
                while rpc.poll(0):
                    msgs.append(pickle.loads(rpc.recv()))
            if leader and fault.get("drop_request") is not None:
                kept = []
                for m in msgs:                       # injected loss of one request message on its way in
                    if isinstance(m, GenerateRequest):
                        n_requests_seen += 1
                        if n_requests_seen - 1 == fault["drop_request"]:
                            continue
                    kept.append(m)
                msgs = kept
            if comm is not None and comm.group_size > 1:
                msgs = comm.broadcast_objects(msgs)
            stop = False
            for m in msgs:
                if isinstance(m, GenerateRequest):
                    sched.add_request(m)
                elif isinstance(m, AbortReq):
                    sched.abort(m.rid)
                elif isinstance(m, ProfileReq):
                    r = sched.handle_profile(m)
                    if leader:
                        rpc.send(pickle.dumps(("profile", r)))
                elif isinstance(m, RpcReq):
                    r = sched.handle_rpc(m)
                    if leader:
                        rpc.send(pickle.dumps(("rpc", r)))
                elif isinstance(m, ShutdownReq):
                    stop = True
            if stop:
                break
            if fault.get("stall_rank") == rank and sched.waiting:
                time.sleep(3600)                    # injected: this rank never reaches the step its peers wait in
            outs = sched.step() if (sched.has_work() or msgs) else []
            if sched.paused and not msgs:
                time.sleep(0.005)                   # paused with work queued: wait for the next message, do not spin
            if leader:
                for o in outs:
                    tx.send_pyobj(o)
            iters += 1
            if fault.get("die_after") is not None and fault.get("die_rank", 0) == rank and iters >= fault["die_after"]:
                os._exit(3)
        if comm is not None:
            comm.shutdown()
    except Exception:
        log.error("scheduler rank %d crashed:\n%s", rank, traceback.format_exc())
        try:
            pipe_writer.send({"status": "error", "rank": rank, "traceback": traceback.format_exc()})
        except Exception:
            pass
        try:
            os.kill(parent_pid, signal.SIGUSR1)
        except Exception:
            pass
        sys.exit(1)


def launch_schedulers(args: EngineArgs, ports: PortArgs, fault: Optional[dict] = None, timeout: float = 1800.0):
    """Spawn one scheduler per rank and wait for every ready message.  Returns (procs, infos);
    raises with the child's traceback if any rank fails or the handshake times out."""
    world = args.tp_size * args.pp_size * args.dp_size
    ctx = mp.get_context("spawn")
    procs, readers = [], []
    for rank in range(world):
        r, w = ctx.Pipe(duplex=False)
        p = ctx.Process(target=run_scheduler_process, args=(args, rank, world, ports, w, os.getpid(), fault),
                        daemon=True)
        p.start()
        w.close()
        procs.append(p)
        readers.append(r)
    infos = []
    deadline = time.time() + timeout
    try:
        for rank, (p, r) in enumerate(zip(procs, readers)):
            while True:
                left = deadline - time.time()
                if left <= 0:
                    raise TimeoutError(f"scheduler rank {rank} did not report ready within {timeout}s")
                if r.poll(min(left, 0.2)):
                    try:
                        info = r.recv()
                    except EOFError:
                        raise RuntimeError(f"scheduler rank {rank} exited before reporting ready "
                                           f"(exit code {p.exitcode})")
                    if info.get("status") != "ready":
                        raise RuntimeError(f"scheduler rank {rank} failed:\n{info.get('traceback')}")
                    infos.append(info)
                    break
                if not p.is_alive():
                    if r.poll(0):
                        continue
                    raise RuntimeError(f"scheduler rank {rank} exited before reporting ready "
                                       f"(exit code {p.exitcode})")
    except Exception:
        kill_process_tree(procs)
        raise
    return procs, infos


def kill_process_tree(procs) -> None:
    for p in procs:
        if p.is_alive():
            p.terminate()
    for p in procs:
        p.join(timeout=5)
        if p.is_alive():
            p.kill()
            p.join(timeout=5)
