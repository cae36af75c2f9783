"""Group scheduler: admission, prefill, fan-out to particles, the decode loop (sequential
or overlapped with host post-processing), finalize and streaming of results.

Role of the reference's scheduler (smcsd/core/scheduler.py:202-1002): waiting / prefill /
running group queues, admission against slot capacity with reservations (:236-243,
:609-650), prefill before decode (:615-630), materialize with rollback (:734-828),
the overlapped loop whose post-processing runs one step late (:415-488), drain and
finalize (:960-1002), idle-time leak checks (:518-561).  This scheduler owns the model
objects and pools directly (the reference reaches them through SGLang's model runner).
"""
from __future__ import annotations

import logging
import os
import time
from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional

import torch

from ..config import EngineArgs
from ..io_types import (GenerateRequest, ParticleOutput, ProfileReq, RequestOutput, RpcReq, RpcResp,
                        validate_request)
from ..memory.pools import BlockTable, KVPool, KVSpec, PageAllocator, StatePool, cobudget_pages
from ..models import build_model
from ..utils import debug as smc_debug
from ..utils import profiling
from .slot_state import HostSnapshot, SlotState
from .worker import PrefillItem, SMCWorker

log = logging.getLogger("smcsd_b200.scheduler")


@dataclass
class SequenceGroup:
    """One user request and its N particles."""
    req: GenerateRequest
    n_particles: int
    parent_row: Optional[int] = None
    x0: Optional[int] = None
    reserved_pages: int = 0
    t_arrive: float = 0.0
    t_admit: float = 0.0
    t_first_token: float = 0.0
    cycles: int = 0
    launched: int = 0          # decode cycles enqueued for this group (processed or still in flight)

    @property
    def rid(self) -> str:
        return self.req.rid


def _resolve_device(args: EngineArgs, local_rank: int = 0) -> torch.device:
    if args.device == "cpu":
        return torch.device("cpu")
    if args.device in ("auto", "cuda") and torch.cuda.is_available():
        dev = torch.device("cuda", args.base_gpu_id + local_rank)
        torch.cuda.set_device(dev)
        return dev
    if args.device == "cuda":
        raise RuntimeError("device='cuda' requested but no GPU is visible")
    return torch.device("cpu")


class SMCScheduler:
    def __init__(self, args: EngineArgs, *, tp_rank: int = 0, tp_size: int = 1, dp_rank: int = 0,
                 local_rank: int = 0, target=None, draft=None, comm=None, pp_rank: int = 0, pp_size: int = 1):
        self.args = args.finalize() if args.defer_bonus is None else args
        a = self.args
        self.tp_rank, self.tp_size, self.dp_rank = tp_rank, tp_size, dp_rank
        self.pp_rank, self.pp_size = pp_rank, pp_size
        if a.n_particles % pp_size:
            raise ValueError("n_particles must be a multiple of the particle-parallel size")
        if pp_size > 1 and tp_size > 1:
            raise NotImplementedError("particle-parallel groups run with replicated (tp_size=1) models")
        self.n_local = a.n_particles // pp_size          # particles of each group held by this rank
        self.device = _resolve_device(a, local_rank)
        on_cuda = self.device.type == "cuda"
        self.dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[a.dtype]
        backend = a.backend
        if backend == "auto":
            backend = "native" if on_cuda and self.dtype == torch.bfloat16 else "torch"
        self.backend = backend
        if os.environ.get("SMC_SYNC_DEBUG") == "1" and on_cuda:
            torch.cuda.set_sync_debug_mode("warn")
        # ---- models -----------------------------------------------------------
        seed = a.random_seed
        self.target = target if target is not None else build_model(
            a.model_path, self.dtype, self.device, tp_rank, tp_size, seed=seed)
        if tp_size > 1 and backend == "native" and self.target.cfg.arch != "llama":
            # the kernel chain of the hybrid model has no collective stages: tensor-parallel hybrids run through the
            # PyTorch forward (heads, FFN channels and vocabulary sharded; partial sums all-reduced)
            if a.backend == "native":
                raise ValueError("tensor-parallel hybrid models run with backend='torch' (or 'auto')")
            backend = self.backend = "torch"
        # replicate_draft=False shards the draft over the tensor-parallel ranks like the target (fused all-gather /
        # reduce-scatter chain and vocab-parallel sampling on the kernel path, NCCL all-reduce on the PyTorch path)
        d_tp = (0, 1) if a.replicate_draft else (tp_rank, tp_size)
        if draft is None and tp_size == 1 and a.draft_model_path == a.model_path:
            draft = self.target           # the target as its own proposal (vanilla arm): one set of weights, two KV pools
        self.draft = draft if draft is not None else build_model(
            a.draft_model_path, self.dtype, self.device, d_tp[0], d_tp[1], seed=seed + 1)
        self.comm = comm
        if comm is not None and tp_size > 1:
            # the PyTorch path (prefill, CPU ranks, cuBLAS baseline) reduces through torch.distributed
            self.target.tp_group = comm.device_group
            if not a.replicate_draft:
                self.draft.tp_group = comm.device_group
        if self.target.cfg.vocab_size != self.draft.cfg.vocab_size:
            raise ValueError("target and draft must share a vocabulary")
        if a.quantization == "fp8":
            # W8A8 on the tensor cores (e4m3 weights with per-row scales, activations quantised per token on the fly);
            # the models keep their bf16 weights for the embedding, the lm_head and the PyTorch reference paths
            if backend != "native" or tp_size > 1 or any(m.cfg.arch != "llama" for m in (self.target, self.draft)):
                raise ValueError("quantization='fp8' needs the kernel backend, dense models and tp_size=1")
            # the draft is bound by launch latency, not by weight bytes, and keeps its five-launch bf16 layers unless
            # SMC_FP8_DRAFT=1 (the importance weights absorb whatever the proposal computes)
            self.target.quantization = "fp8"
            if os.environ.get("SMC_FP8_DRAFT", "0") == "1":
                self.draft.quantization = "fp8"
        self.context_len = int(a.context_length or min(self.target.cfg.max_position, 16384))
        # ---- memory -----------------------------------------------------------
        N, G = self.n_local, a.gamma + 1
        self.max_groups = a.max_running_requests
        n_slots = self.max_groups * N
        n_parent_rows = max(self.max_groups, 4)
        kv8 = a.kv_cache_dtype == "fp8_e4m3"
        if kv8 and (tp_size > 1 or pp_size > 1 or any(m.cfg.arch != "llama" for m in (self.target, self.draft))):
            # the e4m3 cache is read by the fused attention step of the dense chain (and by the PyTorch oracle)
            raise ValueError("kv_cache_dtype='fp8_e4m3' needs dense models, tp_size=1 and no particle parallelism")
        kv_t = KVSpec(len(self.target.cfg.attn_layers), self.target.n_kv_heads, self.target.cfg.head_dim, self.dtype, kv8)
        kv_d = KVSpec(len(self.draft.cfg.attn_layers), self.draft.n_kv_heads, self.draft.cfg.head_dim, self.dtype, kv8)
        n_rows = n_slots + n_parent_rows
        spec_t, spec_d = self.target.state_spec(), self.draft.state_spec()
        state_bytes = sum(s.row_bytes * n_rows for s in (spec_t, spec_d) if s)
        if a.max_total_tokens:
            n_pages = int(a.max_total_tokens)
        elif on_cuda:
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(total * a.mem_fraction_static) - (total - free)
            n_pages = cobudget_pages(budget, kv_t.cell_bytes, kv_d.cell_bytes, 0, state_bytes)
            n_pages = min(n_pages, self.max_groups * (self.context_len + N * self.context_len))
        else:
            n_pages = min(self.max_groups * N * 512 + 4096, 1 << 16)
        if n_pages < N * G * 2:
            raise RuntimeError(f"not enough memory for the KV pools (pages={n_pages})")
        self.alloc = PageAllocator(n_pages, self.device)
        self.bt = BlockTable(n_slots, n_parent_rows, self.context_len, self.device)
        self.kv_t = KVPool(kv_t, n_pages, self.device)
        self.kv_d = KVPool(kv_d, n_pages, self.device)
        self.state_t = StatePool(spec_t, n_rows, self.device) if spec_t else None
        self.state_d = StatePool(spec_d, n_rows, self.device) if spec_d else None
        # ---- native backend -----------------------------------------------------
        self.native_state = None
        self.native_runner = None
        if backend == "native":
            from ..ops import native_backend
            self.native_state, self.native_runner = native_backend.create(self, comm)
        pools = [p for p in (self.state_t, self.state_d) if p is not None]
        self.state = SlotState(max_groups=self.max_groups, n_particles=N, gamma=a.gamma,
                               max_output_len=self.context_len, block_table=self.bt, allocator=self.alloc,
                               device=self.device, seed=seed, resample_threshold=a.resample_threshold,
                               resample_method=a.resample_method, state_pools=pools, native=self.native_state)
        if a.resample_method != "systematic" and backend == "native":
            raise ValueError("the fused resampling kernels implement 'systematic' only")
        if self.native_runner is not None:
            self.native_runner.st = self.state
            self.state.device_status = self.native_runner.status      # travels with every cycle snapshot
        self.worker = SMCWorker(a, self.target, self.draft, self.kv_t, self.kv_d, self.bt, self.alloc,
                                self.state_t, self.state_d, native_runner=self.native_runner, noise_rank=pp_rank)
        if pp_size > 1:
            self._init_particle_parallel(comm)
        # ---- queues -------------------------------------------------------------
        self.waiting: Deque[SequenceGroup] = deque()
        self.running: Dict[str, SequenceGroup] = {}
        self.reserved_pages = 0
        self.last_free_pages = self.min_free_pages = self.alloc.size
        self._log_alloc_retries = os.environ.get("SMC_LOG_ALLOC_RETRIES") == "1" and self.device.type == "cuda"
        self._alloc_retries_seen = 0
        self.paused = False
        self.pending: Deque = deque()       # snapshots awaiting host post-processing
        self.outbox: List = []
        self.final_gen = torch.Generator().manual_seed(seed * 31 + 5)
        self.stats = dict(cycles=0, prefills=0, finished=0, aborted=0, resampled_groups=0, decode_tokens=0)
        self.profiler = None
        self._profile_steps_left = None
        self._cycle_events: List = []
        self._time_cycles = os.environ.get("SMC_TIME_CYCLES", "0") == "1"    # device-timed ms per decode cycle
        self.emit_particles = a.emit_particle_output
        # bytes moved across PCIe by this scheduler (prompt uploads; snapshots and final tokens back)
        self.io_bytes = {"h2d": 0, "d2h": 0}
        self.worker.io_bytes = self.io_bytes

    def _init_particle_parallel(self, comm) -> None:
        """Particles of every group are sharded over the ranks of this model-parallel group."""
        from ..parallel import particle_parallel as ppm
        if comm is None:
            raise RuntimeError("particle-parallel groups need one process per rank")
        kvs = [self.kv_t, self.kv_d]
        if self.native_runner is None:
            self.state.pp = ppm.PpTorch(comm.host_group, self.pp_rank, self.pp_size, kvs)
            return
        from ..parallel.symm import SymmHeap
        st = self.state
        small = ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished", "finished_len", "finish_code",
                 "matched_eos", "all_token_ids", "group_to_slots")
        big = [(self.bt, "table")] + [(kv, n) for kv in kvs for n in ("k", "v")] + \
              [(p, n) for p in st.state_pools for n in ("conv", "temporal")]
        need = sum(getattr(st, f).numel() * getattr(st, f).element_size() + 256 for f in small)
        need += sum(getattr(o, n).numel() * getattr(o, n).element_size() + 256 for o, n in big)
        need += ppm.ParticleParallel.comm_bytes_needed(self.pp_size, st.max_groups, st.N) + (1 << 20)
        heap = SymmHeap(need, self.device, comm.device_group, self.pp_rank, self.pp_size)
        offsets = {}

        def migrate(obj, name):
            t = getattr(obj, name)
            off = heap.alloc(name, t.numel() * t.element_size())
            v = heap.view(off, t.shape, t.dtype)
            v.copy_(t)
            setattr(obj, name, v)
            offsets[v.data_ptr()] = off
            del t
        for f in small:
            migrate(st, f)
        for o, n in big:
            migrate(o, n)
        torch.cuda.empty_cache()
        nbytes = ppm.ParticleParallel.comm_bytes_needed(self.pp_size, st.max_groups, st.N)
        comm_off = heap.alloc("pp_comm", nbytes)
        comm_local = heap.view(comm_off, (nbytes,), torch.uint8)
        ns = self.native_state
        ns.bind(st)
        for nm in (self.native_runner.target, self.native_runner.draft, self.native_runner.pf_target,
                   self.native_runner.pf_draft):
            if nm is not None:
                nm.bt = self.bt.table                  # the block table now lives in the symmetric heap
        drv = ppm.ParticleParallel(st, ns, kvs, self.pp_rank, self.pp_size,
                                   lambda q, t: heap.ptrs[q] + offsets[t.data_ptr()],
                                   [p + comm_off for p in heap.ptrs], comm_local, self.native_runner.status)
        self._pp_heap = heap
        st.pp = ppm.PpNative(comm.host_group, self.pp_rank, self.pp_size, drv)
        heap.barrier()

    # ------------------------------------------------------------------ intake
    def add_request(self, req: GenerateRequest) -> None:
        err = validate_request(req, self.context_len, self.args.gamma)
        if err is None and self.args.max_queued_requests is not None and \
                len(self.waiting) >= self.args.max_queued_requests:
            err = "the request queue is full"
        prio = getattr(req, "priority", None)
        if err is None and prio is not None and not self.args.enable_priority_scheduling:
            # same rule as the reference's scheduler base (smcsd/core/scheduler.py:576-577)
            err = "using priority is disabled for this server; send the request without a priority"
        if err is not None:
            self.stats["aborted"] += 1
            self.outbox.append(RequestOutput(req.rid, [], True, {"type": "abort", "message": err},
                                             len(req.input_ids), 0, aborted=True, error=err))
            return
        g = SequenceGroup(req, self.args.n_particles, t_arrive=time.time())
        if not self.args.enable_priority_scheduling:
            self.waiting.append(g)
            return
        # ordered insert: more urgent groups first, arrival order among equals; a request without a priority is the
        # least urgent.  Admission always takes the head, so a large urgent request is not overtaken by smaller ones.
        low_first = self.args.schedule_low_priority_values_first
        key = (lambda p: p if p is not None else float("inf")) if low_first else \
              (lambda p: -p if p is not None else float("inf"))
        k = key(prio)
        at = len(self.waiting)
        for i, other in enumerate(self.waiting):
            if key(getattr(other.req, "priority", None)) > k:
                at = i
                break
        self.waiting.insert(at, g)

    def abort(self, rid: str) -> None:
        for g in list(self.waiting):
            if g.rid == rid:
                self.waiting.remove(g)
                self.stats["aborted"] += 1
                self.outbox.append(RequestOutput(rid, [], True, {"type": "abort"}, aborted=True))
                return
        g = self.running.get(rid)
        if g is not None:
            self._flush_pending()
            # the pending snapshot may have shown the group finished: then it was finalized and released already
            if self.running.get(rid) is not g:
                return
            self._release_group(g)
            self.stats["aborted"] += 1
            self.outbox.append(RequestOutput(rid, [], True, {"type": "abort"}, aborted=True))

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self.pending)

    def pause_generation(self) -> bool:
        """Stop admitting and advancing groups after the cycle in flight (the snapshot queue is drained first, so a
        paused scheduler holds no unprocessed device results).  Requests that arrive meanwhile wait in the queue."""
        self._flush_pending()
        self.paused = True
        return True

    def continue_generation(self) -> bool:
        self.paused = False
        return True

    # ------------------------------------------------------------------ admission
    def _pages_needed(self, g: SequenceGroup) -> int:
        L = len(g.req.input_ids)
        return L + self.n_local * (g.req.sampling_params.max_new_tokens + 2 * (self.args.gamma + 1))

    def _admit(self) -> List[SequenceGroup]:
        """Admit waiting groups while slots, parent rows and worst-case pages are available.
        Pages are reserved up front, so a running group can never run the pool dry."""
        admitted: List[SequenceGroup] = []
        free_groups = len(self.state.free_rows) - 0
        while self.waiting and free_groups - len(admitted) > 0:
            g = self.waiting[0]
            need = self._pages_needed(g)
            if need > self.alloc.size:
                self.waiting.popleft()
                msg = f"request needs {need} KV pages; the pool holds {self.alloc.size}"
                self.outbox.append(RequestOutput(g.rid, [], True, {"type": "abort", "message": msg},
                                                 len(g.req.input_ids), 0, aborted=True, error=msg))
                self.stats["aborted"] += 1
                continue
            if self.reserved_pages + need > self.alloc.size:
                break
            row = self.bt.alloc_parent_row()
            if row is None:
                break
            self.waiting.popleft()
            g.parent_row = row
            g.t_admit = time.time()
            g.reserved_pages = need
            self.reserved_pages += need
            admitted.append(g)
        return admitted

    # ------------------------------------------------------------------ prefill + fan-out
    def _run_prefill(self, groups: List[SequenceGroup]) -> None:
        self._flush_pending()               # prefill mutates allocator state from the host
        items = []
        for g in groups:
            L = len(g.req.input_ids)
            pages = self.alloc.alloc(L)
            if pages is None:
                raise RuntimeError("page reservation violated")
            self.bt.table[g.parent_row, :L] = pages
            items.append(PrefillItem(g.parent_row, g.req.input_ids))
        if items and (self.state_t is not None or self.state_d is not None):
            # recurrent state of reused parent rows starts at zero: one indexed clear per pool for the whole batch
            prow = torch.tensor([it.row for it in items], dtype=torch.long).to(self.device, non_blocking=True)
            for pool in (self.state_t, self.state_d):
                if pool is not None:
                    pool.clear_rows(prow)
        with profiling.span(f"step[PREFILL smc bs={len(items)} toks={sum(len(i.input_ids) for i in items)}]"):
            x0 = self.worker.prefill(items).tolist()          # one blocking read per prefill batch
        self.stats["prefills"] += len(groups)
        for g, tok in zip(groups, x0):
            g.x0 = int(tok)
            g.t_first_token = time.time()
            self._materialize(g)
        if self.state.pp is not None:
            self.state.pp.align()           # prefill time differs per rank; the next cycle's weight exchange is bounded

    def _materialize(self, g: SequenceGroup) -> None:
        req, sp = g.req, g.req.sampling_params
        L = len(req.input_ids)
        eos = list(req.eos_token_ids or []) + list(sp.stop_token_ids or [])
        done_eos = (not sp.ignore_eos) and g.x0 in eos
        if done_eos or sp.max_new_tokens <= 1:
            # finished at prefill: never fans out
            reason = {"type": "stop", "matched": g.x0} if done_eos else {"type": "length", "length": 1}
            self.alloc.dec_ref_and_free(self.bt.table[g.parent_row, :L])
            self._finish_parent_rows(g)
            self.outbox.append(RequestOutput(g.rid, [g.x0], True, reason, L, 1))
            self.stats["finished"] += 1
            return
        try:
            self.state.allocate_group(g.rid, prompt_len=L, x0=g.x0, last_prompt_token=req.input_ids[-1],
                                      max_new_tokens=sp.max_new_tokens, ignore_eos=sp.ignore_eos, eos_ids=eos,
                                      parent_row=g.parent_row)
        except Exception as e:  # roll back and abort this one group
            log.exception("materialize failed for %s", g.rid)
            self.alloc.dec_ref_and_free(self.bt.table[g.parent_row, :L])
            self._finish_parent_rows(g)
            self.outbox.append(RequestOutput(g.rid, [], True, {"type": "abort", "message": str(e)}, L, 0,
                                             aborted=True, error=str(e)))
            self.stats["aborted"] += 1
            return
        if self.state_t is not None:
            pass  # recurrent state fan-out happens inside allocate_group
        self.bt.free_parent_row(g.parent_row)
        g.parent_row = None
        self.running[g.rid] = g

    def _finish_parent_rows(self, g: SequenceGroup) -> None:
        if g.parent_row is not None:
            for pool in (self.state_t, self.state_d):
                if pool is not None:
                    pool.clear_rows(torch.tensor([g.parent_row], device=self.device))
            self.bt.free_parent_row(g.parent_row)
            g.parent_row = None
        self.reserved_pages -= g.reserved_pages
        g.reserved_pages = 0

    # ------------------------------------------------------------------ decode
    def _run_decode(self) -> None:
        st = self.state
        timed = self._time_cycles and self.device.type == "cuda"
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        if self.native_runner is not None and self.native_runner.can_run_cycle(st):
            G = self.args.gamma + 1
            ctx = max((len(g.req.input_ids) + 1 + (g.launched + 1) * G for g in self.running.values()), default=0)
            plens = [len(g.req.input_ids) for g in self.running.values()]
            # graph replays bypass module hooks, so the span is labelled here for profiler traces
            with profiling.span(f"step[DECODE smc-cycle groups={len(self.running)} ctx<={ctx}]"):
                self.native_runner.run_cycle(st, self.worker, ctx_hint=ctx,   # one captured graph: prologue..resample
                                             prompt_hint=(min(plens), max(plens)) if plens else None)
        else:
            cin = st.prepare_cycle()
            out = self.worker.decode_cycle(cin)
            st.write_back(cin, out)
            n = st.resample()
            if n > 0:
                self.stats["resampled_groups"] += n
        if timed:
            e1.record()
            self._cycle_events.append((e0, e1, st.bs))
            if len(self._cycle_events) > 4096:
                del self._cycle_events[:2048]
        if self._log_alloc_retries:
            # a caching-allocator retry means a hidden cudaFree + synchronisation inside the decode loop
            n = torch.cuda.memory_stats(self.device).get("num_alloc_retries", 0)
            if n != self._alloc_retries_seen:
                log.warning("caching allocator retried %d time(s) during decode cycle %d", n - self._alloc_retries_seen,
                            self.stats["cycles"])
                self._alloc_retries_seen = n
        self.stats["cycles"] += 1
        self.stats["group_cycles"] = self.stats.get("group_cycles", 0) + len(self.running)
        self.stats["decode_tokens"] += st.bs * (self.args.gamma + 1)
        snap = st.snapshot_to_host()
        # finished flags, free-page count, allocator flag, resample counter, (status word), (per-group running counts)
        self.io_bytes["d2h"] += snap.finished.numel() + 16 + (4 if st.device_status is not None else 0) + \
            (4 * st.max_groups if st.pp is not None else 0)
        for g in self.running.values():
            g.launched += 1
        self.pending.append((snap, list(self.running.keys())))

    def _process_snapshot(self, snap: HostSnapshot, rids: List[str]) -> None:
        snap.wait()
        if snap.alloc_error:
            raise RuntimeError("device page allocator ran dry inside a decode cycle")
        if snap.device_status:
            raise RuntimeError(f"the kernels reported device status {snap.device_status} in a decode cycle (bit 1: a wait "
                               "on an mbarrier ran out, 2: a wait on another rank ran out, 4: the page allocator ran "
                               "dry, 8: an index failed its range check)")
        self.last_free_pages = snap.free_pages
        self.min_free_pages = min(self.min_free_pages, snap.free_pages)
        if self.native_runner is not None:
            self.stats["resampled_groups"] = int(snap.resampled[0])
        for rid in rids:
            g = self.running.get(rid)
            if g is None:
                continue
            g.cycles += 1
            if not self.state.group_has_active(rid, snap):
                self._finalize(g)

    def _all_certain_to_finish(self) -> bool:
        """True when the cycles already in flight take every running group to its length limit: each cycle
        appends gamma+1 tokens to the x0 a group starts with, so with overlap on the host knows the last
        cycle without waiting for its snapshot and does not enqueue a wasted one."""
        if not self.pending or not self.running:
            return False
        G = self.args.gamma + 1
        return all(1 + g.launched * G >= g.req.sampling_params.max_new_tokens for g in self.running.values())

    def _flush_pending(self) -> None:
        while self.pending:
            self._process_snapshot(*self.pending.popleft())

    def _finalize(self, g: SequenceGroup) -> None:
        res = self.state.finalize_group(g.rid, self.final_gen)
        self.io_bytes["d2h"] += self.args.n_particles * (self.state.max_output_len * 4 + 40)
        L = len(g.req.input_ids)
        out = RequestOutput(g.rid, res["output_ids"], True, res["finish_reason"], L, len(res["output_ids"]))
        now = time.time()
        out.time_stats = {"queue_s": max(0.0, g.t_admit - g.t_arrive), "ttft_s": max(0.0, g.t_first_token - g.t_arrive),
                          "e2e_s": max(0.0, now - g.t_arrive), "decode_cycles": float(g.cycles)}
        if self.emit_particles:
            self.outbox.append(ParticleOutput(g.rid, res["particle_output_ids"], res["log_Z_hat"],
                                              res["log_w_tilde"], res["picked"]))
        self.outbox.append(out)
        smc_debug.append_diag_record({"event": "finalize", "rid": g.rid, "log_Z_hat": res["log_Z_hat"],
                                      "cycles": g.cycles, "completion_tokens": len(res["output_ids"])})
        self._release_group(g)
        self.stats["finished"] += 1

    def _release_group(self, g: SequenceGroup) -> None:
        self.state.free_group(g.rid)
        self.running.pop(g.rid, None)
        self.reserved_pages -= g.reserved_pages
        g.reserved_pages = 0

    # ------------------------------------------------------------------ one iteration
    def step(self) -> List:
        """One scheduler iteration: admitted prefills run before decode; with overlap on, the host
        post-processes cycle t-1 after enqueuing cycle t (finish detection is one cycle late,
        which is harmless because finished particles are absorbing)."""
        if self.profiler is not None:
            self._profile_tick()
        if self.paused:
            # generation is paused: requests keep arriving (and can be aborted), nothing is admitted or advanced
            out, self.outbox = self.outbox, []
            return out
        admitted = self._admit()
        if self.profiler is not None and (admitted or self.running):
            self.profiler.enter_stage("prefill" if admitted else "decode")
        if admitted:
            self._run_prefill(admitted)
        elif self.running:
            if self._all_certain_to_finish():
                self._flush_pending()
            else:
                self._run_decode()
                keep = 1 if (self.args.enable_overlap and self.device.type == "cuda") else 0
                while len(self.pending) > keep:
                    self._process_snapshot(*self.pending.popleft())
        else:
            self._flush_pending()
            if not self.waiting:
                self.check_idle_invariants()
        out, self.outbox = self.outbox, []
        return out

    def run_until_idle(self) -> List:
        outs: List = []
        while self.has_work():
            if self.paused:
                raise RuntimeError("generation is paused; continue_generation() first")
            outs.extend(self.step())
        outs.extend(self.step())
        return outs

    # ------------------------------------------------------------------ invariants / info
    def check_idle_invariants(self) -> None:
        """With nothing running, every page is free and no slot is held."""
        if self.running or self.pending:
            return
        if os.environ.get("SMC_STRICT_MEM_CHECK", os.environ.get("SGLANG_ENABLE_STRICT_MEM_CHECK_DURING_IDLE", "1")) \
                not in ("1", "true", "True"):
            return
        free = self.alloc.available()
        if free != self.alloc.size:
            raise RuntimeError(f"KV page leak: {self.alloc.size - free} pages still held while idle")
        if len(self.state.free_slots) != self.state.max_slots:
            raise RuntimeError("slot leak while idle")
        if self.reserved_pages != 0:
            raise RuntimeError(f"page reservation leak: {self.reserved_pages}")

    def cycle_timing(self, last: int = 0, reset: bool = False) -> dict:
        """Device time of the recorded decode cycles (CUDA events; needs SMC_TIME_CYCLES=1)."""
        if not self._cycle_events:
            return {"cycles": 0}
        torch.cuda.synchronize(self.device)
        ev = self._cycle_events[-last:] if last else self._cycle_events
        ms = [a.elapsed_time(b) for a, b, _ in ev]
        rows = [n for _, _, n in ev]
        out = {"cycles": len(ms), "ms_mean": sum(ms) / len(ms), "ms_min": min(ms), "ms_max": max(ms),
               "ms_total": sum(ms), "rows_mean": sum(rows) / len(rows)}
        if reset:
            self._cycle_events.clear()
        return out

    def metrics(self) -> dict:
        """Serving metrics: KV pool occupancy (from the last cycle snapshot), resample rate per group-cycle,
        device-timed milliseconds per decode cycle when cycle timing is on."""
        cyc = max(1, self.stats.get("group_cycles", 0))
        m = {"kv_pages": self.alloc.size, "kv_pages_free": self.last_free_pages,
             "kv_occupancy": 1.0 - self.last_free_pages / max(1, self.alloc.size),
             "kv_occupancy_peak": 1.0 - self.min_free_pages / max(1, self.alloc.size),
             "kv_pages_reserved": self.reserved_pages,
             "resample_rate": self.stats.get("resampled_groups", 0) / cyc,
             "decode_cycles": self.stats.get("cycles", 0), "decode_tokens": self.stats.get("decode_tokens", 0)}
        if self._time_cycles:
            m["cycle_ms"] = self.cycle_timing()
        return m

    def server_info(self) -> dict:
        return dict(args=self.args.to_dict(), backend=self.backend, device=str(self.device),
                    kv_pages=self.alloc.size, context_len=self.context_len, stats=dict(self.stats),
                    n_running=len(self.running), n_waiting=len(self.waiting), paused=self.paused,
                    metrics=self.metrics(),
                    target=self.target.cfg.name, draft=self.draft.cfg.name)

    def flush_cache(self) -> bool:
        return not self.has_work()

    # ------------------------------------------------------------------ profiling
    def handle_profile(self, req: ProfileReq) -> dict:
        from ..utils.profiling import SchedulerProfiler
        if req.action == "start":
            self.profiler = SchedulerProfiler(req, rank=self.tp_rank)
            self.profiler.start()
            self._profile_steps_left = req.num_steps
            return {"ok": True}
        if self.profiler is not None:
            path = self.profiler.stop()
            paths = list(self.profiler.paths)
            self.profiler = None
            return {"ok": True, "trace": path, "traces": paths}
        return {"ok": False, "message": "profiler not running"}

    def _profile_tick(self) -> None:
        if self._profile_steps_left is None:
            return
        if self._profile_steps_left <= 0:
            self.profiler.stop()
            self.profiler = None
            self._profile_steps_left = None
        else:
            self._profile_steps_left -= 1

    def score_tokens(self, input_ids: List[int], continuation: List[int], temperature: float = 1.0) -> List[float]:
        """Diagnostic RPC: log softmax(logits / T)[continuation[i + 1]] at position i of ``continuation`` appended to
        the prompt, computed by the engine's own target path (prompt pass, then one verify-shaped pass of up to 16
        tokens: the kernel chain, tensor-parallel or not, with the fused scorer).  Gives tests a logit-level quantity
        that must agree between parallel layouts.  Only for an idle scheduler."""
        if self.running or self.waiting or self.pending:
            raise RuntimeError("score_tokens needs an idle scheduler")
        from .worker import PrefillItem
        E, L = len(continuation), len(input_ids)
        if not (2 <= E <= 16):
            raise ValueError("continuation must hold 2..16 tokens")
        dev = self.device
        row = self.bt.alloc_parent_row()
        pages = self.alloc.alloc(L + E)
        self.bt.table[row, :L + E] = pages
        try:
            self.worker.prefill([PrefillItem(row, list(input_ids))])
            ids = torch.tensor(continuation, dtype=torch.int32, device=dev)
            pos = torch.arange(L, L + E, dtype=torch.int32, device=dev)
            locs = pages[L:L + E].to(torch.int32).contiguous()
            rows = torch.tensor([row], dtype=torch.int32, device=dev)
            pref = torch.tensor([L], dtype=torch.int32, device=dev)
            given = torch.tensor(list(continuation[1:]) + [0], dtype=torch.int32, device=dev)
            if self.native_runner is not None:
                r = self.native_runner
                tok = torch.zeros(E, dtype=torch.int32, device=dev)
                lp = torch.zeros(E, dtype=torch.float32, device=dev)
                r._counters = self.state.counters
                r.target.set_context(L + E, 1, (E,))
                r._model_step("target", ids, pos, locs, rows, pref, 1, E, lm_rows=E, call_id=0,
                              temperature=float(temperature), alpha=1.0, tokens_in=given, tok_out=tok, logp_out=lp)
                out = lp[:E - 1].tolist()
                if r.check_status() != 0:
                    raise RuntimeError(f"device status {r.check_status()}")
            else:
                from ..models.layers import ExtendBatch
                ext = ExtendBatch(ids.long(), pos.long(), locs, rows, pref, extend_len=E, prefix_lens_host=[L])
                logits = self.target.logits_torch(self.target.forward_torch(ext, self.kv_t, self.bt.table))
                lsm = torch.log_softmax(logits.float() / float(temperature), dim=-1)
                out = lsm[torch.arange(E - 1, device=dev), given[:E - 1].long()].tolist()
        finally:
            self.alloc.free(pages)
            self.bt.free_parent_row(row)
        return out

    def handle_rpc(self, req: RpcReq) -> RpcResp:
        try:
            fn = getattr(self, req.method)
            return RpcResp(req.req_id, self.tp_rank, True, fn(**req.kwargs))
        except Exception as e:
            return RpcResp(req.req_id, self.tp_rank, False, repr(e))
