"""Particle-parallel groups: the N particles of every request are sharded over R ranks.

Every rank holds full target and draft replicas and its own paged KV and recurrent-state pools,
prefills the prompt itself (so the prompt prefix is replicated per rank) and advances its
``N_local = N / R`` particles of every group.  Resampling is global: interval weights are
exchanged by peer stores, every rank derives the same systematic-resampling plan from the same
Philox offset, and a destination whose ancestor lives on another GPU pops fresh local pages,
rewrites its block-table suffix and gathers the ancestor's post-prompt KV rows and recurrent state
over NVLink from inside the kernel (``smcsd_b200/ops/csrc/particle_parallel.cu``).  The reference
keeps all particles of a group on one GPU and resamples by pointer copies only
(smcsd/core/kernels/fused_resample_kv.py:98-105); this capability is new here.

``plan_global`` / ``apply_reference`` restate the same algorithm in plain PyTorch for CPU ranks
(gloo) and as the oracle of the kernels.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Sequence, Tuple

import torch

from ..smc import math as smc_math

SLOT_FIELDS = ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished", "finished_len", "finish_code",
               "matched_eos", "all_token_ids")


# ----------------------------------------------------------------------------------- oracle / CPU path
def plan_global(weights_by_rank: Sequence[torch.Tensor], threshold: float, seed: int, step: int, row: int):
    """Resampling decision for one group from every rank's interval log-weights.
    Returns (resample?, [(dst_rank, dst_idx, src_rank, src_idx)], logZ increment)."""
    n_local = int(weights_by_rank[0].numel())
    iw = torch.cat([w.double().cpu() for w in weights_by_rank])
    N = iw.numel()
    w = smc_math.normalize_log_weights(iw)
    ess = float(1.0 / (w * w).sum())
    if N < 2 or threshold <= 0 or not ess < threshold * N:
        return False, [], 0.0
    u = smc_math.philox_uniform(seed, step, row)
    dst, src = smc_math.resample_plan(w, u)
    jobs = [(d // n_local, d % n_local, s // n_local, s % n_local) for d, s in zip(dst, src)]
    return True, jobs, float(smc_math.logz_increment(iw))


def apply_reference(states, kv_pools_by_rank, jobs, row: int) -> None:
    """Plain-PyTorch execution of a global plan over per-rank SlotStates living in one process.
    ``kv_pools_by_rank[r]`` is the list of KV pools (target, draft) of rank r."""
    for dr, di, sr, si in jobs:
        dst_st, src_st = states[dr], states[sr]
        dslot = dst_st.row_slots[row][di]
        sslot = src_st.row_slots[row][si]
        if dr == sr:
            dst_st._copy_particle(dslot, sslot)
            continue
        P = int(dst_st.prompt_lens[dslot])
        Ld, Ls = int(dst_st.seq_lens[dslot]), int(src_st.seq_lens[sslot])
        if Ld > P:
            dst_st.alloc.dec_ref_and_free(dst_st.bt.table[dslot, P:Ld].clone())
        new_pages = dst_st.alloc.alloc(Ls - P)
        dst_st.bt.table[dslot, P:Ls] = new_pages
        src_pages = src_st.bt.table[sslot, P:Ls].long()
        for pd, ps in zip(kv_pools_by_rank[dr], kv_pools_by_rank[sr]):
            pd.k[:, new_pages.long()] = ps.k[:, src_pages].to(pd.k.device)
            pd.v[:, new_pages.long()] = ps.v[:, src_pages].to(pd.v.device)
        for f in ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished", "finished_len", "finish_code",
                  "matched_eos"):
            getattr(dst_st, f)[dslot] = getattr(src_st, f)[sslot].to(dst_st.device)
        n = int(src_st.token_counts[sslot])
        dst_st.all_token_ids[dslot, :n] = src_st.all_token_ids[sslot, :n].to(dst_st.device)
        for pd, ps in zip(dst_st.state_pools, src_st.state_pools):
            pd.conv[:, dslot] = ps.conv[:, sslot].to(pd.conv.device)
            pd.temporal[:, dslot] = ps.temporal[:, sslot].to(pd.temporal.device)


# ----------------------------------------------------------------------------------- kernel path
class PpTensor(C.Structure):
    _fields_ = [("base", C.c_ulonglong), ("layer_stride", C.c_longlong), ("row_bytes", C.c_longlong),
                ("n_layers", C.c_int), ("by_slot", C.c_int)]


class PpRank(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in SLOT_FIELDS + ("block_table", "group_to_slots")] + [("t", PpTensor * 8)]


class PpWorld(C.Structure):
    _fields_ = [("r", PpRank * 8), ("heap_base", C.c_ulonglong * 8), ("n_ranks", C.c_int), ("rank", C.c_int),
                ("n_tensors", C.c_int), ("n_local", C.c_int), ("max_out", C.c_int), ("bt_stride", C.c_int),
                ("max_groups", C.c_int), ("pad", C.c_int)]


class PpLocal(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished",
                                         "finished_len", "finish_code", "matched_eos", "all_token_ids", "block_table",
                                         "prompt_lens", "log_weights", "interval_weights", "refcount", "free_stack",
                                         "free_count", "alloc_error")] + [("n_pages", C.c_int)]


def _tensor_desc(t: torch.Tensor, by_slot: bool, addr: int) -> Tuple[int, int, int, int, int]:
    es = t.element_size()
    return addr, t.stride(0) * es, t[0, 0].numel() * es, t.shape[0], int(by_slot)


class ParticleParallel:
    """Drives the particle-parallel resampling kernels for one rank.

    ``addr(rank, tensor_on_this_rank) -> int`` returns the address at which ``rank`` holds its copy of
    the given local tensor (same offset in the symmetric heap on real ranks; an explicit table in a
    single-GPU emulation).  ``comm_base[r]`` / offsets locate the gather buffer and the two counters."""

    def __init__(self, st, ns, kv_pools, rank: int, world: int, addr: Callable[[int, torch.Tensor], int],
                 comm_base: List[int], comm_local: torch.Tensor, status: torch.Tensor):
        from ..ops import native as K
        self.K = K
        L = K.lib()
        vp, i, ll, d, ull = C.c_void_p, C.c_int, C.c_longlong, C.c_double, C.c_ulonglong
        L.smc_pp_share_weights.argtypes = [vp, vp, vp, vp, i, vp, ll, ll, vp]
        L.smc_pp_collect.argtypes = [vp, vp, vp, vp, vp, i, vp, d, ull, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
        L.smc_pp_fetch.argtypes = [vp, vp, i, vp, vp, vp, vp, vp, i, i, i, vp, vp]
        L.smc_pp_barrier.argtypes = [vp, ll, vp, vp, vp, i, vp]
        L.smc_resample_apply.argtypes = [vp, vp, vp, vp, i, vp]
        for n in ("smc_pp_share_weights", "smc_pp_collect", "smc_pp_fetch", "smc_pp_barrier", "smc_resample_apply",
                  "smc_pp_world_size", "smc_pp_local_size"):
            getattr(L, n).restype = C.c_int
        assert C.sizeof(PpWorld) == L.smc_pp_world_size() and C.sizeof(PpLocal) == L.smc_pp_local_size()
        self.L = L
        self.st, self.ns, self.rank, self.world = st, ns, rank, world
        self.status = status
        dev = st.device
        tensors = []
        for pool in kv_pools:
            tensors += [(pool.k, False), (pool.v, False)]
        for pool in st.state_pools:
            tensors += [(pool.conv, True), (pool.temporal, True)]
        assert len(tensors) <= 8
        self.total_layers = sum(t.shape[0] for t, _ in tensors)
        w = PpWorld()
        for r in range(world):
            for f in SLOT_FIELDS:
                setattr(w.r[r], f, addr(r, getattr(st, f)))
            w.r[r].block_table = addr(r, st.bt.table)
            w.r[r].group_to_slots = addr(r, st.group_to_slots)
            for ti, (t, by_slot) in enumerate(tensors):
                a, ls, rb, nl, bs_ = _tensor_desc(t, by_slot, addr(r, t))
                w.r[r].t[ti].base, w.r[r].t[ti].layer_stride, w.r[r].t[ti].row_bytes = a, ls, rb
                w.r[r].t[ti].n_layers, w.r[r].t[ti].by_slot = nl, bs_
                assert rb % 16 == 0
            w.heap_base[r] = comm_base[r]
        w.n_ranks, w.rank, w.n_tensors, w.n_local = world, rank, len(tensors), st.N
        w.max_out, w.bt_stride, w.max_groups = st.max_output_len, st.bt.table.stride(0), st.max_groups
        self.world_host = w
        raw = bytes(w)
        self.world_dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
        loc = PpLocal()
        for f in ("seq_lens", "verified_ids", "prev_ids", "token_counts", "finished", "finished_len", "finish_code",
                  "matched_eos", "all_token_ids", "prompt_lens", "log_weights", "interval_weights"):
            setattr(loc, f, getattr(st, f).data_ptr())
        loc.block_table = st.bt.table.data_ptr()
        loc.refcount, loc.free_stack = st.alloc.refcount.data_ptr(), st.alloc.free_stack.data_ptr()
        loc.free_count, loc.alloc_error = st.alloc.free_count.data_ptr(), st.alloc.error_flag.data_ptr()
        loc.n_pages = st.alloc.size
        self.loc = loc
        # communication area (same layout on every rank): gather doubles, then two 64-bit counters
        self.gather_off = 0
        n_gather = world * st.max_groups * (st.N + 1)
        self.flag_w_off = (n_gather * 8 + 255) // 256 * 256
        self.flag_b_off = self.flag_w_off + 256
        self.comm_bytes = self.flag_b_off + 256
        assert comm_local.numel() >= self.comm_bytes
        self.comm_local = comm_local
        max_jobs = st.max_slots
        i32 = dict(dtype=torch.int32, device=dev)
        self.rjob_dst, self.rjob_rank = torch.zeros(max_jobs, **i32), torch.zeros(max_jobs, **i32)
        self.rjob_idx, self.rjob_src = torch.zeros(max_jobs, **i32), torch.zeros(max_jobs, **i32)

    @staticmethod
    def comm_bytes_needed(world: int, max_groups: int, n_local: int) -> int:
        return (world * max_groups * (n_local + 1) * 8 + 255) // 256 * 256 + 512

    def _s(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _chk(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with code {rc}")

    def share(self) -> None:
        st, ns = self.st, self.ns
        ns.sync_membership(st)
        self._chk(self.L.smc_pp_share_weights(self.world_dev.data_ptr(), st.interval_weights.data_ptr(),
                                              st.finished.data_ptr(), ns.active_rows.data_ptr(), ns.n_groups, st.group_to_slots.data_ptr(),
                                              self.gather_off, self.flag_w_off, self._s()), "pp_share_weights")

    def collect_and_apply(self, release_only: bool = False, phase: int = 0) -> None:
        """phase 0: everything; 1: collect + local jobs + release of remote destinations; 2: adopt + copy."""
        st, ns, L = self.st, self.ns, self.L
        base = self.comm_local.data_ptr()
        if phase in (0, 1):
            st.counters[1].zero_()
            st.counters[3].zero_()
            self._chk(L.smc_pp_collect(self.world_dev.data_ptr(), C.byref(self.loc), base + self.gather_off,
                                       base + self.flag_w_off, ns.active_rows.data_ptr(), ns.n_groups,
                                       st.group_to_slots.data_ptr(), float(st.threshold), st.seed & (2**64 - 1),
                                       st.counters.data_ptr(), st.group_log_Z.data_ptr(), ns.job_dst.data_ptr(),
                                       ns.job_src.data_ptr(), self.rjob_dst.data_ptr(), self.rjob_rank.data_ptr(),
                                       self.rjob_idx.data_ptr(), st.group_active.data_ptr(), self.status.data_ptr(),
                                       self._s()), "pp_collect")
            max_jobs = ns.n_groups * st.N
            self._chk(L.smc_resample_apply(C.byref(ns._arrays), st.counters.data_ptr(), ns.job_dst.data_ptr(),
                                           ns.job_src.data_ptr(), max_jobs, self._s()), "resample_apply")
            for pool in st.state_pools:
                self.K.state_copy(pool.conv, pool.conv.shape[0], pool.n_rows, st.counters, ns.job_dst, ns.job_src,
                                  max_jobs)
                self.K.state_copy(pool.temporal, pool.temporal.shape[0], pool.n_rows, st.counters, ns.job_dst,
                                  ns.job_src, max_jobs)
        max_jobs = ns.n_groups * st.N
        fetch_phase = {0: 0, 1: 1, 2: 2}[phase]
        self._chk(L.smc_pp_fetch(self.world_dev.data_ptr(), C.byref(self.loc), st.bt.table.stride(0),
                                 st.counters.data_ptr(), self.rjob_dst.data_ptr(), self.rjob_rank.data_ptr(),
                                 self.rjob_idx.data_ptr(), self.rjob_src.data_ptr(), max_jobs, self.total_layers,
                                 fetch_phase, self.status.data_ptr(), self._s()), "pp_fetch")

    def barrier(self, phase: int = 0) -> None:
        base = self.comm_local.data_ptr()
        self._chk(self.L.smc_pp_barrier(self.world_dev.data_ptr(), self.flag_b_off, base + self.flag_b_off,
                                        self.st.counters.data_ptr(), self.status.data_ptr(), phase, self._s()),
                  "pp_barrier")

    def resample(self) -> None:
        """One rank's whole resampling step (real multi-GPU ranks call this once per cycle)."""
        self.share()
        self.collect_and_apply()
        self.barrier()


# ----------------------------------------------------------------------------------- engine-facing drivers
class PpHost:
    """Host-side helpers shared by both execution paths (object gathers at finalize)."""

    def __init__(self, group, rank: int, world: int):
        self.group, self.rank, self.world = group, rank, world

    def all_gather_objects(self, obj):
        import torch.distributed as dist
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def align(self) -> None:
        """Host rendezvous of the ranks after the device has drained.  The in-kernel waits on peers are bounded (about a
        second); host work whose length differs per rank (first-launch module loading, a prefill, a graph capture)
        is followed by this call so that no rank enters a cycle's exchange far ahead of the others."""
        import datetime
        import os

        import torch.distributed as dist
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        # a rank that never arrives (it died, or it took another path through the scheduler) ends this wait with an
        # error that names it, instead of blocking the others for the process group's half-hour default
        limit = datetime.timedelta(seconds=float(os.environ.get("SMC_PP_ALIGN_TIMEOUT_S", "300")))
        if dist.get_backend(self.group) == "gloo":
            dist.monitored_barrier(group=self.group, timeout=limit)
        else:
            dist.barrier(group=self.group)


class PpTorch(PpHost):
    """Particle-parallel resampling over ``torch.distributed`` (gloo on CPU ranks): the plumbing path and the
    oracle of the kernel path.  Payloads of cross-rank ancestors travel as broadcast objects."""

    def __init__(self, group, rank: int, world: int, kv_pools):
        super().__init__(group, rank, world)
        self.kv_pools = kv_pools

    def _export(self, st, slot: int) -> dict:
        P, L = int(st.prompt_lens[slot]), int(st.seq_lens[slot])
        pages = st.bt.table[slot, P:L].long()
        n = int(st.token_counts[slot])
        return dict(
            L=L, n=n, tokens=st.all_token_ids[slot, :n].cpu(),
            scal={f: getattr(st, f)[slot].cpu() for f in ("verified_ids", "prev_ids", "token_counts", "finished",
                                                          "finished_len", "finish_code", "matched_eos")},
            kv=[(p.k[:, pages].cpu(), p.v[:, pages].cpu()) for p in self.kv_pools],
            state=[(p.conv[:, slot].cpu(), p.temporal[:, slot].cpu()) for p in st.state_pools])

    def _import(self, st, slot: int, pay: dict) -> None:
        P, Ld = int(st.prompt_lens[slot]), int(st.seq_lens[slot])
        if Ld > P:
            st.alloc.dec_ref_and_free(st.bt.table[slot, P:Ld].clone())
        L = pay["L"]
        new_pages = st.alloc.alloc(L - P)
        if new_pages is None:
            raise RuntimeError("KV page pool exhausted while adopting a remote ancestor")
        st.bt.table[slot, P:L] = new_pages
        for p, (k, v) in zip(self.kv_pools, pay["kv"]):
            p.k[:, new_pages.long()] = k.to(p.k.device)
            p.v[:, new_pages.long()] = v.to(p.v.device)
        st.seq_lens[slot] = L
        for f, val in pay["scal"].items():
            getattr(st, f)[slot] = val.to(st.device)
        st.all_token_ids[slot, :pay["n"]] = pay["tokens"].to(st.device)
        for p, (c, t) in zip(st.state_pools, pay["state"]):
            p.conv[:, slot] = c.to(p.conv.device)
            p.temporal[:, slot] = t.to(p.temporal.device)

    def resample_torch(self, st) -> int:
        import torch.distributed as dist
        rows = st.active_rows_host
        if not rows:
            return 0
        n_local = st.N
        # running particles per group over all ranks (drives the identical drain decision on every rank)
        alive = torch.zeros(st.max_groups, dtype=torch.int32)
        w_local = torch.zeros(len(rows), n_local, dtype=torch.float64)
        for i, row in enumerate(rows):
            idx = torch.tensor(st.row_slots[row], dtype=torch.long, device=st.device)
            alive[row] = int((~st.finished[idx]).sum())
            w_local[i] = st.interval_weights[idx].cpu()
        dist.all_reduce(alive, group=self.group)
        st.group_active.copy_(alive.to(st.device))
        gathered = [torch.zeros_like(w_local) for _ in range(self.world)]
        dist.all_gather(gathered, w_local, group=self.group)
        # every rank derives the same plans; ancestors are never destinations, so everything another rank needs from
        # this one can be exported before any job is applied and exchanged in one collective per cycle
        plans = []
        exports = {}
        for i, row in enumerate(rows):
            go, jobs, inc = plan_global([g[i] for g in gathered], st.threshold, st.seed, st.step, row)
            if not go:
                continue
            plans.append((row, jobs, inc))
            slots = st.row_slots[row]
            for dr, di, sr, si in jobs:
                if dr != sr and sr == self.rank and (row, si) not in exports:
                    exports[(row, si)] = self._export(st, slots[si])
        if not plans:
            return 0
        remote = self.all_gather_objects(exports)
        for row, jobs, inc in plans:
            slots = st.row_slots[row]
            for dr, di, sr, si in jobs:
                if dr != self.rank:
                    continue
                if sr == self.rank:
                    st._copy_particle(slots[di], slots[si])
                else:
                    self._import(st, slots[di], remote[sr][(row, si)])
            idx = torch.tensor(slots, dtype=torch.long, device=st.device)
            st.interval_weights[idx] = 0.0
            st.log_weights[idx] = 0.0
            st.group_log_Z[row] += inc
        st.n_resamples += len(plans)
        return len(plans)


class PpNative(PpHost):
    """Kernel path: weight exchange, plan and cross-GPU gather all happen in kernels over the symmetric heap."""

    def __init__(self, group, rank: int, world: int, driver: ParticleParallel):
        super().__init__(group, rank, world)
        self.driver = driver

    def resample_native(self, st) -> None:
        self.driver.resample()
