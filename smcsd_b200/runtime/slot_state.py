"""Slot-major particle state: one persistent device tensor per per-particle field, group
lookup rows, and the per-cycle state transitions (page assignment, write-back,
ESS test + systematic resampling, ancestor copy, finalize).

Every transition has a plain-PyTorch implementation here (the CPU path and the oracle
for the kernels) and, on CUDA with the native backend, a fused sm_100a kernel
(``smcsd_b200/ops/csrc/smc_state.cu``) that works on the same tensors without any host
synchronisation, so the whole cycle can sit inside one CUDA graph.

Field inventory and semantics follow the reference's slot state
(smcsd/core/req_state.py:140-313 fields, :333-471 allocate, :593-652 prepare,
:759-947 write-back, :1015-1079 finalize) and its resampling coordinator
(smcsd/core/scheduler.py:83-199, :839-914).  Differences that are deliberate here:
block-table row == slot id (no second indirection), int32 device fields, the page
free list lives on the device, and freed pages return to it inside the resample step
rather than through a one-step-late host buffer.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..memory.pools import BlockTable, PageAllocator, StatePool
from ..smc import math as smc_math
from ..smc.math import EMPTY_SLOT, FINISH_EOS, FINISH_LENGTH, FINISH_NONE, MAX_EOS


@dataclass
class CycleInputs:
    """What one decode cycle reads: produced by ``prepare_cycle``."""
    slots: torch.Tensor         # [bs] active slot ids (int32)
    orig_seq_lens: torch.Tensor  # [bs] S at cycle start
    x0: torch.Tensor            # [bs] verified id (token at position S)
    prev: torch.Tensor          # [bs] token at position S-1 (draft KV possibly pending)
    cache_locs: torch.Tensor    # [bs, gamma+1] fresh pages for positions S..S+gamma


@dataclass
class CycleOutputs:
    tokens: torch.Tensor        # [bs, gamma+1] = d0..d_{gamma-1}, bonus
    logprob_diff: torch.Tensor  # [bs, gamma] alpha*log p_target - log q_draft per position
    bonus_logz: Optional[torch.Tensor]  # [bs] or None


class HostSnapshot:
    """Pinned copy of the fields the host loop needs, guarded by an event (never a stream sync)."""

    def __init__(self, n_slots: int, device: torch.device):
        pin = device.type == "cuda"
        self.finished = torch.zeros(n_slots, dtype=torch.bool, pin_memory=pin)
        self.scalars = torch.zeros(4, dtype=torch.int32, pin_memory=pin)   # free_count, alloc_error, device status, -
        self.resampled = torch.zeros(1, dtype=torch.int64, pin_memory=pin)   # cumulative count of resampled groups
        self.group_active = None            # [max_groups] running particles per group over all ranks (particle-parallel)
        self.event = torch.cuda.Event() if pin else None

    def wait(self) -> None:
        if self.event is not None:
            self.event.synchronize()

    @property
    def free_pages(self) -> int:
        return int(self.scalars[0])

    @property
    def alloc_error(self) -> bool:
        return bool(self.scalars[1])

    @property
    def device_status(self) -> int:
        """Status word of the kernels as of this cycle (0: no wait ran out, no index failed its check)."""
        return int(self.scalars[2])


class SlotState:
    def __init__(self, *, max_groups: int, n_particles: int, gamma: int, max_output_len: int,
                 block_table: BlockTable, allocator: PageAllocator, device, seed: int = 0,
                 resample_threshold: float = 0.5, resample_method: str = "systematic",
                 state_pools: Sequence[StatePool] = (), native=None):
        self.max_groups = max_groups
        self.N = n_particles
        self.gamma = gamma
        self.G = gamma + 1
        self.max_slots = max_groups * n_particles
        self.max_output_len = max_output_len
        self.bt = block_table
        self.alloc = allocator
        self.device = torch.device(device)
        self.seed = seed
        self.threshold = resample_threshold
        self.method = resample_method
        self.state_pools = list(state_pools)
        self.native = native        # module with fused kernels, or None for the torch path
        S, dev = self.max_slots, self.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.seq_lens = torch.zeros(S, **i32)
        self.verified_ids = torch.zeros(S, **i32)
        self.prev_ids = torch.zeros(S, **i32)
        self.token_counts = torch.zeros(S, **i32)
        self.finished = torch.zeros(S, dtype=torch.bool, device=dev)
        self.finished_len = torch.zeros(S, **i32)
        self.finish_code = torch.zeros(S, **i32)
        self.matched_eos = torch.zeros(S, **i32)
        self.ignore_eos = torch.zeros(S, dtype=torch.bool, device=dev)
        self.max_new_tokens = torch.zeros(S, **i32)
        self.prompt_lens = torch.zeros(S, **i32)          # length of the shared (replicated) prompt prefix
        self.eos_ids = torch.full((S, MAX_EOS), -1, **i32)
        self.log_weights = torch.zeros(S, dtype=torch.float64, device=dev)
        self.interval_weights = torch.zeros(S, dtype=torch.float64, device=dev)
        self.all_token_ids = torch.zeros(S, max_output_len, **i32)
        self.group_to_slots = torch.full((max_groups, n_particles), EMPTY_SLOT, **i32)
        self.row_in_use = torch.zeros(max_groups, dtype=torch.bool, device=dev)
        self.group_log_Z = torch.zeros(max_groups, dtype=torch.float64, device=dev)
        self.group_active = torch.zeros(max_groups, **i32)    # particle-parallel: running particles per group, all ranks
        self.pp = None                                        # particle-parallel driver (None: all particles are local)
        self.device_status = None                             # status word of the kernel chains (kernel backend only)
        # device-side counters: [0] cycle step (Philox counter), [1] resample jobs this cycle,
        # [2] groups resampled in total
        self.counters = torch.zeros(4, dtype=torch.int64, device=dev)
        self.step = 0
        self.n_resamples = 0
        # host bookkeeping
        self.free_slots = deque(range(S))
        self.free_rows = list(range(max_groups - 1, -1, -1))
        self.group_rows: Dict[str, int] = {}
        self.row_slots: Dict[int, List[int]] = {}
        self.active_rows_host: List[int] = []
        self.version = 0
        self.active_slots = torch.zeros(0, **i32)
        self.active_rows = torch.zeros(0, **i32)
        self._snapshots = [HostSnapshot(S, dev), HostSnapshot(S, dev)]
        self._phase = 0
        self._pin = dev.type == "cuda"

    # ------------------------------------------------------------------ uploads
    def _upload(self, values, dtype) -> torch.Tensor:
        t = torch.tensor(values, dtype=dtype)
        if self._pin:
            return t.pin_memory().to(self.device, non_blocking=True)
        return t.to(self.device)

    # ------------------------------------------------------------------ membership
    def can_admit(self) -> bool:
        return len(self.free_slots) >= self.N and bool(self.free_rows)

    def allocate_group(self, group_id: str, *, prompt_len: int, x0: int, last_prompt_token: int,
                       max_new_tokens: int, ignore_eos: bool, eos_ids: Sequence[int],
                       parent_row: Optional[int] = None) -> int:
        """Claim N slots and a group row (fan-out 1 -> N).  With ``parent_row`` given, the
        parent's first ``prompt_len`` block-table entries are copied to every particle row
        (one reference each), its recurrent state is copied to every particle, and the
        parent's own reference is dropped (refcount N+1 -> N)."""
        if not self.can_admit():
            raise RuntimeError("no free slots / group rows")
        slots = [self.free_slots.popleft() for _ in range(self.N)]
        row = self.free_rows.pop()
        self.group_rows[group_id] = row
        self.row_slots[row] = slots
        idx = self._upload(slots, torch.int64)
        if parent_row is not None:
            self.bt.copy_row(parent_row, idx, int(prompt_len), self.alloc)
            self.alloc.dec_ref_and_free(self.bt.table[parent_row, :int(prompt_len)])
            src = torch.full_like(idx, parent_row)
            for pool in self.state_pools:
                pool.copy_rows(idx, src)
        self.seq_lens.index_fill_(0, idx, int(prompt_len))
        self.prompt_lens.index_fill_(0, idx, int(prompt_len))
        self.verified_ids.index_fill_(0, idx, int(x0))
        # seeded with the last committed token so the first deferred head rewrites S-1 idempotently
        self.prev_ids.index_fill_(0, idx, int(last_prompt_token))
        self.token_counts.index_fill_(0, idx, 1)
        self.finished.index_fill_(0, idx, False)
        self.finished_len.index_fill_(0, idx, 0)
        self.finish_code.index_fill_(0, idx, FINISH_NONE)
        self.matched_eos.index_fill_(0, idx, -1)
        self.ignore_eos.index_fill_(0, idx, bool(ignore_eos))
        self.max_new_tokens.index_fill_(0, idx, int(max_new_tokens))
        eos = list(dict.fromkeys(int(e) for e in eos_ids))[:MAX_EOS]
        eos_row = eos + [-1] * (MAX_EOS - len(eos))
        self.eos_ids[idx] = self._upload([eos_row] * self.N, torch.int32)
        self.log_weights.index_fill_(0, idx, 0.0)
        self.interval_weights.index_fill_(0, idx, 0.0)
        self.all_token_ids[:, 0].index_fill_(0, idx, int(x0))
        ridx = self._upload([row], torch.int64)
        self.group_to_slots[row] = idx.to(torch.int32)
        self.row_in_use.index_fill_(0, ridx, True)
        self.group_log_Z.index_fill_(0, ridx, 0.0)
        self.active_rows_host.append(row)
        self._rebuild_active()
        return row

    def _rebuild_active(self) -> None:
        self.version += 1
        rows = self.active_rows_host
        slots: List[int] = []
        for r in rows:
            slots.extend(self.row_slots[r])
        self.active_slots = self._upload(slots, torch.int32) if slots else torch.zeros(0, dtype=torch.int32, device=self.device)
        self.active_rows = self._upload(rows, torch.int32) if rows else torch.zeros(0, dtype=torch.int32, device=self.device)

    @property
    def n_active_groups(self) -> int:
        return len(self.active_rows_host)

    @property
    def bs(self) -> int:
        return len(self.active_rows_host) * self.N

    def free_group(self, group_id: str) -> None:
        """Release a finished group's pages, state rows, slots and row."""
        row = self.group_rows.pop(group_id, None)
        if row is None:                       # already released (e.g. finalized by a snapshot that was still pending)
            return
        slots = self.row_slots.pop(row)
        idx = self._upload(slots, torch.int64)
        lens = self.seq_lens[idx].tolist()
        for s, L in zip(slots, lens):
            if L > 0:
                self.alloc.dec_ref_and_free(self.bt.table[s, :L])
        self.seq_lens.index_fill_(0, idx, 0)
        for pool in self.state_pools:
            pool.clear_rows(idx)
        ridx = self._upload([row], torch.int64)
        self.group_to_slots[row] = EMPTY_SLOT
        self.row_in_use.index_fill_(0, ridx, False)
        self.free_slots.extend(slots)
        self.free_rows.append(row)
        self.active_rows_host.remove(row)
        self._rebuild_active()

    # ------------------------------------------------------------------ cycle prologue
    def prepare_cycle(self) -> CycleInputs:
        """Assign gamma+1 fresh pages to every active row and advance its length."""
        slots = self.active_slots
        bs, G = int(slots.numel()), self.G
        if self.native is not None:
            return self.native.prepare_cycle(self, slots)
        sl = slots.long()
        S = self.seq_lens[sl].clone()
        pages = self.alloc.alloc(bs * G)
        if pages is None:
            raise RuntimeError("KV page pool exhausted (admission should have prevented this)")
        pages = pages.view(bs, G)
        cols = S.long().unsqueeze(1) + torch.arange(G, device=self.device).unsqueeze(0)
        self.bt.table[sl.unsqueeze(1), cols] = pages
        self.seq_lens[sl] = S + G
        return CycleInputs(slots=slots, orig_seq_lens=S, x0=self.verified_ids[sl].clone(),
                           prev=self.prev_ids[sl].clone(), cache_locs=pages)

    # ------------------------------------------------------------------ write-back
    def write_back(self, cin: CycleInputs, out: CycleOutputs) -> None:
        if self.native is not None:
            self.native.write_back(self, cin, out)
            return
        sl = cin.slots.long()
        G, gamma = self.G, self.gamma
        tokens = out.tokens.to(torch.int32)
        counts = self.token_counts[sl]
        r = smc_math.write_back_reference(tokens, out.logprob_diff, out.bonus_logz, counts, self.finished[sl],
                                          self.max_new_tokens[sl], self.ignore_eos[sl], self.eos_ids[sl])
        cols = counts.long().unsqueeze(1) + torch.arange(G, device=self.device).unsqueeze(0)
        ok = cols < self.max_output_len
        rows = sl.unsqueeze(1).expand_as(cols)
        self.all_token_ids[rows[ok], cols[ok]] = tokens[ok]
        self.token_counts[sl] = r["new_counts"].to(torch.int32)
        self.verified_ids[sl] = tokens[:, gamma]
        self.prev_ids[sl] = tokens[:, gamma - 1]
        newly = r["newly_finished"]
        self.finished[sl] = self.finished[sl] | newly
        self.finished_len[sl] = torch.where(newly, r["finished_len"].to(torch.int32), self.finished_len[sl])
        self.finish_code[sl] = torch.where(newly, r["finish_code"].to(torch.int32), self.finish_code[sl])
        self.matched_eos[sl] = torch.where(newly, r["matched_eos"].to(torch.int32), self.matched_eos[sl])
        self.log_weights[sl] += r["weight_inc"]
        self.interval_weights[sl] += r["weight_inc"]

    # ------------------------------------------------------------------ resampling
    def resample(self) -> int:
        """ESS test and systematic resampling for every active group; returns how many
        groups resampled (torch path) or -1 when the fused kernels ran (count stays on device)."""
        self.step += 1
        if self.native is not None:
            self.native.collect_and_resample(self)
            return -1
        if self.pp is not None:
            return self.pp.resample_torch(self)
        n_res = 0
        N = self.N
        if N < 2 or self.threshold <= 0.0:
            return 0
        for row in self.active_rows_host:
            slots = self.row_slots[row]
            idx = torch.tensor(slots, dtype=torch.long, device=self.device)
            iw = self.interval_weights[idx]
            w = smc_math.normalize_log_weights(iw)
            ess = float(1.0 / (w * w).sum())
            if not ess < self.threshold * N:
                continue
            if self.method == "systematic":
                u = smc_math.philox_uniform(self.seed, self.step, row)
                dst, src = smc_math.resample_plan(w, u)
            else:
                g = torch.Generator().manual_seed(self.seed * 1000003 + self.step * 131 + row)
                dst, src = smc_math.multinomial_plan(w.cpu(), g)
            self.group_log_Z[row] += smc_math.logz_increment(iw)
            for d, s in zip(dst, src):
                self._copy_particle(slots[d], slots[s])
            self.interval_weights[idx] = 0.0
            self.log_weights[idx] = 0.0
            n_res += 1
        self.n_resamples += n_res
        return n_res

    def _copy_particle(self, dst: int, src: int) -> None:
        Ld = int(self.seq_lens[dst])
        Ls = int(self.seq_lens[src])
        if Ld > 0:
            self.alloc.dec_ref_and_free(self.bt.table[dst, :Ld].clone())
        pages = self.bt.table[src, :Ls]
        self.bt.table[dst, :Ls] = pages
        self.alloc.inc_ref(pages)
        for f in (self.seq_lens, self.verified_ids, self.prev_ids, self.token_counts, self.finished,
                  self.finished_len, self.finish_code, self.matched_eos):
            f[dst] = f[src]
        n = int(self.token_counts[src])
        self.all_token_ids[dst, :n] = self.all_token_ids[src, :n]
        d = torch.tensor([dst], device=self.device)
        s = torch.tensor([src], device=self.device)
        for pool in self.state_pools:
            pool.copy_rows(d, s)

    # ------------------------------------------------------------------ host view
    def snapshot_to_host(self) -> HostSnapshot:
        snap = self._snapshots[self._phase]
        self._phase ^= 1
        snap.finished.copy_(self.finished, non_blocking=True)
        snap.scalars[0:1].copy_(self.alloc.free_count, non_blocking=True)
        snap.scalars[1:2].copy_(self.alloc.error_flag, non_blocking=True)
        snap.resampled.copy_(self.counters[2:3], non_blocking=True)     # groups resampled so far (device counter)
        if self.device_status is not None:
            snap.scalars[2:3].copy_(self.device_status[0:1], non_blocking=True)
        if self.pp is not None:
            if snap.group_active is None:
                snap.group_active = torch.zeros(self.max_groups, dtype=torch.int32, pin_memory=self._pin)
            snap.group_active.copy_(self.group_active, non_blocking=True)
        if snap.event is not None:
            snap.event.record()
        return snap

    def group_has_active(self, group_id: str, snap) -> bool:
        row = self.group_rows[group_id]
        if self.pp is not None:              # the count covers every rank's particles, so all ranks agree
            return int(snap.group_active[row]) > 0
        return not all(bool(snap.finished[s]) for s in self.row_slots[row])

    # ------------------------------------------------------------------ finalize
    def finalize_group(self, group_id: str, generator: Optional[torch.Generator] = None) -> dict:
        """Posterior sample of one particle plus the group's diagnostics (device reads; rare)."""
        row = self.group_rows[group_id]
        slots = self.row_slots[row]
        idx = torch.tensor(slots, dtype=torch.long, device=self.device)
        iw = self.interval_weights[idx].cpu()
        lw = self.log_weights[idx].cpu()
        log_z = float(self.group_log_Z[row].cpu() + torch.logsumexp(iw, 0) - math.log(self.N))
        probs = torch.softmax(lw, dim=0).float()
        pick = int(torch.multinomial(probs, 1, generator=generator))
        flen = self.finished_len[idx].tolist()
        counts = self.token_counts[idx].tolist()
        codes = self.finish_code[idx].tolist()
        matched = self.matched_eos[idx].tolist()
        hist = self.all_token_ids[idx].cpu()
        outs = []
        for j in range(self.N):
            n = flen[j] if codes[j] != FINISH_NONE else counts[j]
            outs.append(hist[j, : min(n, self.max_output_len)].tolist())
        if self.pp is not None:
            # every rank contributes its particles; all ranks end up with the same global view and pick
            parts = self.pp.all_gather_objects(dict(outs=outs, lw=lw.tolist(), iw=iw.tolist(), codes=codes,
                                                    matched=matched))
            outs = [o for p_ in parts for o in p_["outs"]]
            codes = [c for p_ in parts for c in p_["codes"]]
            matched = [m for p_ in parts for m in p_["matched"]]
            lw = torch.tensor([x for p_ in parts for x in p_["lw"]], dtype=torch.float64)
            iw = torch.tensor([x for p_ in parts for x in p_["iw"]], dtype=torch.float64)
            log_z = float(self.group_log_Z[row].cpu() + torch.logsumexp(iw, 0) - math.log(iw.numel()))
            probs = torch.softmax(lw, dim=0).float()
            pick = int(torch.multinomial(probs, 1, generator=generator))
        reason = {"type": "length", "length": len(outs[pick])} if codes[pick] == FINISH_LENGTH else (
            {"type": "stop", "matched": matched[pick]} if codes[pick] == FINISH_EOS else {"type": "abort"})
        return dict(output_ids=outs[pick], finish_reason=reason, picked=pick, particle_output_ids=outs,
                    log_Z_hat=log_z, log_w_tilde=lw.tolist())

    # ------------------------------------------------------------------ leak check
    def held_pages(self) -> int:
        """Distinct pages referenced by live slots (for the idle-time leak check)."""
        pages = []
        for row, slots in self.row_slots.items():
            for s in slots:
                L = int(self.seq_lens[s])
                pages.append(self.bt.table[s, :L])
        if not pages:
            return 0
        return int(torch.unique(torch.cat(pages)).numel())
