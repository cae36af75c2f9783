"""The SMC decode cycle: prefill + x0, draft autoregression (deferred-bonus or legacy
schedule), one batched target verify, per-position log-weight differences and the bonus
token.  Two executions of the same cycle exist: this eager path over the model objects'
plain-PyTorch forwards (CPU, oracle, cuBLAS baseline) and the sm_100a kernel chain of
``ops/native_backend.py`` (captured as one CUDA graph per cycle) that the worker hands over to on a B200.

Algorithm per the reference worker (smcsd/core/worker.py:642-717 prefill and x0,
:780-891 deferred draft schedule, :1046-1092 legacy schedule, :1095-1166 verify,
weights and bonus).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..config import EngineArgs
from ..memory.pools import BlockTable, KVPool, PageAllocator, StatePool
from ..models.layers import ExtendBatch
from ..smc import math as smc_math
from .slot_state import CycleInputs, CycleOutputs


@dataclass
class PrefillItem:
    row: int                 # parent block-table row
    input_ids: List[int]


class SMCWorker:
    def __init__(self, args: EngineArgs, target, draft, kv_target: KVPool, kv_draft: KVPool,
                 block_table: BlockTable, allocator: PageAllocator,
                 state_target: Optional[StatePool] = None, state_draft: Optional[StatePool] = None,
                 native_runner=None, noise_rank: int = 0):
        self.args = args
        self.target, self.draft = target, draft
        self.kv_t, self.kv_d = kv_target, kv_draft
        self.bt, self.alloc = block_table, allocator
        self.state_t, self.state_d = state_target, state_draft
        self.device = block_table.table.device
        self.gamma = args.gamma
        self.G = args.gamma + 1
        self.T_draft = float(args.draft_temperature)
        self.T_target = float(args.target_temperature)
        self.alpha = float(args.power_alpha)
        self.defer_bonus = bool(args.defer_bonus)
        self.native = native_runner
        # x0 is shared by every particle of a group (and by every rank holding some of them): its noise comes
        # from a rank-independent stream; the decode noise differs per rank so particles stay distinct
        self.gen_prefill = torch.Generator(device=self.device)
        self.gen_prefill.manual_seed(int(args.random_seed) * 7919 + 17)
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(int(args.random_seed) * 7919 + 17 + 104729 * (noise_rank + 1) * (1 if noise_rank else 0))
        self.cycles = 0
        self.io_bytes = {"h2d": 0, "d2h": 0}

    # ------------------------------------------------------------------ prefill
    def prefill(self, items: Sequence[PrefillItem]) -> torch.Tensor:
        """Run target and draft over the full prompts and draw x0 from the target's tempered
        power distribution at each prompt's last token.  Returns x0 [n] (device tensor)."""
        if self.native is not None:
            return self.native.prefill(self, items)
        lens = [len(it.input_ids) for it in items]
        ids = torch.tensor([t for it in items for t in it.input_ids], dtype=torch.int64)
        if self.device.type == "cuda":          # prompts cross PCIe from pinned memory
            ids = ids.pin_memory().to(self.device, non_blocking=True)
            self.io_bytes["h2d"] += ids.numel() * 8
        pos = torch.cat([torch.arange(L, device=self.device) for L in lens])
        locs = torch.cat([self.bt.table[it.row, :L] for it, L in zip(items, lens)])
        rows = torch.tensor([it.row for it in items], dtype=torch.int32, device=self.device)
        zeros = torch.zeros(len(items), dtype=torch.int32, device=self.device)
        batch = ExtendBatch(ids, pos, locs, rows, zeros, extend_len=0, extend_lens=lens,
                            prefix_lens_host=[0] * len(items))
        hid = self.target.forward_torch(batch, self.kv_t, self.bt.table, self.state_t)
        last = torch.tensor(lens, device=self.device).cumsum(0) - 1
        logits = self.target.logits_torch(hid[last])
        x0, _, _ = smc_math.gumbel_sample(logits, self.T_target, self.alpha, generator=self.gen_prefill)
        # draft: full prompt for dense drafts; stateful drafts under the deferred schedule stop one
        # token short so the first head forward advances the recurrent state through S-1 exactly once
        if getattr(self.draft, "has_state", False) and self.defer_bonus:
            dl = [L - 1 for L in lens]
            keep = torch.cat([torch.arange(L - 1, device=self.device) + o
                              for L, o in zip(lens, [0] + list(torch.tensor(lens).cumsum(0)[:-1].tolist()))])
            dbatch = ExtendBatch(ids[keep], pos[keep], locs[keep], rows, zeros, extend_len=0, extend_lens=dl,
                                 prefix_lens_host=[0] * len(items))
        else:
            dbatch = batch
        if sum(dbatch.lens()) > 0:
            self.draft.forward_torch(dbatch, self.kv_d, self.bt.table, self.state_d)
        self.io_bytes["d2h"] += 4 * len(items)
        return x0.to(torch.int32)

    # ------------------------------------------------------------------ decode
    def decode_cycle(self, cin: CycleInputs) -> CycleOutputs:
        self.cycles += 1
        if self.native is not None:
            return self.native.decode_cycle(self, cin)
        if self.defer_bonus:
            drafts, logq = self._draft_deferred(cin)
        else:
            drafts, logq = self._draft_legacy(cin)
        return self._verify(cin, drafts, logq)

    def _sample_draft(self, logits: torch.Tensor):
        tok, logp, _ = smc_math.gumbel_sample(logits, self.T_draft, 1.0, generator=self.gen)
        return tok.to(torch.int32), logp

    def _draft_deferred(self, cin: CycleInputs):
        """gamma draft forwards: a two-token head [prev@S-1, x0@S] then gamma-1 single tokens.
        The KV write of d_{gamma-1} is left to the next cycle's head."""
        bs, gamma = cin.slots.numel(), self.gamma
        S = cin.orig_seq_lens.long()
        sl = cin.slots.long()
        # the S-1 page is looked up live: after a resample the row points at the ancestor's pages
        loc_prev = self.bt.table[sl, (S - 1)]
        ids = torch.stack([cin.prev.long(), cin.x0.long()], dim=1).reshape(-1)
        pos = torch.stack([S - 1, S], dim=1).reshape(-1)
        locs = torch.stack([loc_prev.long(), cin.cache_locs[:, 0].long()], dim=1).reshape(-1)
        # SMC accepts every token, so stateful models simply end the pass on the last token's state
        head = ExtendBatch(ids, pos, locs, cin.slots, (S - 1).to(torch.int32), extend_len=2)
        hid = self.draft.forward_torch(head, self.kv_d, self.bt.table, self.state_d)
        logits = self.draft.logits_torch(hid.view(bs, 2, -1)[:, 1])
        d, lq = self._sample_draft(logits)
        drafts, logqs = [d], [lq]
        for s in range(1, gamma):
            step = ExtendBatch(drafts[-1].long(), S + s, cin.cache_locs[:, s].long(), cin.slots,
                               (S + s).to(torch.int32), extend_len=1)
            hid = self.draft.forward_torch(step, self.kv_d, self.bt.table, self.state_d)
            d, lq = self._sample_draft(self.draft.logits_torch(hid))
            drafts.append(d)
            logqs.append(lq)
        return torch.stack(drafts, dim=1), torch.stack(logqs, dim=1)

    def _draft_legacy(self, cin: CycleInputs):
        """gamma+1 single-token forwards; the last one only writes KV (its sample is discarded)."""
        gamma = self.gamma
        S = cin.orig_seq_lens.long()
        cur = cin.x0
        drafts, logqs = [], []
        for s in range(gamma + 1):
            step = ExtendBatch(cur.long(), S + s, cin.cache_locs[:, s].long(), cin.slots,
                               (S + s).to(torch.int32), extend_len=1)
            hid = self.draft.forward_torch(step, self.kv_d, self.bt.table, self.state_d)
            if s == gamma:
                break
            d, lq = self._sample_draft(self.draft.logits_torch(hid))
            drafts.append(d)
            logqs.append(lq)
            cur = d
        return torch.stack(drafts, dim=1), torch.stack(logqs, dim=1)

    def _verify(self, cin: CycleInputs, drafts: torch.Tensor, logq: torch.Tensor) -> CycleOutputs:
        bs, gamma, G = cin.slots.numel(), self.gamma, self.G
        S = cin.orig_seq_lens.long()
        ids = torch.cat([cin.x0.view(bs, 1).long(), drafts.long()], dim=1)            # [bs, G]
        pos = S.unsqueeze(1) + torch.arange(G, device=self.device).unsqueeze(0)
        vb = ExtendBatch(ids.reshape(-1), pos.reshape(-1), cin.cache_locs.reshape(-1).long(), cin.slots,
                         cin.orig_seq_lens.to(torch.int32), extend_len=G)
        hid = self.target.forward_torch(vb, self.kv_t, self.bt.table, self.state_t)
        logits = self.target.logits_torch(hid).view(bs, G, -1)
        score = smc_math.chosen_logprob(logits[:, :gamma], drafts.long(), self.T_target)
        diff = self.alpha * score - logq
        bonus, _, logz = smc_math.gumbel_sample(logits[:, gamma], self.T_target, self.alpha, generator=self.gen)
        tokens = torch.cat([drafts.to(torch.int32), bonus.to(torch.int32).view(bs, 1)], dim=1)
        return CycleOutputs(tokens=tokens, logprob_diff=diff, bonus_logz=logz if self.alpha != 1.0 else None)
