"""Tensor-parallel kernel chain for a dense Llama-style target over NVLink peer memory.

Column-parallel GEMMs (QKV, gate/up, lm_head) consume activations that peers all-gathered into
local memory by kernel-issued stores; row-parallel GEMMs (o_proj, down) finish with a
reduce-scatter epilogue that stores reduced token rows into the owning rank's buffer.  The
residual stream is token-row sharded between them.  No NCCL call appears on this path; the only
synchronisation is a handful of monotonically increasing counters in the symmetric heap, waited
on with bounded spins inside the kernels.  The reference gets the same data flow from SGLang's
TP layers with NCCL all-reduce / all-gather (smcsd/engine.py:78,112, smcsd/core/worker.py:688-695).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import native as K


class TpContext:
    """Symmetric-heap carve-up shared by the TP kernels of one model."""

    FLAG_NAMES = ("ag_a", "ag_b", "rs_o", "rs_down", "sample")

    def __init__(self, heap, rank: int, tp: int, max_tokens: int, d: int, nchunks: int, device):
        self.heap, self.rank, self.tp = heap, rank, tp
        self.max_tokens, self.d, self.nchunks = max_tokens, d, nchunks
        self.rpr_max = (max_tokens + tp - 1) // tp
        self.off: Dict[str, int] = {}
        for n in self.FLAG_NAMES:
            self.off["flag_" + n] = heap.alloc("flag_" + n, 256)
        self.off["xn_a"] = heap.alloc("xn_a", max_tokens * d * 2)
        self.off["xn_b"] = heap.alloc("xn_b", max_tokens * d * 2)
        self.off["rs_o"] = heap.alloc("rs_o", tp * self.rpr_max * d * 4)
        self.off["rs_down"] = heap.alloc("rs_down", tp * self.rpr_max * d * 4)
        self.off["gather"] = heap.alloc("gather", tp * max_tokens * nchunks * 32)
        self.peers = K.TpPeers()
        for i in range(8):
            self.peers.base[i] = heap.ptrs[i] if i < tp else 0
        self.peers.tp, self.peers.rank = tp, rank
        self.base = heap.ptrs[rank]
        self.arrive = torch.zeros(8, dtype=torch.int32, device=device)   # local arrival counters per call site
        self.epoch = torch.zeros(1, dtype=torch.int64, device=device)

    def local_ptr(self, name: str) -> int:
        return self.base + self.off[name]

    def link(self, *, ag: Optional[str] = None, ag_uses: int = 1, ag_idx: int = 0, rs: Optional[str] = None,
             rows_per_rank: int = 1, arrive_slot: int = 0) -> K.TpLink:
        L = K.TpLink()
        L.ag_flag = self.local_ptr("flag_" + ag) if ag else None
        L.epoch = self.epoch.data_ptr()
        L.ag_uses, L.ag_idx, L.ag_inc = ag_uses, ag_idx, self.tp
        for i in range(8):
            L.peer_base[i] = self.peers.base[i]
        if rs:
            L.rs_off = self.off[rs]
            L.rs_flag_off = self.off["flag_" + rs]
        L.tp, L.rank, L.rows_per_rank = self.tp, self.rank, rows_per_rank
        L.arrive = self.arrive[arrive_slot:].data_ptr()
        return L


class NativeLlamaTP:
    """Same interface as ``NativeLlama`` for a model whose weights hold this rank's shard."""

    def __init__(self, model, kv, block_table, max_tokens, max_logit_rows, attn_splits, status, pdl, heap,
                 heap_view=None):
        self.m, self.kv, self.bt = model, kv, block_table
        c = model.cfg
        self.c = c
        dev = model.device
        self.T = max_tokens
        self.status, self.pdl = status, pdl
        self.tp, self.rank = model.tp_size, model.tp_rank
        self.nq, self.nkv, self.D = model.n_heads, model.n_kv_heads, c.head_dim
        self.d, self.ffn = c.hidden_size, model.ffn
        self.nqkv = (self.nq + 2 * self.nkv) * self.D
        self.Vshard = model.lm_head.shape[0]
        self.V = self.Vshard
        self.nchunks = 32
        self.ctx = TpContext(heap, self.rank, self.tp, max_tokens, self.d, self.nchunks, dev)
        view = heap_view or (lambda off, shape, dt: heap.view(off, shape, dt))
        o = self.ctx.off
        self.xn_a = view(o["xn_a"], (max_tokens, self.d), torch.bfloat16)
        self.xn_b = view(o["xn_b"], (max_tokens, self.d), torch.bfloat16)
        self.rs_o = view(o["rs_o"], (self.tp, self.ctx.rpr_max, self.d), torch.float32)
        self.rs_down = view(o["rs_down"], (self.tp, self.ctx.rpr_max, self.d), torch.float32)
        self.xn = self.xn_a
        f32, bf16 = torch.float32, torch.bfloat16
        self.h = torch.zeros(self.ctx.rpr_max, self.d, dtype=f32, device=dev)       # this rank's token rows
        self.attn = torch.empty(max_tokens, self.nq * self.D, dtype=bf16, device=dev)
        self.q = torch.empty(max_tokens, self.nq * self.D, dtype=bf16, device=dev)    # rotated queries (prompt passes)
        self.epoch_host = 0                  # forwards issued so far (the device epoch counts the same)
        self.act = torch.empty(max_tokens, self.ffn, dtype=bf16, device=dev)
        self.qkv = torch.empty(max_tokens, self.nqkv, dtype=f32, device=dev)
        self.ctx_hint = 0                    # context-length bound that sizes the attention key splits, see set_context
        self.part_acc = self.part_ml = torch.empty(1, dtype=f32, device=dev)     # unused by the fused kernel
        self.logits = torch.empty(max_logit_rows, self.Vshard, dtype=f32, device=dev)
        assert model.gu_block == 64 and (2 * self.ffn) % 128 == 0, "TP path needs the fused SwiGLU layout"
        self._splits_cache: Dict = {}

    def _splits(self, N, Kd, M):
        key = (N, Kd, M)
        if key not in self._splits_cache:
            self._splits_cache[key] = K.gemm_cluster_splits(N, Kd, M)
        return self._splits_cache[key]

    def forward(self, ids, positions, cache_locs, rows, prefix_lens, bs: int, E: int, two_pass: bool = False):
        for _ in self.stages(ids, positions, cache_locs, rows, prefix_lens, bs, E, two_pass):
            pass
        return self.xn_a

    def stages(self, ids, positions, cache_locs, rows, prefix_lens, bs: int, E: int, two_pass: bool = False):
        """The forward as a generator that yields after every kernel launch.  On real ranks it is
        simply exhausted; a single-GPU emulation of several ranks advances all ranks' generators in
        lockstep so that no kernel ever waits on a launch that comes later in the stream.
        ``two_pass`` (prompt passes): rows of one launch may be consecutive 16-token blocks of the same sequence, so
        every K/V row of this rank's heads is written before attention reads all keys through the block table."""
        m, c, pdl, ctx = self.m, self.c, self.pdl, self.ctx
        T = bs * E
        assert T <= self.T
        L = len(m.layers)
        tp = self.tp
        rpr = (T + tp - 1) // tp
        my_rows = max(0, min(rpr, T - self.rank * rpr))
        self._last_L = L
        ctx.epoch.add_(1)
        self.epoch_host += 1
        o = ctx.off
        st = self.status
        scale = self.D ** -0.5
        # embedding rows of this rank -> norm -> all-gather into xn_a
        K.tp_norm_allgather(ctx.peers, self.h, None, 0, 1, 0, tp, ctx.epoch, ids, m.embed, m.layers[0].ln1, o["xn_a"],
                            o["flag_ag_a"], rpr, my_rows, self.d, c.rms_eps, False, ctx.arrive[0:], st, pdl)
        yield
        for li, Lw in enumerate(m.layers):
            lk = ctx.link(ag="ag_a", ag_uses=L + 1, ag_idx=li)
            K.gemm_skinny_tp(Lw.wqkv, self.xn_a, self.qkv, M=T, splits=self._splits(self.nqkv, self.d, T),
                             epi=K.EPI_STORE_F32, link=lk, ldo=self.qkv.stride(0), status=st, pdl=pdl)
            yield
            q_in = None
            if two_pass:
                K.rope_kv_write(self.qkv, 1, 0, positions, cache_locs, m.rope, self.q, self.kv.k[li], self.kv.v[li],
                                M=T, Hq=self.nq, Hkv=self.nkv, D=self.D, status=st, pdl=pdl)
                q_in = self.q
            K.attention_fused(self.qkv, positions, cache_locs, m.rope, self.kv.k[li], self.kv.v[li], self.bt, rows,
                              prefix_lens, self.attn, self.part_acc, self.part_ml, bs=bs, E=E, Hq=self.nq,
                              Hkv=self.nkv, D=self.D, KS=self._ks(bs, E), scale=scale, status=st, pdl=pdl, q_in=q_in)
            yield
            lk = ctx.link(rs="rs_o", rows_per_rank=rpr, arrive_slot=1)
            K.gemm_skinny_tp(Lw.wo, self.attn, None, M=T, splits=self._splits(self.d, self.nq * self.D, T),
                             epi=K.EPI_RS_F32, link=lk, ldo=self.d, status=st, pdl=pdl)
            yield
            K.tp_norm_allgather(ctx.peers, self.h, self.rs_o, ctx.local_ptr("flag_rs_o"), L, li, tp, ctx.epoch, None,
                                None, Lw.ln2, o["xn_b"], o["flag_ag_b"], rpr, my_rows, self.d, c.rms_eps, False,
                                ctx.arrive[2:], st, pdl)
            yield
            lk = ctx.link(ag="ag_b", ag_uses=L, ag_idx=li)
            K.gemm_skinny_tp(Lw.wgu, self.xn_b, self.act, M=T, splits=self._gu_splits(T), epi=K.EPI_SWIGLU_BF16, link=lk,
                             ldo=self.act.stride(0), status=st, pdl=pdl)
            yield
            lk = ctx.link(rs="rs_down", rows_per_rank=rpr, arrive_slot=3)
            K.gemm_skinny_tp(Lw.wdown, self.act, None, M=T, splits=self._splits(self.d, self.ffn, T),
                             epi=K.EPI_RS_F32, link=lk, ldo=self.d, status=st, pdl=pdl)
            yield
            w_next = m.layers[li + 1].ln1 if li + 1 < L else m.final_norm
            K.tp_norm_allgather(ctx.peers, self.h, self.rs_down, ctx.local_ptr("flag_rs_down"), L, li, tp, ctx.epoch,
                                None, None, w_next, o["xn_a"], o["flag_ag_a"], rpr, my_rows, self.d, c.rms_eps, False,
                                ctx.arrive[4:], st, pdl)
            yield
        self._last_L = L


    def set_context(self, ctx: int, bs: int, Es=(1, 2)) -> tuple:
        """Record the context-length hint for the attention key splits; returns the splits chosen for forwards of
        ``Es`` new tokens per sequence (part of a captured graph's identity: they fix the launch grids)."""
        self.ctx_hint = int(ctx)
        return tuple(self._ks(bs, E) for E in Es)

    def _ks(self, bs: int, E: int) -> int:
        return K.attn_kv_splits(self.ctx_hint, bs, self.nkv, E, self.nq // self.nkv, self.D)

    def _gu_splits(self, M: int) -> int:
        key = ("gu", M)
        s = self._splits_cache.get(key)
        if s is None:
            s = self._splits_cache[key] = K.gemm_swiglu_splits(2 * self.ffn, self.d, M)
        return s

    def lm_head(self, rows: int, row_offset: int = 0, row_step: int = 1):
        """This rank's vocabulary shard of the logits [rows, Vshard] (waits for the last all-gather)."""
        L = self._last_L
        lk = self.ctx.link(ag="ag_a", ag_uses=L + 1, ag_idx=L)
        K.gemm_skinny_tp(self.m.lm_head, self.xn_a[row_offset:], self.logits, M=rows, splits=1, epi=K.EPI_STORE_F32,
                         link=lk, ldx=self.d * row_step, ldo=self.logits.stride(0), status=self.status, pdl=self.pdl)
        return self.logits

    def wait_final_rows(self) -> None:
        """Stream-ordered wait until every rank's rows of the last forward have landed in ``xn_a`` (for callers that
        read the gathered activations with ordinary kernels instead of a GEMM that waits by itself)."""
        L = self._last_L
        want = ((self.epoch_host - 1) * (L + 1) + L + 1) * self.tp
        if getattr(self, "_wait_outcome", None) is None:
            self._wait_outcome = torch.zeros(1, dtype=torch.int32, device=self.h.device)
        K.tp_wait_counter(self.ctx.local_ptr("flag_ag_a"), want, self._wait_outcome, self.status)

    def tp_sample(self, *, rows, temperature, alpha, tokens_in, seed, cycle_counter, call_id, tok_out, logp_out,
                  logz_out, phase: int = 0, epoch=None):
        """Vocab-parallel fused sampling / scoring: partials are exchanged by peer stores, every rank
        merges all shards and ends up with identical tokens and log-probabilities.  The exchange counter is expected
        to advance once per ``epoch`` tick: by default the forward counter (one sampling call per forward); callers
        that sample less often pass their own counter and bump it once per call."""
        ctx, c = self.ctx, self.c
        K.tp_sample_or_score(ctx.peers, self.logits, rows=rows, Vshard=self.Vshard, v0=self.rank * self.Vshard,
                             Vtotal=c.vocab_size, temperature=temperature, alpha=alpha,
                             softcap=float(c.logit_softcap), tokens_in=tokens_in, seed=seed,
                             cycle_counter=cycle_counter, call_id=call_id, gather_off=ctx.off["gather"],
                             gather_local_ptr=ctx.local_ptr("gather"), flag_off=ctx.off["flag_sample"],
                             flag_local_ptr=ctx.local_ptr("flag_sample"), uses=1, idx=0,
                             epoch=ctx.epoch if epoch is None else epoch,
                             nchunks=self.nchunks, tok_out=tok_out, logp_out=logp_out, logz_out=logz_out,
                             arrive=ctx.arrive[5:], status=self.status, pdl=self.pdl, phase=phase)
