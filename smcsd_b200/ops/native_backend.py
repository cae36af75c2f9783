"""The sm_100a execution path: model forwards as chains of the hand-written kernels, the SMC
state transitions as device kernels, and the whole decode cycle captured in one CUDA graph.

One cycle = prologue (page assignment) -> draft head + gamma-1 single draft steps, each followed
by the fused Gumbel sampler -> target verify -> fused scoring / bonus draw -> write-back -> ESS
test, systematic resampling and ancestor copy.  Nothing in it touches the host, so a replay is a
single launch and the host loop only reads a pinned snapshot one cycle later.  (The reference
captures draft + verify + scoring and leaves write-back / resampling as eager launches:
smcsd/model_executor/smc_draft_phase_graph_runner.py:824-1197, smcsd/core/scheduler.py:879-914.)
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..models.layers import ExtendBatch
from ..runtime.slot_state import CycleInputs, CycleOutputs
from . import native as K


# Shared-prefix group pass on the tcgen05 kernel instead of the mma.sync one (SMC_ATTN_TC): 0 never, 1 for forwards of
# more than two tokens per sequence (the verify shape, where its 128-row tiles are well filled), 2 always.
ATTN_TC_DEFAULT = 1


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    return default if v is None or v == "" else int(v)


def _env_flag(name: str, default: bool) -> bool:
    v = os.environ.get(name)
    return default if v is None else v.strip().lower() in ("1", "true", "yes", "on")


class NativeLlama:
    """Kernel-chain forward of a dense Llama-style model over a paged KV cache."""

    def __init__(self, model, kv, block_table: torch.Tensor, max_tokens: int, max_logit_rows: int,
                 attn_splits: int, status: torch.Tensor, pdl: bool):
        self.m, self.kv, self.bt = model, kv, block_table
        c = model.cfg
        self.c = c
        dev = model.device
        self.T = max_tokens
        self.status = status
        self.pdl = pdl
        self.attn_splits = attn_splits
        self.nq, self.nkv, self.D = model.n_heads, model.n_kv_heads, c.head_dim
        self.d, self.ffn = c.hidden_size, model.ffn
        self.nqkv = (self.nq + 2 * self.nkv) * self.D
        self.V = model.lm_head.shape[0]
        f32, bf16 = torch.float32, torch.bfloat16
        self.h = torch.empty(max_tokens, self.d, dtype=f32, device=dev)
        self.xn = torch.empty(max_tokens, self.d, dtype=bf16, device=dev)
        self.q = torch.empty(max_tokens, self.nq * self.D, dtype=bf16, device=dev)
        self.attn = torch.empty(max_tokens, self.nq * self.D, dtype=bf16, device=dev)
        self.act = torch.empty(max_tokens, self.ffn, dtype=bf16, device=dev)
        self.qkv = torch.empty(max_tokens, self.nqkv, dtype=f32, device=dev)
        self.ctx_hint = 0                    # context-length bound that sizes the attention key splits, see set_context
        self.part_acc = self.part_ml = torch.empty(1, dtype=f32, device=dev)     # unused by the fused kernel
        self.logits = torch.empty(max_logit_rows, self.V, dtype=f32, device=dev)
        self.fuse_swiglu = model.gu_block == 64 and (2 * self.ffn) % 128 == 0
        if not self.fuse_swiglu:
            self.gu = torch.empty(max_tokens, 2 * self.ffn, dtype=f32, device=dev)
        self._splits_cache: Dict = {}
        self._lm_parts = None                # per-(row, vocabulary slab) partials of the fused lm_head sampler
        # shared-prefix attention: parked state per (token, head) and, filled by the runner when the batch changes,
        # the per-sequence shared lengths and the block-table rows / shared lengths of every NP-th sequence
        self.att_state = torch.zeros(max_tokens, self.nq, self.D + 2, dtype=f32, device=dev)
        self.att_state_tc = None             # [key split, token, head, D + 2] states of the tcgen05 group pass
        self.cascade_bufs = None
        self._cascade: Dict = {}
        self.attn_tc = _env_int("SMC_ATTN_TC", ATTN_TC_DEFAULT)
        # RMSNorm folded into the GEMMs: consumers read the raw bf16 residual stream ``hb`` and scale by 1/rms in
        # their epilogue; residual GEMMs emit ``hb`` and per-slab sums of squares.  Five launches per layer.
        self.quant = getattr(model, "quantization", None)
        self.fold = self.fuse_swiglu and model.tp_size == 1 and _env_flag("SMC_FOLD_NORM", True) and self.quant is None
        if self.quant == "fp8":
            # W8A8: e4m3 weights with per-row scales (quantised once per model), per-token activation scales
            if not self.fuse_swiglu or model.tp_size != 1:
                raise ValueError("quantization='fp8' needs the fused SwiGLU layout and tp_size=1")
            if getattr(model, "_w8", None) is None:
                model._w8 = [{n: K.quantize_weight_e4m3(getattr(L, n)) for n in ("wqkv", "wo", "wgu", "wdown")}
                             for L in model.layers]
            wide = max(self.d, self.nq * self.D, self.ffn)
            self.x8 = torch.zeros(max_tokens, (wide + 15) // 16 * 16, dtype=torch.uint8, device=dev)
            self.xs = torch.zeros(max_tokens, dtype=f32, device=dev)
        if self.fold:
            model.fold_norms()
            self.hb = torch.empty(max_tokens, self.d, dtype=bf16, device=dev)
            self.n_parts = (self.d + 127) // 128
            self.ssq = torch.zeros(self.n_parts, max_tokens, dtype=f32, device=dev)

    def _forward_folded(self, ids, positions, cache_locs, rows, prefix_lens, bs: int, E: int, two_pass: bool):
        m, c, pdl = self.m, self.c, self.pdl
        T = bs * E
        K.add_rmsnorm(self.h, None, None, M=T, d=self.d, eps=c.rms_eps, ids=ids, embed=m.embed, hb=self.hb,
                      ssq=self.ssq, pdl=pdl)
        parts = 1
        scale = self.D ** -0.5
        ld = self.ssq.stride(0)
        for li, L in enumerate(m.layers):
            K.gemm_skinny_norm(L.wqkv, self.hb, self.qkv, M=T, splits=self._splits(self.nqkv, self.d, T),
                               epi=K.EPI_STORE_F32, ldo=self.qkv.stride(0), status=self.status, ssq_in=self.ssq,
                               ssq_parts=parts, norm_d=self.d, norm_eps=c.rms_eps, ssq_ld=ld, pdl=pdl)
            self._attention(li, positions, cache_locs, rows, prefix_lens, bs, E, two_pass, scale)
            K.gemm_skinny_norm(L.wo, self.attn, self.h, M=T, splits=self._splits(self.d, self.nq * self.D, T),
                               epi=K.EPI_RESID_F32, ldo=self.d, status=self.status, ssq_out=self.ssq, hb_out=self.hb,
                               ssq_ld=ld, pdl=pdl)
            parts = self.n_parts
            K.gemm_skinny_norm(L.wgu, self.hb, self.act, M=T, splits=self._gu_splits(T), epi=K.EPI_SWIGLU_BF16,
                               ldo=self.act.stride(0), status=self.status, ssq_in=self.ssq, ssq_parts=parts,
                               norm_d=self.d, norm_eps=c.rms_eps, ssq_ld=ld, pdl=pdl)
            K.gemm_skinny_norm(L.wdown, self.act, self.h, M=T, splits=self._splits(self.d, self.ffn, T),
                               epi=K.EPI_RESID_F32, ldo=self.d, status=self.status, ssq_out=self.ssq, hb_out=self.hb,
                               ssq_ld=ld, pdl=pdl)
        return self.hb

    def _attention(self, li: int, positions, cache_locs, rows, prefix_lens, bs: int, E: int, two_pass: bool,
                   scale: float) -> None:
        """Attention step of layer ``li``.  One fused launch (rope, KV write, attention) by default.  With a
        shared-prefix plan (see ``set_prefix``) three launches: rope + KV write, one pass over the prompt keys for
        several particles of a group at a time, then the per-particle pass over the remaining keys that folds the
        parked state in (the reference describes this "cascade" for decode: docs/smc/performance.md:116-128)."""
        m, pdl, T = self.m, self.pdl, bs * E
        k, v = self.kv.k[li], self.kv.v[li]
        plan = None if two_pass else self._cascade.get(E)
        if plan is None or bs % plan["NP"] != 0:
            q_in = None
            if two_pass:
                K.rope_kv_write(self.qkv, 1, 0, positions, cache_locs, m.rope, self.q, k, v, M=T, Hq=self.nq,
                                Hkv=self.nkv, D=self.D, status=self.status, pdl=pdl)
                q_in = self.q
            K.attention_fused(self.qkv, positions, cache_locs, m.rope, k, v, self.bt, rows, prefix_lens, self.attn,
                              bs=bs, E=E, Hq=self.nq, Hkv=self.nkv, D=self.D, KS=self._ks(bs, E), scale=scale,
                              status=self.status, pdl=pdl, q_in=q_in)
            return
        NP, cb = plan["NP"], self.cascade_bufs
        if not plan["tc"] and NP * E <= 16 and k.dtype != torch.uint8:
            # two launches: the group pass rotates its (at most 16) tokens' queries itself and writes nothing; the
            # per-particle pass is the ordinary step (rope, KV write, new-token tile) started behind the shared keys
            K.attention_fused(self.qkv, positions, cache_locs, m.rope, k, v, self.bt, cb["rows_g"][NP], cb["shared_g"][NP],
                              None, bs=bs // NP, E=NP * E, Hq=self.nq, Hkv=self.nkv, D=self.D, KS=plan["KSg"],
                              scale=scale, status=self.status, pdl=pdl, part_out=self.att_state, causal=False)
            K.attention_fused(self.qkv, positions, cache_locs, m.rope, k, v, self.bt, rows, prefix_lens, self.attn, bs=bs,
                              E=E, Hq=self.nq, Hkv=self.nkv, D=self.D, KS=plan["KSs"], scale=scale, status=self.status,
                              pdl=pdl, key_begin=cb["shared"], part_in=self.att_state)
            return
        if plan["tc"]:
            # two launches: the tcgen05 group pass rotates the queries itself and parks one state per key split; the
            # per-particle pass is the ordinary step (rope, KV write, new-token tile) started behind the shared keys
            if self.att_state_tc is None:
                self.att_state_tc = torch.zeros(8, self.T, self.nq, self.D + 2, dtype=torch.float32, device=self.h.device)
            K.attention_prefix_tc(None, k, v, self.bt, cb["rows_g"][NP], cb["shared_g"][NP], self.att_state_tc,
                                  n_seq=bs // NP, E=NP * E, T=self.T, Hq=self.nq, Hkv=self.nkv, D=self.D,
                                  KS=plan["KSg"], scale=scale, status=self.status, qkv=self.qkv, q_off=0,
                                  positions=positions, rope=m.rope, pdl=pdl)
            K.attention_fused(self.qkv, positions, cache_locs, m.rope, k, v, self.bt, rows, prefix_lens, self.attn,
                              bs=bs, E=E, Hq=self.nq, Hkv=self.nkv, D=self.D, KS=plan["KSs"], scale=scale,
                              status=self.status, pdl=pdl, key_begin=cb["shared"],
                              part_in=self.att_state_tc, part_in_n=plan["KSg"],
                              part_in_stride=self.att_state_tc.stride(0))
            return
        K.rope_kv_write(self.qkv, 1, 0, positions, cache_locs, m.rope, self.q, k, v, M=T, Hq=self.nq, Hkv=self.nkv,
                        D=self.D, status=self.status, pdl=pdl)
        K.attention_fused(self.qkv, positions, cache_locs, m.rope, k, v, self.bt, cb["rows_g"][NP], cb["shared_g"][NP],
                          None, bs=bs // NP, E=NP * E, Hq=self.nq, Hkv=self.nkv, D=self.D, KS=plan["KSg"], scale=scale,
                          status=self.status, pdl=pdl, q_in=self.q, part_out=self.att_state, causal=False)
        K.attention_fused(self.qkv, positions, cache_locs, m.rope, k, v, self.bt, rows, prefix_lens, self.attn, bs=bs,
                          E=E, Hq=self.nq, Hkv=self.nkv, D=self.D, KS=plan["KSs"], scale=scale, status=self.status,
                          pdl=pdl, q_in=self.q, key_begin=cb["shared"], part_in=self.att_state)

    def set_context(self, ctx: int, bs: int, Es=(1, 2)) -> tuple:
        """Record the context-length hint for the attention key splits; returns the splits chosen for forwards of
        ``Es`` new tokens per sequence (part of a captured graph's identity: they fix the launch grids)."""
        self.ctx_hint = int(ctx)
        return tuple(self._ks(bs, E) for E in Es)

    # Shortest shared prompt for which the extra launch per layer pays off.  Measured on B200 (8 particles, 256 own
    # tokens each): single-token steps with the mma.sync group pass 0.87x at 4k, 1.1x at 8k, 1.5x at 16k, 2.0x at 32k
    # prompt tokens.  The verify shape (9 tokens x 4 heads per particle) loses at every length with the mma.sync group
    # pass (bound by its issue rate) and wins with the tcgen05 one: pages scattered 0.83x at 4k, 1.1x at 8k, 1.25x at
    # 16k, 1.5x at 32k; prompt in consecutive pages 0.88x at 4k, 1.3x at 8k, 1.7x at 16k, 2.1x at 32k.
    # SMC_CASCADE_VERIFY=1 / 0 forces the verify-shape passes on / off.
    CASCADE_MIN_PROMPT = 8192
    CASCADE_MIN_PROMPT_VERIFY = 8192

    def set_prefix(self, min_prompt: int, max_prompt: int, bs: int, n_particles: int, Es=(1, 2)) -> tuple:
        """Plan the shared-prefix passes for forwards of ``Es`` new tokens per sequence: ``min_prompt`` / ``max_prompt``
        bound the prompt lengths of the running groups (all particles of a group share the prompt's pages).  Returns
        the plan's identity for the graph key (empty when the passes are off)."""
        self._cascade = {}
        thr = _env_int("SMC_CASCADE_MIN_PROMPT", self.CASCADE_MIN_PROMPT)
        if self.cascade_bufs is None or min_prompt < thr or thr <= 0:
            return ()
        G = self.nq // self.nkv
        key = []
        verify_env = os.environ.get("SMC_CASCADE_VERIFY", "")
        for E in Es:
            tc = self.D in (64, 128) and n_particles in self.cascade_bufs["rows_g"] and \
                (self.attn_tc >= 2 or (self.attn_tc == 1 and E > 2)) and self.kv.k.dtype != torch.uint8
            if E > 2:
                on = tc and min_prompt >= max(thr, self.CASCADE_MIN_PROMPT_VERIFY) if verify_env == "" else verify_env == "1"
                if not on:
                    continue
            NP = 0
            if tc:                                   # the tcgen05 pass tiles its query rows: whole groups at once
                NP = n_particles
                ksg = K.attention_tc_splits(bs // NP, self.nkv, max_prompt, NP * E * G)
            else:
                for cand in (8, 4, 2):
                    if n_particles % cand == 0 and cand * E * G <= 128 and cand in self.cascade_bufs["rows_g"]:
                        NP = cand
                        break
                if NP == 0:
                    continue
                n_mt = (NP * E * G + 15) // 16
                n_kw = max(1, 8 // n_mt)
                base = (bs // NP) * self.nkv
                ksg = 1
                while ksg < 8 and base * ksg * 2 <= 148 and max_prompt // (ksg * 2 * 32 * n_kw) >= 2:
                    ksg *= 2
            suffix = max(self.ctx_hint - min_prompt, 1)
            kss = K.attn_kv_splits(suffix, bs, self.nkv, E, G, self.D)
            self._cascade[E] = {"NP": NP, "KSg": ksg, "KSs": kss, "tc": tc}
            key.append((E, NP, ksg, kss, tc))
        return tuple(key)

    def _ks(self, bs: int, E: int) -> int:
        ks = K.attn_kv_splits(self.ctx_hint, bs, self.nkv, E, self.nq // self.nkv, self.D)
        cap = max(1, int(self.attn_splits))          # attention_num_kv_splits bounds the planner's choice (1 = never split)
        while ks > cap:
            ks //= 2
        return ks

    def final_hidden(self, rows_idx: torch.Tensor) -> torch.Tensor:
        """Post-final-norm hidden rows (bf16) for callers that project with PyTorch (x0 at prefill)."""
        from ..models.layers import rmsnorm
        if self.fold:
            return rmsnorm(self.h[rows_idx], self.m.final_norm, self.c.rms_eps).to(torch.bfloat16)
        return self.xn[rows_idx]

    def _splits(self, N: int, Kdim: int, M: int) -> int:
        key = (N, Kdim, M)
        s = self._splits_cache.get(key)
        if s is None:
            s = self._splits_cache[key] = K.gemm_cluster_splits(N, Kdim, M)
        return s

    def _gemm(self, W: torch.Tensor, X: torch.Tensor, out: torch.Tensor, M: int, epi: int, ldx: Optional[int] = None):
        """fp32 store / residual-accumulate GEMM; split-K is reduced on chip inside a CTA cluster."""
        N, Kdim = W.shape
        K.gemm_skinny(W, X, out, M=M, splits=self._splits(N, Kdim, M), epi=epi, ldx=ldx, ldo=out.stride(0),
                      status=self.status, pdl=self.pdl)

    def forward(self, ids: torch.Tensor, positions: torch.Tensor, cache_locs: torch.Tensor, rows: torch.Tensor,
                prefix_lens: torch.Tensor, bs: int, E: int, two_pass: bool = False) -> torch.Tensor:
        """Runs every layer for bs*E tokens; returns the final-norm activations ``xn`` [T, d] (bf16).
        ``two_pass`` (prefill): rows of one launch may be consecutive 16-token blocks of the same sequence, so all
        K/V rows are written by a separate kernel before attention reads every key through the block table.
        Seven launches per layer: QKV GEMM, fused attention step, o-proj GEMM (h +=), RMSNorm,
        gate/up GEMM with SwiGLU epilogue, down GEMM (h +=), RMSNorm."""
        m, c, pdl = self.m, self.c, self.pdl
        T = bs * E
        assert T <= self.T
        if self.fold:
            return self._forward_folded(ids, positions, cache_locs, rows, prefix_lens, bs, E, two_pass)
        if self.quant == "fp8":
            return self._forward_fp8(ids, positions, cache_locs, rows, prefix_lens, bs, E, two_pass)
        L0 = m.layers[0]
        K.add_rmsnorm(self.h, L0.ln1, self.xn, M=T, d=self.d, eps=c.rms_eps, ids=ids, embed=m.embed, pdl=pdl)
        n_layers = len(m.layers)
        scale = self.D ** -0.5
        for li, L in enumerate(m.layers):
            self._gemm(L.wqkv, self.xn, self.qkv, T, K.EPI_STORE_F32)
            self._attention(li, positions, cache_locs, rows, prefix_lens, bs, E, two_pass, scale)
            self._gemm(L.wo, self.attn, self.h, T, K.EPI_RESID_F32)
            K.add_rmsnorm(self.h, L.ln2, self.xn, M=T, d=self.d, eps=c.rms_eps, pdl=pdl)
            if self.fuse_swiglu:
                K.gemm_skinny(L.wgu, self.xn, self.act, M=T, splits=self._gu_splits(T), epi=K.EPI_SWIGLU_BF16,
                              ldo=self.act.stride(0),
                              status=self.status, pdl=pdl)
            else:
                self._gemm(L.wgu, self.xn, self.gu, T, K.EPI_STORE_F32)
                K.swiglu_partials(self.gu, 1, 0, self.act, M=T, ffn=self.ffn, blk=m.gu_block, pdl=pdl)
            self._gemm(L.wdown, self.act, self.h, T, K.EPI_RESID_F32)
            w_next = m.layers[li + 1].ln1 if li + 1 < n_layers else m.final_norm
            K.add_rmsnorm(self.h, w_next, self.xn, M=T, d=self.d, eps=c.rms_eps, pdl=pdl)
        return self.xn

    def _forward_fp8(self, ids, positions, cache_locs, rows, prefix_lens, bs: int, E: int, two_pass: bool):
        """W8A8 layer chain: every projection reads e4m3 weights (half the bytes of bf16) and per-token quantised
        activations through tcgen05.mma.kind::f8f6f4; norms, attention, residual stream and lm_head stay as in the bf16
        chain.  Nine launches per layer: two norms that also emit the e4m3 rows, two quantisation passes (attention
        output, SwiGLU output), four GEMMs, attention."""
        m, c, pdl = self.m, self.c, self.pdl
        T = bs * E
        st, ldx = self.status, self.x8.stride(0)
        K.add_rmsnorm_q8(self.h, m.layers[0].ln1, self.xn, self.x8, self.xs, M=T, d=self.d, eps=c.rms_eps, ids=ids,
                         embed=m.embed, pdl=pdl)
        n_layers = len(m.layers)
        scale = self.D ** -0.5
        nqd = self.nq * self.D

        def gemm(w, x, kdim, out, epi, splits, ldo):
            if x is not None:                       # x None: the norm kernel already left the e4m3 rows in x8
                K.quant_rows_e4m3(x, self.x8, self.xs, M=T, K=kdim, pdl=pdl)
            K.gemm_skinny_fp8(w[0], w[1], self.x8, self.xs, out, M=T, splits=splits, epi=epi, ldx=ldx, ldo=ldo,
                              status=st, pdl=pdl)
        for li, L in enumerate(m.layers):
            w8 = m._w8[li]
            gemm(w8["wqkv"], None, self.d, self.qkv, K.EPI_STORE_F32, self._splits(self.nqkv, self.d // 2, T),
                 self.qkv.stride(0))
            self._attention(li, positions, cache_locs, rows, prefix_lens, bs, E, two_pass, scale)
            gemm(w8["wo"], self.attn, nqd, self.h, K.EPI_RESID_F32, self._splits(self.d, nqd // 2, T), self.d)
            K.add_rmsnorm_q8(self.h, L.ln2, self.xn, self.x8, self.xs, M=T, d=self.d, eps=c.rms_eps, pdl=pdl)
            gemm(w8["wgu"], None, self.d, self.act, K.EPI_SWIGLU_BF16, self._gu_splits(T), self.act.stride(0))
            gemm(w8["wdown"], self.act, self.ffn, self.h, K.EPI_RESID_F32, self._splits(self.d, self.ffn // 2, T), self.d)
            w_next = m.layers[li + 1].ln1 if li + 1 < n_layers else m.final_norm
            K.add_rmsnorm_q8(self.h, w_next, self.xn, self.x8, self.xs, M=T, d=self.d, eps=c.rms_eps, pdl=pdl)
        return self.xn

    def _gu_splits(self, M: int) -> int:
        key = ("gu", M)
        s = self._splits_cache.get(key)
        if s is None:
            s = self._splits_cache[key] = K.gemm_swiglu_splits(2 * self.ffn, self.d, M)
        return s

    def lm_head_sample(self, rows: int, row_offset: int, row_step: int, *, temperature: float, alpha: float,
                       tokens_in, seed: int, cycle_counter, call_id: int, tok_out, logp_out, logz_out) -> None:
        """lm_head over the final hidden rows ``row_offset + i * row_step`` with sampling / scoring done in the GEMM
        epilogue: the [rows, V] logits never reach memory (what the reference does with an all-gathered logits
        tensor plus two sampling kernels: smcsd/core/worker.py:684-707, smcsd/core/kernels/fused_sampling.py:42-214)."""
        V = self.c.vocab_size
        if self._lm_parts is None or self._lm_parts.numel() < K.lm_parts_bytes(rows, V):
            self._lm_parts = torch.empty(K.lm_parts_bytes(max(rows, self.logits.shape[0]), V), dtype=torch.uint8,
                                         device=self.h.device)
        kw = {}
        if self.fold:
            X = self.hb[row_offset:]
            kw = dict(ssq_in=self.ssq[:, row_offset:], ssq_parts=self.n_parts, ssq_ld=self.ssq.stride(0), norm_d=self.d,
                      norm_eps=self.c.rms_eps, ssq_mstride=row_step)
        else:
            X = self.xn[row_offset:]
        K.lm_head_sample(self.m.lm_head, X, M=rows, V=V, ldx=self.d * row_step, status=self.status,
                         temperature=temperature, alpha=alpha, softcap=float(self.c.logit_softcap), tokens_in=tokens_in,
                         seed=seed, cycle_counter=cycle_counter, call_id=call_id, parts=self._lm_parts, tok_out=tok_out,
                         logp_out=logp_out, logz_out=logz_out, pdl=self.pdl, **kw)

    def lm_head(self, rows: int, row_offset: int = 0, row_step: int = 1) -> torch.Tensor:
        """fp32 logits [rows, V] of the final hidden rows ``row_offset + i * row_step``."""
        if self.fold:
            K.gemm_skinny_norm(self.m.lm_head, self.hb[row_offset:], self.logits, M=rows, splits=1,
                               epi=K.EPI_STORE_F32, ldx=self.d * row_step, ldo=self.logits.stride(0),
                               status=self.status, ssq_in=self.ssq[:, row_offset:], ssq_parts=self.n_parts,
                               norm_d=self.d, norm_eps=self.c.rms_eps, ssq_ld=self.ssq.stride(0),
                               ssq_mstride=row_step, pdl=self.pdl)
            return self.logits
        X = self.xn[row_offset:]
        K.gemm_skinny(self.m.lm_head, X, self.logits, M=rows, splits=1, epi=K.EPI_STORE_F32,
                      ldx=self.d * row_step, ldo=self.logits.stride(0), status=self.status, pdl=self.pdl)
        return self.logits


class NativeState:
    """Device-kernel versions of the SlotState transitions (bound to one SlotState)."""

    def __init__(self, max_bs: int, gamma: int, device, n_particles: int = 0):
        self.G = gamma + 1
        self.gamma = gamma
        self.device = device
        i32 = dict(dtype=torch.int32, device=device)
        G, g = self.G, gamma
        self.bufs = dict(
            orig_seq=torch.zeros(max_bs, **i32), x0=torch.zeros(max_bs, **i32), prev=torch.zeros(max_bs, **i32),
            cache_locs=torch.zeros(max_bs * G, **i32), positions_verify=torch.zeros(max_bs * G, **i32),
            step_pos=torch.zeros(G * max_bs, **i32), step_locs=torch.zeros(G * max_bs, **i32),
            head_ids=torch.zeros(max_bs * 2, **i32), head_pos=torch.zeros(max_bs * 2, **i32),
            head_locs=torch.zeros(max_bs * 2, **i32), head_prefix=torch.zeros(max_bs, **i32),
            verify_ids=torch.zeros(max_bs * G, **i32), verify_given=torch.zeros(max_bs * G, **i32))
        self.io = K.make_cycle_io(self.bufs)
        self.active = torch.zeros(max_bs, **i32)
        self.active_rows = torch.zeros(max_bs, **i32)
        self.drafts = torch.zeros(g * max_bs, **i32)                 # [gamma, bs] step-major
        self.logq = torch.zeros(g * max_bs, dtype=torch.float32, device=device)
        self.verify_tok = torch.zeros(max_bs * G, **i32)
        self.verify_logp = torch.zeros(max_bs * G, dtype=torch.float32, device=device)
        self.verify_logz = torch.zeros(max_bs * G, dtype=torch.float32, device=device)
        self.tokens_out = torch.zeros(max_bs * G, **i32)
        self.diff_out = torch.zeros(max_bs * g, dtype=torch.float32, device=device)
        self.job_dst = torch.zeros(max_bs, **i32)
        self.job_src = torch.zeros(max_bs, **i32)
        self._arrays = None
        self._version = -1
        self.bs = 0
        self.n_groups = 0
        self.fused_write_back = True
        # shared-prefix attention inputs, rewritten when the batch changes: keys every particle of a group shares
        # (its prompt minus one, so that the draft head's shorter prefix is covered as well), and for NP = 2, 4, 8 the
        # (and the group size) the block-table row and shared length of every NP-th sequence
        self.shared = torch.zeros(max_bs, **i32)
        sizes = {2, 4, 8} | ({int(n_particles)} if n_particles > 1 else set())
        self.rows_g = {n: torch.zeros(max(1, max_bs // n), **i32) for n in sizes}
        self.shared_g = {n: torch.zeros(max(1, max_bs // n), **i32) for n in sizes}

    def bind(self, st) -> None:
        self._arrays = K.make_slot_arrays(st)

    def sync_membership(self, st) -> None:
        """Refresh the persistent active-slot buffers after a group joined or left."""
        if st.version == self._version:
            return
        self._version = st.version
        self.bs = int(st.active_slots.numel())
        self.n_groups = len(st.active_rows_host)
        if self.bs:
            self.active[: self.bs].copy_(st.active_slots, non_blocking=True)
            self.active_rows[: self.n_groups].copy_(st.active_rows, non_blocking=True)
            bs = self.bs
            self.shared[:bs] = (st.prompt_lens[st.active_slots.long()] - 1).clamp_(min=0)
            for n in self.rows_g:
                if bs % n == 0:
                    self.rows_g[n][: bs // n] = self.active[:bs:n]
                    self.shared_g[n][: bs // n] = self.shared[:bs:n]

    # ---- SlotState hooks --------------------------------------------------------
    def prepare_cycle(self, st, slots) -> CycleInputs:
        if self._arrays is None:
            self.bind(st)
        self.sync_membership(st)
        bs, G = self.bs, self.G
        K.prepare_cycle(self._arrays, self.active, bs, G, st.counters, self.io)
        b = self.bufs
        return CycleInputs(slots=self.active[:bs], orig_seq_lens=b["orig_seq"][:bs], x0=b["x0"][:bs],
                           prev=b["prev"][:bs], cache_locs=b["cache_locs"][: bs * G].view(bs, G))

    def write_back(self, st, cin: CycleInputs, out: CycleOutputs) -> None:
        """Eager-path entry: the outputs come from a torch-computed cycle, so restage them."""
        if not self.fused_write_back:
            # SMC_FUSED_WRITE_BACK=0: the PyTorch reference of the same state transition
            native, st.native = st.native, None
            try:
                st.write_back(cin, out)
            finally:
                st.native = native
            return
        bs, g, G = self.bs, self.gamma, self.G
        self.drafts[: g * bs].view(g, bs).copy_(out.tokens[:, :g].t())
        self.verify_tok[: bs * G].view(bs, G)[:, g] = out.tokens[:, g]
        # store diff as alpha * logp - logq with logq = 0
        self.logq[: g * bs].zero_()
        self.verify_logp[: bs * G].view(bs, G)[:, :g] = out.logprob_diff.float()
        use_logz = out.bonus_logz is not None
        if use_logz:
            self.verify_logz[: bs * G].view(bs, G)[:, g] = out.bonus_logz.float()
        K.write_back(self._arrays, self.active, bs, g, self.drafts, self.logq, self.verify_tok, self.verify_logp,
                     self.verify_logz, 1.0, use_logz, self.tokens_out, self.diff_out)

    def write_back_native(self, st, alpha: float) -> None:
        K.write_back(self._arrays, self.active, self.bs, self.gamma, self.drafts, self.logq, self.verify_tok,
                     self.verify_logp, self.verify_logz, alpha, alpha != 1.0, self.tokens_out, self.diff_out)

    def collect_and_resample(self, st) -> None:
        if st.pp is not None:                     # particles of a group are spread over several GPUs
            st.pp.resample_native(st)
            return
        K.collect_resample(self._arrays, self.active_rows, self.n_groups, st.group_to_slots, st.N, float(st.threshold),
                           st.seed, st.counters, st.group_log_Z, self.job_dst, self.job_src)
        max_jobs = self.n_groups * (st.N - 1)
        for pool in st.state_pools:
            K.state_copy(pool.conv, pool.conv.shape[0], pool.n_rows, st.counters, self.job_dst, self.job_src, max_jobs)
            K.state_copy(pool.temporal, pool.temporal.shape[0], pool.n_rows, st.counters, self.job_dst, self.job_src,
                         max_jobs)


class NativeRunner:
    """Drives the kernel-chain forwards for one scheduler; owns the captured cycle graphs."""

    def __init__(self, sched, nstate: NativeState, comm=None):
        a = sched.args
        self.args = a
        self.ns = nstate
        self.comm = comm
        self.heap = None
        self.sched_models = (sched.target, sched.draft)
        self.device = sched.device
        self.gamma, self.G = a.gamma, a.gamma + 1
        self.max_bs = sched.max_groups * a.n_particles
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        pdl = _env_flag("SMC_PDL", True)
        self.pdl = pdl
        splits = int(a.attention_num_kv_splits)
        self.target = self._wrap(sched.target, sched.kv_t, sched.bt.table, self.max_bs * self.G, self.max_bs * self.G,
                                 splits, pdl, sched.state_t)
        self.draft = self._wrap(sched.draft, sched.kv_d, sched.bt.table, self.max_bs * 2, self.max_bs, splits, pdl,
                                sched.state_d)
        for nm in (self.target, self.draft):
            if type(nm) is NativeLlama:
                nm.cascade_bufs = {"shared": nstate.shared, "rows_g": nstate.rows_g, "shared_g": nstate.shared_g}
        self.nchunks = 32
        rows = self.max_bs * self.G
        self.sample_scratch = torch.empty(K.sample_scratch_bytes(rows, self.nchunks), dtype=torch.uint8,
                                          device=self.device)
        self.seed = int(a.random_seed) * 1000003 + 12345 + 7919 * getattr(sched, "pp_rank", 0)
        self.graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.use_graph = bool(a.cycle_graph)
        # capture caps (SMC_DRAFT_GRAPH_MAX_BS / SMC_DRAFT_GRAPH_MAX_CONTEXT): larger batches or contexts launch eagerly
        self.graph_max_bs = int(a.graph_max_bs)
        self.graph_max_context = int(a.graph_max_context)
        self.T_draft, self.T_target, self.alpha = float(a.draft_temperature), float(a.target_temperature), float(a.power_alpha)
        self.defer = bool(a.defer_bonus)
        # A/B switches (environment > argument > default on).  Switching a fused step off routes it to the PyTorch
        # implementation of the same step; such cycles launch eagerly, like the reference's downgrade of its graph
        # runners (smcsd/core/worker.py:296-327, smcsd/core/req_state.py:129-133).
        self.fused_sampling = bool(a.fused_sampling)
        self.fused_write_back = bool(a.fused_write_back)
        self.fast_verify = bool(a.fast_verify)
        self.draft_phase_graph = bool(a.draft_phase_graph)
        self.fused_lm_head = _env_flag("SMC_FUSED_LM_HEAD", True)     # sampling inside the lm_head epilogue (A/B knob)
        self.switched_off = not (self.fused_sampling and self.fused_write_back and self.fast_verify)
        if self.switched_off or _env_flag("SMC_DEFER_BONUS_EAGER", False):
            if self.use_graph:
                import logging
                logging.getLogger(__name__).warning(
                    "cycle graph disabled: a fused step is switched off (fused_sampling=%s fused_write_back=%s "
                    "fast_verify=%s) or SMC_DEFER_BONUS_EAGER is set", self.fused_sampling, self.fused_write_back,
                    self.fast_verify)
            self.use_graph = False
            self.draft_phase_graph = self.draft_phase_graph and not self.switched_off
        self._torch_gen = None
        self.draft_graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.launches_per_cycle = 0
        # Whole-forward persistent kernels (one launch per model forward, lm_head fused with sampling) for dense
        # unsharded models and batches of up to 128 token rows.  Opt-in (SMC_PERSISTENT=1): measured on B200 they cut
        # a decode cycle from 841 launches to 14 but are slower than the one-kernel-per-step chains (1B draft step
        # 1.30 ms against 0.86 ms, 8B verify 6.0 ms against 4.1 ms), whose GEMMs pick a cluster size per matrix.
        self.pf_target = self.pf_draft = None
        if _env_flag("SMC_PERSISTENT", False):
            from .native_forward import PersistentLlama, supported
            for name, nm in (("pf_target", self.target), ("pf_draft", self.draft)):
                if isinstance(nm, NativeLlama) and nm.fold and supported(nm.m, 1) and nm.kv.k.dtype != torch.uint8:
                    setattr(self, name, PersistentLlama(nm.m, nm.kv, nm.bt, 128, self.status))

    def _wrap(self, model, kv, bt, max_tokens, max_logit_rows, splits, pdl, state=None):
        if model.cfg.arch != "llama":
            from .native_hybrid import NativeHybrid
            return NativeHybrid(model, kv, bt, max_tokens, max_logit_rows, splits, self.status, pdl, runner=self,
                                state=state)
        if model.tp_size > 1:
            # tensor-parallel target: peers are reached through the symmetric heap, never through NCCL
            from ..parallel.symm import SymmHeap
            from .native_tp import NativeLlamaTP
            if self.comm is None:
                raise RuntimeError("a tensor-parallel model needs a process group (launch one rank per GPU)")
            if self.heap is None:
                # one heap for every tensor-parallel chain of this rank: decode and prompt-sized chains of the target
                # and, with replicate_draft=False, of the draft
                pf = self.PREFILL_MAX_TOKENS_TP
                cap = self.max_bs * self.G
                need = 8 << 20
                for mdl in self.sched_models:
                    if mdl.tp_size > 1 and mdl.cfg.arch == "llama":
                        need += 4 * (cap + pf) * mdl.cfg.hidden_size * 8 + (cap + pf) * 32 * 32 * mdl.tp_size + (1 << 20)
                self.heap = SymmHeap(need, self.device, self.comm.device_group, self.comm.group_rank,
                                     self.comm.group_size)
            model.tp_group = self.comm.device_group      # the PyTorch prefill path all-reduces through NCCL
            return NativeLlamaTP(model, kv, bt, max_tokens, max_logit_rows, splits, self.status, pdl, self.heap)
        return NativeLlama(model, kv, bt, max_tokens, max_logit_rows, splits, self.status, pdl)

    # ---- prefill ---------------------------------------------------------------------------------------
    PREFILL_BLOCK = 16
    PREFILL_MAX_TOKENS = 4096
    PREFILL_MAX_TOKENS_TP = 1024         # token capacity of the tensor-parallel prompt chain (symmetric-heap buffers)

    def _prefill_chain(self, which: str):
        """Kernel chains sized for prompt passes (built on first use; weights are shared with the decode chains)."""
        key = "_pf_" + which
        nm = getattr(self, key, None)
        if nm is None:
            base = self.target if which == "target" else self.draft
            if isinstance(base, NativeLlama):
                nm = NativeLlama(base.m, base.kv, base.bt, self.PREFILL_MAX_TOKENS, 8, base.attn_splits, self.status,
                                 self.pdl)
            elif type(base).__name__ == "NativeHybrid":
                nm = type(base)(base.m, base.kv, base.bt, self.PREFILL_MAX_TOKENS, 8, base.attn_splits, self.status,
                                self.pdl, runner=self, state=base.state)
            elif type(base).__name__ == "NativeLlamaTP" and self.heap is not None:
                # tensor-parallel prompts run through the same fused all-gather / reduce-scatter chain as decode
                nm = type(base)(base.m, base.kv, base.bt, self.PREFILL_MAX_TOKENS_TP, 256, 8, self.status, self.pdl,
                                self.heap)
            else:
                return None
            setattr(self, key, nm)
        nm.bt = (self.target if which == "target" else self.draft).bt
        return nm

    def prefill(self, worker, items) -> torch.Tensor:
        """Prompt pass through the kernel chains: every prompt is cut into 16-token blocks that run as rows of one
        batch (block j of a prompt attends to its 16j cached predecessors plus itself), so prefill reuses the
        decode kernels with token-tile GEMMs.  Gated-DeltaNet layers of hybrid models walk each prompt once, token
        by token, with the state held in registers.  Tensor-parallel targets and over-long batches take the plain
        PyTorch forward.  Dense prompts longer than the chains' token capacity run in several passes over
        consecutive blocks (earlier passes have already cached their keys)."""
        B = self.PREFILL_BLOCK
        lens = [len(it.input_ids) for it in items]
        n_blocks = [(L + B - 1) // B for L in lens]
        T = sum(n_blocks) * B
        tgt, drf = self._prefill_chain("target"), self._prefill_chain("draft")
        stateful = any(getattr(nm.m, "has_state", False) for nm in (tgt, drf) if nm is not None)
        if tgt is None or drf is None or (T > self.PREFILL_MAX_TOKENS and stateful) or len(items) > 256:
            native, worker.native = worker.native, None
            try:
                return worker.prefill(items)
            finally:
                worker.native = native
        dev = self.device
        ids_h = torch.zeros(T, dtype=torch.int32)
        pos_h = torch.zeros(T, dtype=torch.int32)
        valid_h = torch.zeros(T, dtype=torch.bool)
        rows_h, pref_h, last_rows = [], [], []
        t = 0
        for it, L, nb in zip(items, lens, n_blocks):
            ids_h[t:t + L] = torch.tensor(it.input_ids, dtype=torch.int32)
            pos_h[t:t + nb * B] = torch.arange(nb * B, dtype=torch.int32).clamp_(max=max(L - 1, 0))
            valid_h[t:t + L] = True
            rows_h += [it.row] * nb
            pref_h += [j * B for j in range(nb)]
            last_rows.append(t + L - 1)
            t += nb * B
        pin = lambda x: x.pin_memory().to(dev, non_blocking=True)
        ids, pos, valid = pin(ids_h), pin(pos_h), pin(valid_h)
        worker.io_bytes["h2d"] += ids_h.numel() * 9
        rows = pin(torch.tensor(rows_h, dtype=torch.int32))
        pref = pin(torch.tensor(pref_h, dtype=torch.int32))
        # page of every (padded) token: the prompt's pages, scratch page 0 for the padding -- one gather for the batch
        row_of = torch.zeros(T, dtype=torch.long)
        col_of = torch.zeros(T, dtype=torch.long)
        t = 0
        for it, L, nb in zip(items, lens, n_blocks):
            row_of[t:t + L] = it.row
            col_of[t:t + L] = torch.arange(L)
            t += nb * B
        locs = torch.where(valid, self.st.bt.table[pin(row_of), pin(col_of)], torch.zeros((), dtype=torch.int32, device=dev))
        worker.io_bytes["h2d"] += T * 16
        bs = sum(n_blocks)
        for nm in (tgt, drf):
            nm.set_context(max(lens), bs)

        def seqs_for(nm, short: int):
            # prompts as variable-length rows for the recurrent layers (None for dense models)
            if not getattr(nm.m, "has_state", False):
                return {}
            offs, t = [], 0
            for nb in n_blocks:
                offs.append(t)
                t += nb * B
            return {"seqs": {"rows": pin(torch.tensor([it.row for it in items], dtype=torch.int32)),
                             "off": pin(torch.tensor(offs, dtype=torch.int32)),
                             "len": pin(torch.tensor([max(L - short, 0) for L in lens], dtype=torch.int32)),
                             "n": len(items), "max": max(lens)}}
        cb = max(1, min(nm.T for nm in (tgt, drf)) // B)     # blocks per pass
        last = torch.tensor(last_rows, dtype=torch.long, device=dev)

        def grab(nm, idx):
            """Final-layer rows ``idx`` of the chain's buffers: raw bf16 residual rows + their sums of squares when the
            norm is folded into the lm_head, the normalised rows otherwise."""
            if hasattr(nm, "wait_final_rows"):          # tensor-parallel chain: peers' rows must have landed first
                nm.wait_final_rows()
                rows_n = nm.xn_a[idx]
                return {"x": rows_n, "ssq": None, "normed": rows_n}
            if getattr(nm, "fold", False):
                return {"x": nm.hb[idx], "ssq": nm.ssq[:, idx], "normed": nm.final_hidden(idx)}
            return {"x": nm.final_hidden(idx), "ssq": None, "normed": nm.final_hidden(idx)}

        def run(nm, short: int, want_hidden: bool):
            if bs <= cb:
                nm.forward(ids, pos, locs, rows, pref, bs, B, two_pass=True, **seqs_for(nm, short))
                parts = [grab(nm, last)] if want_hidden else []
            else:
                parts, order = [], []
                for c0 in range(0, bs, cb):
                    nb = min(cb, bs - c0)
                    tok = slice(c0 * B, (c0 + nb) * B)
                    nm.set_context(max(lens), nb)
                    nm.forward(ids[tok], pos[tok], locs[tok], rows[c0:c0 + nb], pref[c0:c0 + nb], nb, B, two_pass=True)
                    if want_hidden:
                        here = [(i, r - tok.start) for i, r in enumerate(last_rows) if tok.start <= r < tok.stop]
                        if here:
                            order += [i for i, _ in here]
                            parts.append(grab(nm, pin(torch.tensor([r for _, r in here], dtype=torch.long))))
                if want_hidden and order != sorted(order):
                    raise RuntimeError("prompt blocks are laid out in request order")
            if not want_hidden:
                return None
            fold = parts[0]["ssq"] is not None
            return {"n": len(items), "x": torch.cat([q["x"] for q in parts], 0),
                    "ssq": torch.cat([q["ssq"] for q in parts], 1) if fold else None,
                    "normed": lambda: torch.cat([q["normed"] for q in parts], 0)}
        x0 = self._sample_x0(tgt, run(tgt, 0, True), worker)
        # a stateful draft under the deferred schedule stops one token short: the first head forward of the decode
        # loop advances its recurrent state through the last prompt token exactly once
        run(drf, 1 if self.defer else 0, False)
        worker.io_bytes["d2h"] += 4 * len(items)
        return x0.to(torch.int32)

    def _sample_x0(self, nm, hidden, worker) -> torch.Tensor:
        """x0 of every prompt: a draw from softmax(alpha * logits / T_target) of the last prompt token.  Dense chains
        project and sample with the fused lm_head kernel (no logits in memory, noise keyed by the running count of
        prefilled prompts); other targets project with PyTorch (reference: smcsd/core/worker.py:668-707)."""
        n = hidden["n"]
        if hasattr(nm, "tp_sample") and n <= nm.logits.shape[0]:
            # vocabulary-parallel target: this rank's logits shard of the last prompt tokens, then the fused sampler
            # that exchanges per-chunk partials by peer stores (every rank draws the same x0)
            dev = self.device
            if getattr(self, "_x0_epoch", None) is None:
                self._x0_epoch = torch.zeros(1, dtype=torch.int64, device=dev)
                self._x0_counter_tp = torch.zeros(1, dtype=torch.int64, device=dev)
                self._x0_done_tp = 0
            self._x0_epoch.add_(1)
            self._x0_counter_tp.fill_(self._x0_done_tp)
            self._x0_done_tp += n
            X = hidden["x"].contiguous()
            K.gemm_skinny(nm.m.lm_head, X, nm.logits, M=n, splits=1, epi=K.EPI_STORE_F32, ldo=nm.logits.stride(0),
                          status=self.status)
            tok = torch.zeros(n, dtype=torch.int32, device=dev)
            lp = torch.zeros(n, dtype=torch.float32, device=dev)
            nm.tp_sample(rows=n, temperature=self.T_target, alpha=self.alpha, tokens_in=None, seed=self.seed ^ 0x5EED,
                         cycle_counter=self._x0_counter_tp, call_id=4096, tok_out=tok, logp_out=lp, logz_out=None,
                         epoch=self._x0_epoch)
            return tok
        if type(nm) is NativeLlama and self.fused_sampling and self.fused_lm_head and n <= 256:
            dev = self.device
            if getattr(self, "_x0_counter", None) is None:
                self._x0_counter = torch.zeros(1, dtype=torch.int64, device=dev)
                self._x0_done = 0
            self._x0_counter.fill_(self._x0_done)
            self._x0_done += n
            tok = torch.zeros(n, dtype=torch.int32, device=dev)
            lp = torch.zeros(n, dtype=torch.float32, device=dev)
            V = nm.c.vocab_size
            if nm._lm_parts is None or nm._lm_parts.numel() < K.lm_parts_bytes(n, V):
                nm._lm_parts = torch.empty(K.lm_parts_bytes(max(n, 8), V), dtype=torch.uint8, device=dev)
            kw = {}
            if hidden["ssq"] is not None:
                ssq = hidden["ssq"].contiguous()
                kw = dict(ssq_in=ssq, ssq_parts=ssq.shape[0], ssq_ld=ssq.stride(0), norm_d=nm.d, norm_eps=nm.c.rms_eps)
            X = hidden["x"].contiguous()
            K.lm_head_sample(nm.m.lm_head, X, M=n, V=V, ldx=X.stride(0), status=self.status, temperature=self.T_target,
                             alpha=self.alpha, softcap=float(nm.c.logit_softcap), tokens_in=None,
                             seed=self.seed ^ 0x5EED, cycle_counter=self._x0_counter, call_id=4096, parts=nm._lm_parts,
                             tok_out=tok, logp_out=lp, logz_out=None, **kw)
            return tok
        from ..smc import math as smc_math
        logits = self.target.m.logits_torch(hidden["normed"]())
        x0, _, _ = smc_math.gumbel_sample(logits, self.T_target, self.alpha, generator=worker.gen_prefill)
        return x0

    # ---- the cycle, as a sequence of kernel launches ---------------------------------
    def _sample_torch(self, nm, rows: int, temperature: float, alpha: float, tokens_in, tok_out, logp_out,
                      logz_out) -> None:
        """PyTorch Gumbel-max / scoring chain over the logits in memory (the path SMC_FUSED_SAMPLING=0 selects;
        same math as smcsd/core/worker.py:721-778)."""
        V = nm.c.vocab_size
        x = nm.logits[:rows, :V].float()
        cap = float(nm.c.logit_softcap)
        if cap > 0:
            x = torch.tanh(x / cap) * cap
        base = x / temperature
        scaled = base * alpha
        lse_s = torch.logsumexp(scaled, dim=-1)
        lse_b = torch.logsumexp(base, dim=-1) if alpha != 1.0 else lse_s
        if self._torch_gen is None:
            self._torch_gen = torch.Generator(device=self.device)
            self._torch_gen.manual_seed(self.seed & 0x7FFFFFFF)
        u = torch.rand(scaled.shape, generator=self._torch_gen, device=self.device).clamp_(1e-10, 1.0 - 1e-7)
        tok = torch.argmax(scaled - torch.log(-torch.log(u)), dim=-1)
        logp = scaled.gather(1, tok[:, None])[:, 0] - lse_s
        logz = lse_s - alpha * lse_b if alpha != 1.0 else torch.zeros_like(lse_s)
        if tokens_in is not None:
            given = tokens_in[:rows].long()
            score = given >= 0
            g = given.clamp(min=0)
            tok = torch.where(score, g, tok)
            logp = torch.where(score, base.gather(1, g[:, None])[:, 0] - lse_b, logp)
            logz = torch.where(score, torch.zeros_like(logz), logz)
        tok_out[:rows].copy_(tok.to(torch.int32))
        logp_out[:rows].copy_(logp)
        if logz_out is not None:
            logz_out[:rows].copy_(logz)

    def _sample(self, nm, rows: int, call_id: int, temperature: float, alpha: float, tokens_in, tok_out, logp_out,
                logz_out) -> None:
        if not self.fused_sampling and not hasattr(nm, "tp_sample"):
            self._sample_torch(nm, rows, temperature, alpha, tokens_in, tok_out, logp_out, logz_out)
            return
        if hasattr(nm, "tp_sample"):
            nm.tp_sample(rows=rows, temperature=temperature, alpha=alpha, tokens_in=tokens_in, seed=self.seed,
                         cycle_counter=self._counters, call_id=call_id, tok_out=tok_out, logp_out=logp_out,
                         logz_out=logz_out)
            return
        K.sample_or_score(nm.logits, rows=rows, V=nm.c.vocab_size if nm.m.tp_size == 1 else nm.V, splits=1,
                          split_stride=0, row_stride=nm.logits.stride(0), temperature=temperature, alpha=alpha,
                          softcap=float(nm.c.logit_softcap), tokens_in=tokens_in, seed=self.seed,
                          cycle_counter=self._counters, call_id=call_id, scratch=self.sample_scratch,
                          nchunks=self.nchunks, tok_out=tok_out, logp_out=logp_out, logz_out=logz_out, pdl=self.pdl)

    def _use_pf(self, which: str, tokens: int) -> bool:
        pf = self.pf_target if which == "target" else self.pf_draft
        return pf is not None and tokens <= pf.T and not self.switched_off

    def _verify_torch(self, nm, ids, pos, locs, rows, prefix, bs: int, E: int) -> None:
        """Target verify through the plain PyTorch forward (cuBLAS GEMMs, reference attention loop): what
        SMC_FAST_VERIFY=0 selects.  Fills the chain's logits buffer."""
        T = bs * E
        pl = prefix[:bs].tolist()
        ext = ExtendBatch(ids[:T].long(), pos[:T].long(), locs[:T], rows[:bs], prefix[:bs], extend_len=E,
                          prefix_lens_host=pl)
        hid = nm.m.forward_torch(ext, nm.kv, nm.bt)
        nm.logits[:T, :nm.c.vocab_size].copy_(nm.m.logits_torch(hid))

    def _model_step(self, which: str, ids, pos, locs, rows, prefix, bs: int, E: int, *, lm_rows: int, lm_off: int = 0,
                    lm_step: int = 1, call_id: int = 0, temperature: float = 1.0, alpha: float = 1.0, tokens_in=None,
                    tok_out=None, logp_out=None, logz_out=None) -> None:
        """One model forward for bs sequences of E new tokens, followed (when lm_rows > 0) by the lm_head over rows
        lm_off + i * lm_step and the fused sampler / scorer: one persistent launch, or the kernel chain."""
        if self._use_pf(which, bs * E):
            pf = self.pf_target if which == "target" else self.pf_draft
            pf.run(ids, pos, locs, rows, prefix, bs, E, lm_rows=lm_rows, lm_off=lm_off, lm_step=lm_step,
                   temperature=temperature, alpha=alpha, tokens_in=tokens_in, seed=self.seed,
                   cycle_counter=self._counters, call_id=call_id, tok_out=tok_out, logp_out=logp_out,
                   logz_out=logz_out)
            return
        nm = self.target if which == "target" else self.draft
        if which == "target" and not self.fast_verify and isinstance(nm, NativeLlama):
            self._verify_torch(nm, ids, pos, locs, rows, prefix, bs, E)
        else:
            nm.forward(ids, pos, locs, rows, prefix, bs, E)
            if lm_rows > 0 and self.fused_sampling and self.fused_lm_head and type(nm) is NativeLlama and lm_rows <= 256:
                # sampling / scoring inside the lm_head epilogue: no logits in memory, one merge launch
                nm.lm_head_sample(lm_rows, lm_off, lm_step, temperature=temperature, alpha=alpha, tokens_in=tokens_in,
                                  seed=self.seed, cycle_counter=self._counters, call_id=call_id, tok_out=tok_out,
                                  logp_out=logp_out, logz_out=logz_out)
                return
            if lm_rows > 0:
                nm.lm_head(lm_rows, row_offset=lm_off, row_step=lm_step)
        if lm_rows > 0:
            self._sample(nm, lm_rows, call_id, temperature, alpha, tokens_in, tok_out, logp_out, logz_out)

    def _cycle_body(self, st) -> None:
        self._draft_body(st)
        self._verify_body(st)

    def _draft_body(self, st) -> None:
        ns, b = self.ns, self.ns.bufs
        bs, g, G = ns.bs, self.gamma, self.G
        self._counters = st.counters
        rows = ns.active[:bs]
        dr, lq = ns.drafts, ns.logq
        Td = self.T_draft
        if self.defer:
            self._model_step("draft", b["head_ids"], b["head_pos"], b["head_locs"], rows, b["head_prefix"], bs, 2,
                             lm_rows=bs, lm_off=1, lm_step=2, call_id=0, temperature=Td, tok_out=dr[:bs],
                             logp_out=lq[:bs])
            for s in range(1, g):
                sl = slice(s * bs, (s + 1) * bs)
                self._model_step("draft", dr[(s - 1) * bs: s * bs], b["step_pos"][sl], b["step_locs"][sl], rows,
                                 b["step_pos"][sl], bs, 1, lm_rows=bs, call_id=s, temperature=Td, tok_out=dr[sl],
                                 logp_out=lq[sl])
        else:
            for s in range(g + 1):
                sl = slice(s * bs, (s + 1) * bs)
                ids = b["x0"] if s == 0 else dr[(s - 1) * bs: s * bs]
                self._model_step("draft", ids, b["step_pos"][sl], b["step_locs"][sl], rows, b["step_pos"][sl], bs, 1,
                                 lm_rows=bs if s < g else 0, call_id=s, temperature=Td,
                                 tok_out=dr[sl] if s < g else None, logp_out=lq[sl] if s < g else None)

    def _verify_body(self, st) -> None:
        ns, b = self.ns, self.ns.bufs
        bs, g, G = ns.bs, self.gamma, self.G
        self._counters = st.counters
        rows = ns.active[:bs]
        dr = ns.drafts
        K.assemble_verify(ns.io, dr, bs, g)
        self._model_step("target", b["verify_ids"], b["positions_verify"], b["cache_locs"], rows, b["orig_seq"], bs, G,
                         lm_rows=bs * G, call_id=g + 1, temperature=self.T_target, alpha=self.alpha,
                         tokens_in=b["verify_given"], tok_out=ns.verify_tok, logp_out=ns.verify_logp,
                         logz_out=ns.verify_logz)

    def decode_cycle(self, worker, cin: CycleInputs) -> CycleOutputs:
        """Eager kernel chain for one cycle (the graph path replays the same launches)."""
        st = self.st
        ns = self.ns
        # this entry is driven step by step from the host, so one small read for the attention split plan is fine
        ctx = int(cin.orig_seq_lens.max().item()) + self.G if cin.orig_seq_lens.numel() else 0
        self.target.set_context(ctx, ns.bs, (self.G,))
        self.draft.set_context(ctx, ns.bs, (1, 2))
        self._plan_prefix(st, ns.bs, None)          # the step-by-step path keeps the single-launch attention
        if self.draft_phase_graph and not self.switched_off and ns.bs <= self.graph_max_bs:
            # draft-only graph (SMC_DRAFT_PHASE_GRAPH): the gamma draft forwards and their sampling replay as one
            # launch, verify and scoring stay eager.  The draft part only reads the buffers the prologue kernel filled
            # and its noise is keyed by the cycle counter, so running it once eagerly before the capture is harmless.
            key = (ns.bs, self.draft.set_context(self.target.ctx_hint, ns.bs, (1, 2)))
            gr = self.draft_graphs.get(key)
            if gr is None:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self._draft_body(st)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    self._draft_body(st)
                self.draft_graphs[key] = gr
            gr.replay()
            self._verify_body(st)
        else:
            self._cycle_body(st)
        bs, g, G = ns.bs, self.gamma, self.G
        drafts = ns.drafts[: g * bs].view(g, bs).t()
        tokens = torch.cat([drafts, ns.verify_tok[: bs * G].view(bs, G)[:, g:]], dim=1)
        diff = self.alpha * ns.verify_logp[: bs * G].view(bs, G)[:, :g] - ns.logq[: g * bs].view(g, bs).t()
        logz = ns.verify_logz[: bs * G].view(bs, G)[:, g] if self.alpha != 1.0 else None
        return CycleOutputs(tokens=tokens, logprob_diff=diff, bonus_logz=logz)

    # ---- whole-cycle graph ----------------------------------------------------------
    def can_run_cycle(self, st) -> bool:
        """The whole cycle as one kernel sequence (graph, or the same launches eagerly beyond the capture caps).
        With a fused step switched off, or the draft-only graph asked for, the scheduler drives the cycle step by
        step instead: prologue kernel, ``decode_cycle``, write-back, resampling."""
        return not self.switched_off and not (self.draft_phase_graph and not self.use_graph)

    def _full_cycle(self, st) -> None:
        ns = self.ns
        K.prepare_cycle(ns._arrays, ns.active, ns.bs, self.G, st.counters, ns.io)
        self._cycle_body(st)
        ns.write_back_native(st, self.alpha)
        ns.collect_and_resample(st)

    def _plan_prefix(self, st, bs: int, prompt_hint) -> tuple:
        """Shared-prefix attention plans of both models for this cycle (part of the graph key)."""
        lo, hi = prompt_hint if prompt_hint else (0, 0)
        key = ()
        for nm, Es in ((self.target, (self.G,)), (self.draft, (1, 2))):
            if type(nm) is NativeLlama:
                key += (nm.set_prefix(int(lo), int(hi), bs, st.N, Es),)
        return key

    def run_cycle(self, st, worker, ctx_hint: int = 0, prompt_hint=None) -> None:
        """One decode cycle.  ``ctx_hint``: upper bound of the sequence lengths this cycle reaches (known on the host
        from prompt lengths and cycle counts); it selects how many key ranges the attention steps split into, and
        with it which captured graph runs.  ``prompt_hint``: (shortest, longest) prompt among the running groups; long
        shared prompts switch the attention steps to their shared-prefix passes."""
        ns = self.ns
        if ns._arrays is None:
            ns.bind(st)
        ns.sync_membership(st)
        st.step += 1
        bs = ns.bs
        key = (bs, self.target.set_context(ctx_hint, bs, (self.G,)), self.draft.set_context(ctx_hint, bs, (1, 2)))
        if self._use_pf("target", bs * self.G):
            key += (self.pf_target.set_context(ctx_hint, bs, (self.G,)),)
        if self._use_pf("draft", bs * 2):
            key += (self.pf_draft.set_context(ctx_hint, bs, (1, 2)),)
        key += self._plan_prefix(st, bs, prompt_hint)
        if not self.use_graph or bs > self.graph_max_bs or ctx_hint > self.graph_max_context:
            self._full_cycle(st)           # same kernels, launched one by one (beyond the capture caps)
            return
        gr = self.graphs.get(key)
        if gr is None:
            # warm up once eagerly on a side stream (also JIT-free: everything is precompiled), then capture
            gr = torch.cuda.CUDAGraph()
            saved = self._save_state(st)
            self._align_ranks(st)          # every rank enters the eager cycle's cross-rank waits together
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            # The eager cycle only has to launch every kernel once before the capture; its effects are rolled back by
            # putting the metadata back.  That is exact for ancestor copies on one GPU (they copy page ids), but a
            # cross-GPU adoption refills the destination's released pages with the ancestor's KV rows.  So with
            # particle-parallel groups the eager cycle runs with resampling off on every rank (the exchange, plan and
            # fetch kernels still launch and find nothing to do).
            threshold = st.threshold
            if st.pp is not None:
                st.threshold = 0.0
            try:
                with torch.cuda.stream(s):
                    self._full_cycle(st)
            finally:
                st.threshold = threshold
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            self._restore_state(st, saved)
            n0 = K.launch_count
            with torch.cuda.graph(gr):
                self._full_cycle(st)
            self.launches_per_cycle = K.launch_count - n0
            self._restore_state(st, saved)
            self.graphs[key] = gr
            self._align_ranks(st)          # capture time differs per rank; replay starts together
        gr.replay()

    def _align_ranks(self, st) -> None:
        """Host rendezvous of the ranks that share requests (particle- or tensor-parallel) around a graph capture: the
        in-kernel waits on peers are bounded at about a second, and eager launching and capturing take the ranks
        different amounts of host time."""
        if st.pp is not None:
            st.pp.align()
        elif self.comm is not None and getattr(self.comm, "group_size", 1) > 1:
            torch.cuda.synchronize()
            self.comm.barrier()

    # capture runs the cycle for real; put the mutable state back afterwards
    def _mutable(self, st) -> List[torch.Tensor]:
        al = st.alloc
        ts = [st.seq_lens, st.verified_ids, st.prev_ids, st.token_counts, st.finished, st.finished_len, st.finish_code,
              st.matched_eos, st.log_weights, st.interval_weights, st.group_log_Z, st.counters, al.refcount,
              al.free_stack, al.free_count, al.error_flag, st.bt.table, st.all_token_ids]
        if getattr(st, "group_active", None) is not None:
            ts.append(st.group_active)
        for pool in st.state_pools:
            ts += [pool.conv, pool.temporal]
        return ts

    def _save_state(self, st):
        return [t.clone() for t in self._mutable(st)]

    def _restore_state(self, st, saved) -> None:
        step = st.counters[0:1].clone()
        for t, s in zip(self._mutable(st), saved):
            t.copy_(s)
        if st.pp is not None:
            # cross-rank counters advanced during the warm-up cycle; keep the cycle number in step with them
            st.counters[0:1].copy_(step)

    def check_status(self) -> int:
        self._status_host.copy_(self.status)
        return int(self._status_host[0])


def create(sched, comm=None):
    """Build the device-state and runner objects for a scheduler."""
    if not torch.cuda.is_available():
        raise RuntimeError("the native backend needs a CUDA device")
    K.lib()     # fail loudly if the kernel library is missing
    ns = NativeState(sched.max_groups * sched.args.n_particles, sched.args.gamma, sched.device, sched.args.n_particles)
    ns.fused_write_back = bool(sched.args.fused_write_back)
    runner = NativeRunner(sched, ns, comm)
    return ns, runner
