"""Kernel-chain forward of the hybrid Gated-DeltaNet model on sm_100a.

Attention layers reuse the fused attention step (per-head q/k RMSNorm, partial rotary, sigmoid
output gate all inside that kernel); Gated-DeltaNet layers run in-projection GEMM -> conv + SiLU ->
recurrent delta-rule step with gated RMSNorm -> out-projection GEMM accumulating into the residual
stream; prompt passes replace the token-by-token delta rule by the chunk-parallel tcgen05 kernel.  The recurrent state lives in the state pool and follows particles through resampling by
the same (dst, src) job list as the KV block table.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from . import native as K


class NativeHybrid:
    def __init__(self, model, kv, block_table, max_tokens, max_logit_rows, attn_splits, status, pdl, runner=None,
                 state=None):
        self.m, self.kv, self.bt = model, kv, block_table
        c = model.cfg
        self.c = c
        dev = model.device
        self.T, self.status, self.pdl = max_tokens, status, pdl
        self.state = state
        self.nq, self.nkv, self.D = c.n_heads, c.n_kv_heads, c.head_dim
        self.d, self.ffn = c.hidden_size, c.ffn_size
        self.V = model.lm_head.shape[0]
        f32, bf16 = torch.float32, torch.bfloat16
        gate = 2 if c.attn_output_gate else 1
        self.nqkv = (self.nq * gate + 2 * self.nkv) * self.D
        self.win_rows = max((L.win.shape[0] for L in model.layers if L.win is not None), default=8)
        self.h = torch.empty(max_tokens, self.d, dtype=f32, device=dev)
        self.xn = torch.empty(max_tokens, self.d, dtype=bf16, device=dev)
        self.attn = torch.zeros(max_tokens, max(self.nq * self.D, model.value_dim), dtype=bf16, device=dev)
        self.act = torch.empty(max_tokens, self.ffn, dtype=bf16, device=dev)
        self.qkv = torch.empty(max_tokens, max(self.nqkv, self.win_rows), dtype=f32, device=dev)
        self.conv_out = torch.empty(max_tokens, model.conv_dim, dtype=f32, device=dev)
        self.attn_splits = attn_splits
        self._q = None                      # rotated queries of a prompt pass (allocated on first use)
        self.ctx_hint = 0                    # context-length bound that sizes the attention key splits, see set_context
        self.part_acc = self.part_ml = torch.empty(1, dtype=f32, device=dev)     # unused by the fused kernel
        self.logits = torch.empty(max_logit_rows, self.V, dtype=f32, device=dev)
        self.fuse_swiglu = model.gu_block == 64 and (2 * self.ffn) % 128 == 0
        if not self.fuse_swiglu:
            self.gu = torch.empty(max_tokens, 2 * self.ffn, dtype=f32, device=dev)
        self._splits_cache: Dict = {}
        # prompt passes of at least 64 tokens per row run the delta rule chunk-parallel on tcgen05 (SMC_GDN_CHUNKED=0:
        # token by token, as the decode steps do)
        self.gdn_chunked = os.environ.get("SMC_GDN_CHUNKED", "1") != "0"

    def _gemm(self, W, X, out, M, epi, ldo=None):
        N, Kd = W.shape
        key = (N, Kd, M)
        if key not in self._splits_cache:
            self._splits_cache[key] = K.gemm_cluster_splits(N, Kd, M)
        K.gemm_skinny(W, X, out, M=M, splits=self._splits_cache[key], epi=epi, ldo=ldo or out.stride(0),
                      status=self.status, pdl=self.pdl)

    def forward(self, ids, positions, cache_locs, rows, prefix_lens, bs: int, E: int, two_pass: bool = False,
                seqs=None):
        """``two_pass`` + ``seqs`` (prompt passes): the batch rows are consecutive E-token blocks of whole prompts.
        Attention layers first write every new K/V row to the cache, then each block attends through the block
        table; Gated-DeltaNet layers walk each prompt once from its first to its last real token
        (``seqs`` = state rows, token offsets and token counts of the prompts, int32 tensors)."""
        m, c, pdl = self.m, self.c, self.pdl
        T = bs * E
        assert T <= self.T and self.state is not None
        if two_pass and self._q is None:
            self._q = torch.empty(self.T, self.nq * self.D, dtype=torch.bfloat16, device=m.device)
        po = c.norm_plus_one
        K.add_rmsnorm(self.h, m.layers[0].ln1, self.xn, M=T, d=self.d, eps=c.rms_eps, ids=ids, embed=m.embed,
                      plus_one=po, pdl=pdl)
        nL = len(m.layers)
        scale = self.D ** -0.5
        nq = self.nq * self.D
        for li, L in enumerate(m.layers):
            if L.kind == "full_attention":
                ki = m.kv_index[li]
                qkv = self.qkv[:, :self.nqkv]
                self._gemm(L.wqkv, self.xn, self.qkv, T, K.EPI_STORE_F32)
                gate_off = nq if c.attn_output_gate else -1
                k_off = 2 * nq if c.attn_output_gate else nq
                q_in = None
                if two_pass:
                    K.rope_kv_write_heads(self.qkv, positions, cache_locs, m.rope, self._q, self.kv.k[ki],
                                          self.kv.v[ki], M=T, Hq=self.nq, Hkv=self.nkv, D=self.D, status=self.status,
                                          q_off=0, k_off=k_off, v_off=k_off + self.nkv * self.D, qn_w=L.q_norm,
                                          kn_w=L.k_norm, norm_eps=c.rms_eps, norm_plus_one=po, pdl=pdl)
                    q_in = self._q
                K.attention_fused(self.qkv, positions, cache_locs, m.rope, self.kv.k[ki], self.kv.v[ki], self.bt, rows,
                                  prefix_lens, self.attn, self.part_acc, self.part_ml, bs=bs, E=E, Hq=self.nq,
                                  Hkv=self.nkv, D=self.D, KS=self._ks(bs, E), scale=scale, status=self.status, q_off=0,
                                  gate_off=gate_off, k_off=k_off, v_off=k_off + self.nkv * self.D, qn_w=L.q_norm,
                                  kn_w=L.k_norm, norm_eps=c.rms_eps, norm_plus_one=po, pdl=pdl, q_in=q_in)
                # the attention output rows are packed [T, Hq*D] at the start of the shared buffer
                self._gemm(L.wo, self.attn.view(-1)[: T * nq].view(T, nq), self.h, T, K.EPI_RESID_F32)
            else:
                si = m.state_index[li]
                self._gemm(L.win, self.xn, self.qkv, T, K.EPI_STORE_F32)
                vd = m.value_dim
                mix = self.attn.view(-1)[: T * vd].view(T, vd)
                if seqs is not None:
                    K.gdn_step(self.qkv, self.state.conv[si], self.state.temporal[si], seqs["rows"], L.conv_w,
                               L.dt_bias, L.A_log, L.gnorm_w, self.conv_out, mix, bs=seqs["n"], E=0,
                               Hk=c.gdn_n_k_heads, Hv=c.gdn_n_v_heads, dk=c.gdn_head_k_dim, dv=c.gdn_head_v_dim,
                               W=c.gdn_conv_width, eps=c.rms_eps, pdl=pdl, tok_off=seqs["off"], tok_len=seqs["len"],
                               chunked=self.gdn_chunked and T >= K.GDN_CHUNK_MIN_TOKENS * seqs["n"], status=self.status,
                               max_len=seqs.get("max", 0))
                else:
                    K.gdn_step(self.qkv, self.state.conv[si], self.state.temporal[si], rows, L.conv_w, L.dt_bias,
                               L.A_log, L.gnorm_w, self.conv_out, mix, bs=bs, E=E, Hk=c.gdn_n_k_heads,
                               Hv=c.gdn_n_v_heads, dk=c.gdn_head_k_dim, dv=c.gdn_head_v_dim, W=c.gdn_conv_width,
                               eps=c.rms_eps, pdl=pdl)
                self._gemm(L.wout, mix, self.h, T, K.EPI_RESID_F32)
            K.add_rmsnorm(self.h, L.ln2, self.xn, M=T, d=self.d, eps=c.rms_eps, plus_one=po, pdl=pdl)
            if self.fuse_swiglu:
                K.gemm_skinny(L.wgu, self.xn, self.act, M=T, splits=self._gu_splits(T), epi=K.EPI_SWIGLU_BF16,
                              ldo=self.act.stride(0),
                              status=self.status, pdl=pdl)
            else:
                self._gemm(L.wgu, self.xn, self.gu, T, K.EPI_STORE_F32)
                K.swiglu_partials(self.gu, 1, 0, self.act, M=T, ffn=self.ffn, blk=m.gu_block, pdl=pdl)
            self._gemm(L.wdown, self.act, self.h, T, K.EPI_RESID_F32)
            w_next = m.layers[li + 1].ln1 if li + 1 < nL else m.final_norm
            K.add_rmsnorm(self.h, w_next, self.xn, M=T, d=self.d, eps=c.rms_eps, plus_one=po, pdl=pdl)
        return self.xn

    def final_hidden(self, token_rows: torch.Tensor) -> torch.Tensor:
        """Final-norm activations of selected token rows of the last forward."""
        return self.xn[token_rows]

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
        K.gemm_skinny(self.m.lm_head, self.xn[row_offset:], self.logits, M=rows, splits=1, epi=K.EPI_STORE_F32,
                      ldx=self.d * row_step, ldo=self.logits.stride(0), status=self.status, pdl=self.pdl)
        return self.logits
