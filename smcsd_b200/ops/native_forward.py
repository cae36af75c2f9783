"""Whole-forward persistent kernel for dense Llama-style models (``csrc/forward_persistent.cu``).

One launch runs embedding, every decoder layer (QKV GEMM, attention over the paged KV cache, o-proj, gate/up with
SwiGLU, down) and the lm_head fused with Gumbel sampling / token scoring, for batches of up to 128 token rows.
The weight stream runs ahead of the activations across phase boundaries and a decode cycle shrinks from several
hundred dependent launches to about a dozen.  Measured on B200 the per-phase cost (grid barrier, activation fetch,
K-split reduction inside clusters of eight) is still higher than that of the stand-alone GEMM kernels, which choose a
cluster size per matrix, so the runner uses this path only when ``SMC_PERSISTENT=1`` is set.

The reference runs each of these steps as separate library / Triton launches inside a CUDA graph
(smcsd/model_executor/smc_draft_phase_graph_runner.py:1043-1082 for the draft loop, :666-719 for verify + scoring).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional, Tuple

import torch

from . import native as K


class PfParams(C.Structure):
    _fields_ = (
        [(n, C.c_int) for n in ("L", "d", "Hq", "Hkv", "D", "ffn", "V", "nqkv", "rd", "max_pos", "n_pages",
                                "bt_stride")]
        + [(n, C.c_float) for n in ("rms_eps", "softcap", "scale", "pad0")]
        + [(n, C.c_void_p) for n in ("maps", "embed", "rope", "k_pool", "v_pool")]
        + [("kv_layer_stride", C.c_longlong), ("block_table", C.c_void_p)]
        + [(n, C.c_int) for n in ("bs", "E", "M", "BN", "KS", "lm_rows", "n_mt", "n_kw", "att_stg", "stages",
                                  "ring_bytes", "att_bytes", "lm_row_off", "lm_row_step")]
        + [(n, C.c_void_p) for n in ("ids", "positions", "cache_locs", "rows", "prefix_lens", "h", "hb", "ssq", "qkv",
                                     "attn", "act")]
        + [("ssq_ld", C.c_int), ("pad1", C.c_int)]
        + [(n, C.c_void_p) for n in ("att_part", "att_ctr")]
        + [("inv_temp", C.c_float), ("alpha", C.c_float), ("tokens_in", C.c_void_p), ("seed", C.c_ulonglong),
           ("cycle_counter", C.c_void_p), ("call_id", C.c_int), ("pad2", C.c_int)]
        + [(n, C.c_void_p) for n in ("sparts", "tok_out", "logp_out", "logz_out", "sync", "status", "trace")]
    )


_declared = False


def _lib():
    global _declared
    L = K.lib()
    if not _declared:
        vp, i, ll = C.c_void_p, C.c_int, C.c_longlong
        L.smc_pf_params_size.restype = C.c_int
        L.smc_pf_num_ctas.argtypes = [i]
        L.smc_pf_num_ctas.restype = C.c_int
        L.smc_pf_encode_map.argtypes = [vp, vp, ll, ll, ll, i]
        L.smc_pf_encode_map.restype = C.c_int
        L.smc_pf_plan.argtypes = [i, i, i, i] + [C.POINTER(C.c_int)] * 6
        L.smc_pf_plan.restype = C.c_int
        L.smc_pf_forward.argtypes = [vp, i, vp]
        L.smc_pf_forward.restype = C.c_int
        assert C.sizeof(PfParams) == L.smc_pf_params_size(), "PfParams layout mismatch"
        _declared = True
    return L


def supported(model, max_tokens: int) -> bool:
    """Dense, unsharded Llama-style model with a head size and batch the persistent kernel is built for."""
    c = model.cfg
    return (c.arch == "llama" and model.tp_size == 1 and c.head_dim in (64, 128) and c.hidden_size % 128 == 0
            and model.gu_block == 64 and (2 * model.ffn) % 128 == 0 and max_tokens <= 128
            and c.rotary_dim % 8 == 0 and (c.head_dim - c.rotary_dim) % 4 == 0
            and (model.n_heads // model.n_kv_heads) * 1 <= 96)


class PersistentLlama:
    """Buffers, tensor-map tables and launch plans of the persistent forward for one model."""

    def __init__(self, model, kv, block_table: torch.Tensor, max_tokens: int, status: torch.Tensor):
        L = _lib()
        model.fold_norms()
        self.m, self.kv, self.bt = model, kv, block_table
        c = model.cfg
        self.c = c
        dev = model.device
        self.dev = dev
        self.status = status
        self.T = int(max_tokens)
        self.nq, self.nkv, self.D = model.n_heads, model.n_kv_heads, c.head_dim
        self.d, self.ffn = c.hidden_size, model.ffn
        self.nqkv = (self.nq + 2 * self.nkv) * self.D
        self.V = model.lm_head.shape[0]
        self.nl = len(model.layers)
        self.ncta = L.smc_pf_num_ctas(self.D)
        if self.ncta <= 0:
            raise K.NativeError(f"cannot size the persistent grid (code {self.ncta})")
        f32, bf16, i32 = torch.float32, torch.bfloat16, torch.int32
        T = self.T
        self.h = torch.zeros(T, self.d, dtype=f32, device=dev)
        self.hb = torch.zeros(T, self.d, dtype=bf16, device=dev)
        self.ssq_ld = T
        self.ssq = torch.zeros(self.d // 128, T, dtype=f32, device=dev)
        self.qkv = torch.zeros(T, self.nqkv, dtype=f32, device=dev)
        self.attn = torch.zeros(T, self.nq * self.D, dtype=bf16, device=dev)
        self.act = torch.zeros(T, self.ffn, dtype=bf16, device=dev)
        self.att_ctr = torch.zeros(max(1, T * self.nkv), dtype=i32, device=dev)
        self.att_part = torch.zeros(1, dtype=f32, device=dev)
        self.sparts = torch.zeros(128 * self.ncta * 8, dtype=f32, device=dev)
        self.sync = torch.zeros(4, dtype=torch.int32, device=dev)
        self.coop = os.environ.get("SMC_PF_COOP", "1") not in ("0", "false", "off")
        self.ctx_hint = 0
        self.trace: Optional[torch.Tensor] = None       # int64 [phases, ctas, 2] when a phase timeline is wanted
        self._tables: Dict[Tuple, torch.Tensor] = {}
        self._plans: Dict[Tuple, Tuple] = {}

    # ---- launch geometry -----------------------------------------------------------------------------
    @staticmethod
    def bn_for(M: int) -> int:
        for bn in (16, 32, 48, 64, 80, 96, 112, 128):
            if M <= bn:
                return bn
        raise ValueError("more than 128 token rows")

    def plan(self, E: int, BN: int):
        key = (E, BN)
        pl = self._plans.get(key)
        if pl is None:
            outs = [C.c_int(0) for _ in range(6)]
            rc = _lib().smc_pf_plan(self.D, E, self.nq // self.nkv, BN, *[C.byref(o) for o in outs])
            if rc != 0:
                raise K.NativeError(f"smc_pf_plan failed with code {rc}")
            pl = self._plans[key] = tuple(o.value for o in outs)   # n_mt, n_kw, att_stg, att_bytes, stages, ring_bytes
        return pl

    def kv_splits(self, bs: int, E: int, ctx: int) -> int:
        """Key-range splits of the attention phase: as many as keep every CTA on one (sequence, kv head, split) item
        with at least two 32-key tiles per key-way."""
        n_mt, n_kw = self.plan(E, self.bn_for(bs * E))[:2]
        ks = 1
        while ks < 8 and bs * self.nkv * ks * 2 <= self.ncta and ctx // (ks * 2 * 32 * n_kw) >= 2:
            ks *= 2
        return ks

    def set_context(self, ctx: int, bs: int, Es=(1, 2)) -> tuple:
        self.ctx_hint = int(ctx)
        return tuple(self.kv_splits(bs, E, self.ctx_hint) for E in Es)

    def _table(self, M: int, BN: int, lm_rows: int, lm_off: int, lm_step: int) -> torch.Tensor:
        key = (M, BN, lm_rows, lm_off, lm_step)
        t = self._tables.get(key)
        if t is None:
            L = _lib()
            n = 4 * self.nl + 5
            host = torch.zeros(n, 128, dtype=torch.uint8)
            base = host.data_ptr()

            def enc(i, tensor_ptr, rows, cols, ld, box):
                rc = L.smc_pf_encode_map(C.c_void_p(base + 128 * i), C.c_void_p(tensor_ptr), rows, cols, ld, box)
                if rc != 0:
                    raise K.NativeError(f"tensor map encode failed with code {rc}")
            for li, lw in enumerate(self.m.layers):
                for j, W in enumerate((lw.wqkv, lw.wo, lw.wgu, lw.wdown)):
                    assert W.is_contiguous()
                    enc(4 * li + j, W.data_ptr(), W.shape[0], W.shape[1], W.shape[1], 128)
            Wl = self.m.lm_head
            enc(4 * self.nl, Wl.data_ptr(), Wl.shape[0], Wl.shape[1], Wl.shape[1], 128)
            x0 = 4 * self.nl + 1
            enc(x0, self.hb.data_ptr(), M, self.d, self.d, BN)
            enc(x0 + 1, self.attn.data_ptr(), M, self.nq * self.D, self.nq * self.D, BN)
            enc(x0 + 2, self.act.data_ptr(), M, self.ffn, self.ffn, BN)
            enc(x0 + 3, self.hb.data_ptr() + 2 * self.d * lm_off, max(lm_rows, 1), self.d, self.d * max(lm_step, 1), BN)
            t = self._tables[key] = host.to(self.dev)
        return t

    # ---- one forward ------------------------------------------------------------------------------
    def run(self, ids, positions, cache_locs, rows, prefix_lens, bs: int, E: int, *, lm_rows: int = 0, lm_off: int = 0,
            lm_step: int = 1, temperature: float = 1.0, alpha: float = 1.0, tokens_in=None, seed: int = 0,
            cycle_counter=None, call_id: int = 0, tok_out=None, logp_out=None, logz_out=None) -> None:
        M = bs * E
        if M > self.T:
            raise ValueError("batch exceeds the persistent kernel's buffers")
        BN = self.bn_for(M)
        n_mt, n_kw, att_stg, att_bytes, stages, ring_bytes = self.plan(E, BN)
        KS = self.kv_splits(bs, E, self.ctx_hint)
        need = bs * self.nkv * KS * n_mt * (16 * self.D + 64)
        if KS > 1 and self.att_part.numel() < need:
            self.att_part = torch.zeros(need, dtype=torch.float32, device=self.dev)
        c, m = self.c, self.m
        p = PfParams()
        p.L, p.d, p.Hq, p.Hkv, p.D, p.ffn, p.V, p.nqkv = self.nl, self.d, self.nq, self.nkv, self.D, self.ffn, self.V, self.nqkv
        p.rd, p.max_pos = m.rope.shape[1], m.rope.shape[0]
        p.n_pages, p.bt_stride = self.kv.k.shape[1] - 1, self.bt.stride(0)
        p.rms_eps, p.softcap, p.scale = float(c.rms_eps), float(c.logit_softcap), float(self.D) ** -0.5
        p.maps = self._table(M, BN, lm_rows, lm_off, lm_step).data_ptr()
        p.embed, p.rope = m.embed.data_ptr(), m.rope.data_ptr()
        p.k_pool, p.v_pool = self.kv.k.data_ptr(), self.kv.v.data_ptr()
        p.kv_layer_stride = self.kv.k.stride(0)
        p.block_table = self.bt.data_ptr()
        p.bs, p.E, p.M, p.BN, p.KS, p.lm_rows = bs, E, M, BN, KS, lm_rows
        p.n_mt, p.n_kw, p.att_stg, p.stages, p.ring_bytes, p.att_bytes = n_mt, n_kw, att_stg, stages, ring_bytes, att_bytes
        p.lm_row_off, p.lm_row_step = lm_off, lm_step
        p.ids, p.positions, p.cache_locs = ids.data_ptr(), positions.data_ptr(), cache_locs.data_ptr()
        p.rows, p.prefix_lens = rows.data_ptr(), prefix_lens.data_ptr()
        p.h, p.hb, p.ssq, p.qkv = self.h.data_ptr(), self.hb.data_ptr(), self.ssq.data_ptr(), self.qkv.data_ptr()
        p.attn, p.act, p.ssq_ld = self.attn.data_ptr(), self.act.data_ptr(), self.ssq_ld
        p.att_part, p.att_ctr = self.att_part.data_ptr(), self.att_ctr.data_ptr()
        p.inv_temp, p.alpha = 1.0 / float(temperature), float(alpha)
        p.tokens_in = None if tokens_in is None else tokens_in.data_ptr()
        p.seed = int(seed) & 0xFFFFFFFFFFFFFFFF
        p.cycle_counter = None if cycle_counter is None else cycle_counter.data_ptr()
        p.call_id = int(call_id)
        p.sparts = self.sparts.data_ptr()
        p.tok_out = None if tok_out is None else tok_out.data_ptr()
        p.logp_out = None if logp_out is None else logp_out.data_ptr()
        p.logz_out = None if logz_out is None else logz_out.data_ptr()
        p.sync, p.status = self.sync.data_ptr(), self.status.data_ptr()
        p.trace = None if self.trace is None else self.trace.data_ptr()
        if lm_rows > 0 and (cycle_counter is None or tok_out is None or logp_out is None):
            raise ValueError("sampling outputs and the cycle counter are required when lm_rows > 0")
        K._check(_lib().smc_pf_forward(C.byref(p), int(self.coop), K._stream()), "smc_pf_forward")

    def n_phases(self, lm_rows: int) -> int:
        return 1 + 5 * self.nl + (2 if lm_rows > 0 else 0)

    def enable_trace(self) -> torch.Tensor:
        """Allocate the phase-timeline buffer: per (phase, CTA) eight nanosecond stamps (0: inputs seen ready, 1: work done, 2..: details of the GEMM epilogue)."""
        self.trace = torch.zeros(self.n_phases(1), self.ncta, 8, dtype=torch.int64, device=self.dev)
        return self.trace

    def reset_sync(self) -> None:
        """Rearm the barrier counters after a launch that reported an error."""
        self.sync.zero_()
        self.att_ctr.zero_()
