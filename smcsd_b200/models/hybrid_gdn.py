"""Qwen3.5-style hybrid decoder: Gated-DeltaNet (linear attention) layers interleaved with gated
full-attention layers (every ``full_attention_interval``-th layer), (1 + w) RMSNorm, per-head
q/k RMSNorm, partial rotary embedding, SwiGLU MLP.

Parameter names and math follow the HF implementation shipped with transformers
(models/qwen3_5/modeling_qwen3_5.py: Qwen3_5GatedDeltaNet :356-533, Qwen3_5Attention :620-692,
torch_recurrent_gated_delta_rule :314-353); HF checkpoints load unchanged.  The reference serves
these models through SGLang's hybrid linear-attention backend (smcsd/core/hybrid_multistep_backend.py,
smcsd/core/worker.py:549-602).

Fused weight layout per layer type:
  attention  wqkv [2*Hq*D + 2*Hkv*D, d] = query heads | output-gate heads | key heads | value heads
  GDN        win  [conv_dim + value_dim + 2*Hv, d] = mixed qkv (conv input) | z | b | a
Recurrent state per sequence row: conv window [conv_dim, width-1] and S [Hv, dk, dv] (fp32).
Because SMC accepts every drafted token, a multi-token pass always ends on the state of its
last token, so the state is advanced in place (no per-position snapshots are needed).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from ..memory.pools import StateSpec
from .config import ModelConfig
from .layers import ExtendBatch, apply_rope, paged_attention_reference, rmsnorm, rope_table, swiglu
from .llama import interleave_gate_up, split_gate_up
from .loader import Checkpoint, strip_prefixes


@dataclass
class HybridLayerWeights:
    kind: str                      # "full_attention" | "linear_attention"
    ln1: torch.Tensor
    ln2: torch.Tensor
    wgu: torch.Tensor
    wdown: torch.Tensor
    # attention
    wqkv: Optional[torch.Tensor] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    wo: Optional[torch.Tensor] = None
    # gated delta net
    win: Optional[torch.Tensor] = None
    conv_w: Optional[torch.Tensor] = None      # [conv_dim, width]
    dt_bias: Optional[torch.Tensor] = None     # [Hv] fp32
    A_log: Optional[torch.Tensor] = None       # [Hv] fp32
    gnorm_w: Optional[torch.Tensor] = None     # [dv]
    wout: Optional[torch.Tensor] = None        # [d, value_dim]


def gdn_recurrent_step(S, q, k, v, g, beta):
    """One token of the gated delta rule for a batch of heads.
    S [.., dk, dv] fp32; q, k [.., dk] (l2-normalised, q pre-scaled); v [.., dv]; g, beta [..]."""
    S = S * g.exp().unsqueeze(-1).unsqueeze(-1)
    kv_mem = (S * k.unsqueeze(-1)).sum(dim=-2)
    delta = (v - kv_mem) * beta.unsqueeze(-1)
    S = S + k.unsqueeze(-1) * delta.unsqueeze(-2)
    out = (S * q.unsqueeze(-1)).sum(dim=-2)
    return S, out


def gdn_chunked(S, q, k, v, g, beta, chunk: int = 64):
    """Chunk-parallel gated delta rule for long passes (prefill): same recurrence as ``gdn_recurrent_step`` applied
    token by token, evaluated with the WY / forward-substitution form inside chunks of ``chunk`` tokens.
    S [H, dk, dv]; q, k [T, H, dk]; v [T, H, dv]; g, beta [T, H].  Returns (S_final, out [T, H, dv])."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    pad = (-T) % chunk
    if pad:
        z = lambda x: torch.cat([x, x.new_zeros(pad, *x.shape[1:])], dim=0)
        q, k, v, g, beta = z(q), z(k), z(v), z(g), z(beta)
    n = (T + pad) // chunk
    # [H, n, C, *]
    q, k, v = (x.view(n, chunk, H, -1).permute(2, 0, 1, 3) for x in (q, k, v))
    g = g.view(n, chunk, H).permute(2, 0, 1)
    beta = beta.view(n, chunk, H).permute(2, 0, 1)
    gc = g.cumsum(-1)
    k_beta, v_beta = k * beta.unsqueeze(-1), v * beta.unsqueeze(-1)
    tril = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    decay = torch.where(tril, (gc.unsqueeze(-1) - gc.unsqueeze(-2)).exp(), torch.zeros((), device=q.device))
    strict = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), -1)
    A = -(k_beta @ k.transpose(-1, -2)) * decay
    A = torch.where(strict, A, torch.zeros((), device=q.device))
    for i in range(1, chunk):
        row = A[..., i, :i].clone()
        A[..., i, :i] = row + (row.unsqueeze(-1) * A[..., :i, :i]).sum(-2)
    A = A + torch.eye(chunk, device=q.device)
    v_w = A @ v_beta
    k_cum = A @ (k_beta * gc.exp().unsqueeze(-1))
    out = torch.empty(H, n, chunk, dv, device=q.device, dtype=q.dtype)
    for c in range(n):
        qc, kc, vc = q[:, c], k[:, c], v_w[:, c]
        local = torch.where(tril, (qc @ kc.transpose(-1, -2)) * decay[:, c], torch.zeros((), device=q.device))
        v_new = vc - k_cum[:, c] @ S
        out[:, c] = (qc * gc[:, c].exp().unsqueeze(-1)) @ S + local @ v_new
        last = gc[:, c, -1]
        S = S * last.exp().view(H, 1, 1) + (kc * (last.unsqueeze(-1) - gc[:, c]).exp().unsqueeze(-1)).transpose(-1, -2) @ v_new
    out = out.permute(1, 2, 0, 3).reshape(n * chunk, H, dv)[:T]
    return S, out


class HybridGDNModel:
    has_state = True

    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", tp_rank: int = 0, tp_size: int = 1,
                 max_positions: Optional[int] = None):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.tp_rank, self.tp_size = tp_rank, tp_size
        w = tp_size
        if cfg.n_heads % w or cfg.n_kv_heads % w or cfg.ffn_size % w or cfg.gdn_n_k_heads % w or cfg.gdn_n_v_heads % w:
            raise ValueError("tensor-parallel size must divide the attention, KV, Gated-DeltaNet head counts and the FFN size")
        # per-rank shares: attention heads, KV heads, Gated-DeltaNet key / value heads, FFN channels, vocabulary rows
        self.n_heads, self.n_kv_heads, self.ffn = cfg.n_heads // w, cfg.n_kv_heads // w, cfg.ffn_size // w
        self.gdn_k_heads, self.gdn_v_heads = cfg.gdn_n_k_heads // w, cfg.gdn_n_v_heads // w
        self.vocab_shard = (cfg.vocab_size + w - 1) // w
        self.gu_block = 64 if self.ffn % 64 == 0 else self.ffn
        self.layers: List[HybridLayerWeights] = []
        self.embed = self.lm_head = self.final_norm = None
        mp = min(max_positions or cfg.max_position, cfg.max_position)
        self.rope = rope_table(cfg.rotary_dim, cfg.rope_theta, cfg.rope_scaling, mp, self.device)
        self.tp_group = None                              # torch.distributed group of the tensor-parallel ranks
        self.kv_index = {li: i for i, li in enumerate(cfg.attn_layers)}
        self.state_index = {li: i for i, li in enumerate(cfg.gdn_layers)}
        self.key_dim = self.gdn_k_heads * cfg.gdn_head_k_dim
        self.value_dim = self.gdn_v_heads * cfg.gdn_head_v_dim
        self.conv_dim = 2 * self.key_dim + self.value_dim

    def state_spec(self) -> StateSpec:
        c = self.cfg
        return StateSpec(len(c.gdn_layers), self.conv_dim, c.gdn_conv_width, self.gdn_v_heads, c.gdn_head_k_dim,
                         c.gdn_head_v_dim, conv_dtype=torch.float32, state_dtype=torch.float32)

    def all_tensors(self):
        for t in (self.embed, self.lm_head, self.final_norm):
            if t is not None:
                yield t
        for L in self.layers:
            for t in vars(L).values():
                if isinstance(t, torch.Tensor):
                    yield t

    def weight_bytes(self) -> int:
        seen, n = set(), 0
        for t in self.all_tensors():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()
        return n

    # ---- construction ---------------------------------------------------------------
    def _rows(self, w: torch.Tensor, n_units: int) -> torch.Tensor:
        """This rank's share of a tensor whose leading dimension is ``n_units`` equal blocks (heads, channels)."""
        if self.tp_size == 1:
            return w
        per = w.shape[0] // n_units * (n_units // self.tp_size)
        return w[self.tp_rank * per:(self.tp_rank + 1) * per]

    def _cols(self, w: torch.Tensor, n_units: int) -> torch.Tensor:
        if self.tp_size == 1:
            return w
        per = w.shape[1] // n_units * (n_units // self.tp_size)
        return w[:, self.tp_rank * per:(self.tp_rank + 1) * per]

    def _shard_vocab(self, head: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1:
            return head
        lo = self.tp_rank * self.vocab_shard
        hi = min(lo + self.vocab_shard, head.shape[0])
        out = torch.zeros(self.vocab_shard, head.shape[1], dtype=head.dtype, device=head.device)
        if hi > lo:
            out[:hi - lo] = head[lo:hi]
        return out

    def _pack_attn(self, ln1, ln2, wg, wu, wd, q_proj, k_proj, v_proj, o_proj, q_norm, k_norm) -> HybridLayerWeights:
        """Arguments are the full (unsharded) tensors; the rank keeps its heads / FFN channels."""
        c = self.cfg
        H, Hkv, D = c.n_heads, c.n_kv_heads, c.head_dim
        k_proj, v_proj, o_proj = self._rows(k_proj, Hkv), self._rows(v_proj, Hkv), self._cols(o_proj, H)
        if c.attn_output_gate:
            qp = self._rows(q_proj, H).view(self.n_heads, 2, D, -1)         # HF stores [query | gate] per head
            q_rows, gate_rows = qp[:, 0].reshape(self.n_heads * D, -1), qp[:, 1].reshape(self.n_heads * D, -1)
            wqkv = torch.cat([q_rows, gate_rows, k_proj, v_proj], dim=0).contiguous()
        else:
            wqkv = torch.cat([self._rows(q_proj, H), k_proj, v_proj], dim=0).contiguous()
        wg, wu, wd = self._rows(wg, self.tp_size), self._rows(wu, self.tp_size), self._cols(wd, self.tp_size)
        return HybridLayerWeights("full_attention", ln1.contiguous(), ln2.contiguous(),
                                  interleave_gate_up(wg.contiguous(), wu.contiguous(), self.gu_block), wd.contiguous(),
                                  wqkv=wqkv, q_norm=q_norm.contiguous(), k_norm=k_norm.contiguous(),
                                  wo=o_proj.contiguous())

    def _pack_gdn(self, ln1, ln2, wg, wu, wd, w_qkv, w_z, w_b, w_a, conv_w, dt_bias, A_log, gnorm_w, w_out):
        """Arguments are the full tensors.  A rank keeps its key heads' q and k channels and its value heads' v, z,
        b, a channels (of the in-projection and of the depthwise conv alike) and the matching out-projection columns."""
        c = self.cfg
        Hk, Hv = c.gdn_n_k_heads, c.gdn_n_v_heads
        kd, vd = Hk * c.gdn_head_k_dim, Hv * c.gdn_head_v_dim

        def mixed(t):           # [q | k | v] channel blocks of the conv input
            return torch.cat([self._rows(t[:kd], Hk), self._rows(t[kd:2 * kd], Hk), self._rows(t[2 * kd:], Hv)], dim=0)
        win = torch.cat([mixed(w_qkv), self._rows(w_z, Hv), self._rows(w_b, Hv), self._rows(w_a, Hv)], dim=0)
        pad = (-win.shape[0]) % 8
        if pad:                                    # keep the row count friendly to 16-byte tiles
            win = torch.cat([win, torch.zeros(pad, win.shape[1], dtype=win.dtype, device=win.device)], dim=0)
        wg, wu, wd = self._rows(wg, self.tp_size), self._rows(wu, self.tp_size), self._cols(wd, self.tp_size)
        return HybridLayerWeights("linear_attention", ln1.contiguous(), ln2.contiguous(),
                                  interleave_gate_up(wg.contiguous(), wu.contiguous(), self.gu_block), wd.contiguous(),
                                  win=win.contiguous(), conv_w=mixed(conv_w).contiguous(),
                                  dt_bias=self._rows(dt_bias.float(), Hv).contiguous(),
                                  A_log=self._rows(A_log.float(), Hv).contiguous(), gnorm_w=gnorm_w.contiguous(),
                                  wout=self._cols(w_out, Hv).contiguous())

    def init_random(self, seed: int = 0, std: float = 0.02) -> "HybridGDNModel":
        c = self.cfg
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        dev, dt = self.device, self.dtype

        def rnd(*shape, scale=std):
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale).to(dt)

        d, f = c.hidden_size, c.ffn_size
        kd_full, vd_full = c.gdn_n_k_heads * c.gdn_head_k_dim, c.gdn_n_v_heads * c.gdn_head_v_dim
        conv_full = 2 * kd_full + vd_full
        self.embed = rnd(c.vocab_size, d)
        self.final_norm = torch.zeros(d, dtype=dt, device=dev)
        for li in range(c.n_layers):
            ln1, ln2 = rnd(d, scale=0.05), rnd(d, scale=0.05)
            wg, wu, wd = rnd(f, d), rnd(f, d), rnd(d, f)
            if c.layer_type(li) == "full_attention":
                qmul = 2 if c.attn_output_gate else 1
                self.layers.append(self._pack_attn(ln1, ln2, wg, wu, wd, rnd(c.q_size * qmul, d), rnd(c.kv_size, d),
                                                   rnd(c.kv_size, d), rnd(d, c.q_size), rnd(c.head_dim, scale=0.05),
                                                   rnd(c.head_dim, scale=0.05)))
            else:
                Hv = c.gdn_n_v_heads
                A = torch.empty(Hv, device=dev).uniform_(0.5, 8.0, generator=g)
                self.layers.append(self._pack_gdn(
                    ln1, ln2, wg, wu, wd, rnd(conv_full, d), rnd(vd_full, d), rnd(Hv, d), rnd(Hv, d),
                    rnd(conv_full, c.gdn_conv_width, scale=0.3), torch.ones(Hv, device=dev), torch.log(A),
                    torch.ones(c.gdn_head_v_dim, dtype=dt, device=dev), rnd(d, vd_full)))
        head = self.embed if c.tie_embeddings else rnd(c.vocab_size, d)
        self.lm_head = head if self.tp_size == 1 else self._shard_vocab(head)
        return self

    def load_hf(self, path: str) -> "HybridGDNModel":
        ck = Checkpoint(path)
        pre = strip_prefixes(ck)
        c, dev, dt = self.cfg, self.device, self.dtype

        def get(name, dtype=None):
            return ck.get(name).to(device=dev, dtype=dtype or dt, copy=True)   # never alias the mmap

        self.embed = get(f"{pre}embed_tokens.weight")
        self.final_norm = get(f"{pre}norm.weight")
        for li in range(c.n_layers):
            p = f"{pre}layers.{li}."
            common = (get(p + "input_layernorm.weight"), get(p + "post_attention_layernorm.weight"),
                      get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight"), get(p + "mlp.down_proj.weight"))
            if c.layer_type(li) == "full_attention":
                a = p + "self_attn."
                self.layers.append(self._pack_attn(*common, get(a + "q_proj.weight"), get(a + "k_proj.weight"),
                                                   get(a + "v_proj.weight"), get(a + "o_proj.weight"),
                                                   get(a + "q_norm.weight"), get(a + "k_norm.weight")))
            else:
                a = p + "linear_attn."
                self.layers.append(self._pack_gdn(
                    *common, get(a + "in_proj_qkv.weight"), get(a + "in_proj_z.weight"), get(a + "in_proj_b.weight"),
                    get(a + "in_proj_a.weight"), get(a + "conv1d.weight").squeeze(1), get(a + "dt_bias", torch.float32),
                    get(a + "A_log", torch.float32), get(a + "norm.weight"), get(a + "out_proj.weight")))
        for cand in ("lm_head.weight", "language_model.lm_head.weight"):
            if cand in ck and not c.tie_embeddings:
                self.lm_head = self._shard_vocab(get(cand))
                break
        else:
            self.lm_head = self.embed if self.tp_size == 1 else self._shard_vocab(self.embed)
        ck.close()
        return self

    # ---- plain-PyTorch forward --------------------------------------------------------
    def _gdn_layer(self, L: HybridLayerWeights, x: torch.Tensor, batch: ExtendBatch, state, si: int) -> torch.Tensor:
        """x [T, d] normalised input; returns the mixer output [T, d] and advances the recurrent state."""
        c = self.cfg
        Hk, Hv, dk, dv, W = self.gdn_k_heads, self.gdn_v_heads, c.gdn_head_k_dim, c.gdn_head_v_dim, c.gdn_conv_width
        proj = (x @ L.win.t()).float()
        mixed = proj[:, :self.conv_dim]
        z = proj[:, self.conv_dim:self.conv_dim + self.value_dim].view(-1, Hv, dv)
        bb = proj[:, self.conv_dim + self.value_dim:self.conv_dim + self.value_dim + Hv]
        aa = proj[:, self.conv_dim + self.value_dim + Hv:self.conv_dim + self.value_dim + 2 * Hv]
        beta = torch.sigmoid(bb)
        g = -L.A_log.exp() * F.softplus(aa + L.dt_bias)
        out = torch.empty(x.shape[0], Hv, dv, dtype=torch.float32, device=x.device)
        srows = (batch.state_rows if batch.state_rows is not None else batch.rows).long()
        conv_w = L.conv_w.float()
        rep = Hv // Hk
        t0 = 0
        for b, e_len in enumerate(batch.lens()):
            if e_len == 0:
                continue
            r = srows[b]
            window = state.conv[si, r].float()               # [conv_dim, W-1]
            S = state.temporal[si, r].float()                # [Hv, dk, dv]
            seq = torch.cat([window, mixed[t0:t0 + e_len].t()], dim=1)      # [conv_dim, W-1+e]
            conv = F.silu(F.conv1d(seq.unsqueeze(0), conv_w.unsqueeze(1), groups=self.conv_dim).squeeze(0))  # [conv_dim, e]
            state.conv[si, r] = seq[:, -(W - 1):].to(state.conv.dtype)
            conv = conv.t()
            q = conv[:, :self.key_dim].reshape(e_len, Hk, dk)
            k = conv[:, self.key_dim:2 * self.key_dim].reshape(e_len, Hk, dk)
            v = conv[:, 2 * self.key_dim:].reshape(e_len, Hv, dv)
            q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * (dk ** -0.5)
            k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            if rep > 1:
                q = q.repeat_interleave(rep, dim=1)
                k = k.repeat_interleave(rep, dim=1)
            if e_len >= 32:          # prefill: chunk-parallel form
                S, o = gdn_chunked(S, q, k, v, g[t0:t0 + e_len], beta[t0:t0 + e_len])
                out[t0:t0 + e_len] = o
            else:
                for t in range(e_len):
                    S, o = gdn_recurrent_step(S, q[t], k[t], v[t], g[t0 + t], beta[t0 + t])
                    out[t0 + t] = o
            state.temporal[si, r] = S.to(state.temporal.dtype)
            t0 += e_len
        # gated RMSNorm over each head's dv (plain weight), then the output projection
        y = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + c.rms_eps)
        y = (y.to(x.dtype).float() * L.gnorm_w.float()) * F.silu(z)
        return y.reshape(x.shape[0], -1).to(x.dtype) @ L.wout.t()

    def _attn_layer(self, L: HybridLayerWeights, x, batch: ExtendBatch, kv, block_table, ki: int) -> torch.Tensor:
        c = self.cfg
        T, H, Hkv, D = x.shape[0], self.n_heads, self.n_kv_heads, c.head_dim
        qkv = x @ L.wqkv.t()
        nq = H * D
        off = 2 * nq if c.attn_output_gate else nq
        q = qkv[:, :nq].view(T, H, D)
        gate = qkv[:, nq:2 * nq] if c.attn_output_gate else None
        k = qkv[:, off:off + Hkv * D].view(T, Hkv, D)
        v = qkv[:, off + Hkv * D:].view(T, Hkv, D)
        q = rmsnorm(q, L.q_norm, c.rms_eps, plus_one=c.norm_plus_one)
        k = rmsnorm(k, L.k_norm, c.rms_eps, plus_one=c.norm_plus_one)
        q = apply_rope(q, batch.positions, self.rope)
        k = apply_rope(k, batch.positions, self.rope)
        kv.write(ki, batch.cache_locs, k, v)
        a = paged_attention_reference(q, kv.k[ki], kv.v[ki], block_table, batch, Hkv).reshape(T, -1)
        if gate is not None:
            a = (a.float() * torch.sigmoid(gate.float())).to(x.dtype)
        return a @ L.wo.t()

    def forward_torch(self, batch: ExtendBatch, kv, block_table: torch.Tensor, state=None) -> torch.Tensor:
        c = self.cfg
        if state is None:
            raise ValueError("hybrid models need a recurrent-state pool")
        h = self.embed[batch.input_ids.long()]
        for li, L in enumerate(self.layers):
            x = rmsnorm(h, L.ln1, c.rms_eps, plus_one=c.norm_plus_one)
            if L.kind == "full_attention":
                h = h + self._all_reduce(self._attn_layer(L, x, batch, kv, block_table, self.kv_index[li]))
            else:
                h = h + self._all_reduce(self._gdn_layer(L, x, batch, state, self.state_index[li]))
            x = rmsnorm(h, L.ln2, c.rms_eps, plus_one=c.norm_plus_one)
            gate, up = split_gate_up(x @ L.wgu.t(), self.gu_block)
            h = h + self._all_reduce(swiglu(gate, up) @ L.wdown.t())
        return rmsnorm(h, self.final_norm, c.rms_eps, plus_one=c.norm_plus_one)

    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of the ranks' partial products (row-parallel projections: attention / Gated-DeltaNet out, MLP down)."""
        if self.tp_size > 1 and self.tp_group is not None:
            import torch.distributed as dist
            x = x.contiguous()
            dist.all_reduce(x, group=self.tp_group)
        return x

    def logits_torch(self, hidden: torch.Tensor) -> torch.Tensor:
        lg = (hidden @ self.lm_head.t()).float()
        if self.tp_size > 1 and self.tp_group is not None:
            import torch.distributed as dist
            parts = [torch.empty_like(lg) for _ in range(self.tp_size)]
            dist.all_gather(parts, lg, group=self.tp_group)
            lg = torch.cat(parts, dim=-1)[..., :self.cfg.vocab_size]
        if self.cfg.logit_softcap > 0:
            cap = self.cfg.logit_softcap
            lg = torch.tanh(lg / cap) * cap
        return lg
