"""Dense Llama-style decoder: fused weight layout, HF loading, random init and the
plain-PyTorch forward (oracle, CPU path, cuBLAS baseline).

Weight layout (shared with the sm_100a kernels, which stream these matrices as the
128-row operand of a swapped GEMM):
  wqkv [q + 2*kv, d]   rows = all query heads, then key heads, then value heads
  wo   [d, q]
  wgu  [2*ffn, d]      gate and up rows interleaved in blocks of ``gu_block`` channels
                       (block j: gate channels [j*B,(j+1)*B) then up channels of the same range)
                       so a GEMM tile holds matching gate/up rows and can apply SwiGLU itself
  wdown [d, ffn]
Under tensor parallelism every matrix holds this rank's shard (heads / ffn channels).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .config import ModelConfig
from .layers import ExtendBatch, apply_rope, paged_attention_reference, rmsnorm, rope_table, swiglu
from .loader import Checkpoint, strip_prefixes


@dataclass
class LlamaLayerWeights:
    ln1: torch.Tensor
    wqkv: torch.Tensor
    wo: torch.Tensor
    ln2: torch.Tensor
    wgu: torch.Tensor
    wdown: torch.Tensor


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    f, d = gate.shape
    g = gate.view(f // block, 1, block, d)
    u = up.view(f // block, 1, block, d)
    return torch.cat([g, u], dim=1).reshape(2 * f, d).contiguous()


def split_gate_up(y: torch.Tensor, block: int):
    """Inverse view of ``interleave_gate_up`` on a GEMM output [T, 2*ffn]."""
    T, two_f = y.shape
    v = y.view(T, two_f // (2 * block), 2, block)
    return v[:, :, 0, :].reshape(T, -1), v[:, :, 1, :].reshape(T, -1)


class LlamaModel:
    def __init__(self, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu", tp_rank: int = 0, tp_size: int = 1,
                 max_positions: Optional[int] = None):
        self.cfg = cfg
        self.dtype = dtype
        self.device = torch.device(device)
        self.tp_rank, self.tp_size = tp_rank, tp_size
        assert cfg.n_heads % tp_size == 0 and cfg.n_kv_heads % tp_size == 0 and cfg.ffn_size % tp_size == 0
        self.n_heads = cfg.n_heads // tp_size
        self.n_kv_heads = cfg.n_kv_heads // tp_size
        self.ffn = cfg.ffn_size // tp_size
        self.gu_block = 64 if self.ffn % 64 == 0 else self.ffn
        self.vocab_shard = (cfg.vocab_size + tp_size - 1) // tp_size
        self.layers: List[LlamaLayerWeights] = []
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None      # [V (or this rank's vocab shard), d]
        self.final_norm: Optional[torch.Tensor] = None
        mp = min(max_positions or cfg.max_position, cfg.max_position)
        self.rope = rope_table(cfg.rotary_dim, cfg.rope_theta, cfg.rope_scaling, mp, self.device)
        self.tp_group = None                              # torch.distributed group for the baseline path

    # ---- parameters ------------------------------------------------------------
    @property
    def kv_layers(self) -> int:
        return self.cfg.n_layers

    def weight_bytes(self) -> int:
        n = 0
        for t in self.all_tensors():
            n += t.numel() * t.element_size()
        return n

    def all_tensors(self):
        seen = set()
        for t in [self.embed, self.lm_head, self.final_norm]:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                yield t
        for L in self.layers:
            for t in (L.ln1, L.wqkv, L.wo, L.ln2, L.wgu, L.wdown):
                yield t

    def init_random(self, seed: int = 0, std: float = 0.02) -> "LlamaModel":
        """Random weights drawn on the target device; every TP rank draws the full matrix
        from the same seed and keeps its shard, so sharded and unsharded runs agree."""
        c = self.cfg
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)

        def rnd(*shape, scale=std):
            return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * scale).to(self.dtype)

        self.embed = rnd(c.vocab_size, c.hidden_size)
        self.final_norm = torch.ones(c.hidden_size, dtype=self.dtype, device=self.device)
        r, w = self.tp_rank, self.tp_size
        for _ in range(c.n_layers):
            wq = rnd(c.q_size, c.hidden_size)
            wk = rnd(c.kv_size, c.hidden_size)
            wv = rnd(c.kv_size, c.hidden_size)
            wo = rnd(c.hidden_size, c.q_size)
            wg = rnd(c.ffn_size, c.hidden_size)
            wu = rnd(c.ffn_size, c.hidden_size)
            wd = rnd(c.hidden_size, c.ffn_size)
            self.layers.append(self._pack_layer(
                torch.ones(c.hidden_size, dtype=self.dtype, device=self.device), wq, wk, wv, wo,
                torch.ones(c.hidden_size, dtype=self.dtype, device=self.device), wg, wu, wd))
        head = self.embed if c.tie_embeddings else rnd(c.vocab_size, c.hidden_size)
        self.lm_head = self._shard_vocab(head)
        return self

    def _shard_vocab(self, head: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1:
            return head
        lo = self.tp_rank * self.vocab_shard
        hi = min(lo + self.vocab_shard, head.shape[0])
        out = torch.zeros(self.vocab_shard, head.shape[1], dtype=head.dtype, device=head.device)
        out[:hi - lo] = head[lo:hi]
        return out

    def _pack_layer(self, ln1, wq, wk, wv, wo, ln2, wg, wu, wd) -> LlamaLayerWeights:
        r, w = self.tp_rank, self.tp_size
        if w > 1:
            def rows(t):
                n = t.shape[0] // w
                return t[r * n:(r + 1) * n]

            def cols(t):
                n = t.shape[1] // w
                return t[:, r * n:(r + 1) * n]
            wq, wk, wv, wg, wu = rows(wq), rows(wk), rows(wv), rows(wg), rows(wu)
            wo, wd = cols(wo), cols(wd)
        wqkv = torch.cat([wq, wk, wv], dim=0).contiguous()
        wgu = interleave_gate_up(wg.contiguous(), wu.contiguous(), self.gu_block)
        return LlamaLayerWeights(ln1.contiguous(), wqkv, wo.contiguous(), ln2.contiguous(), wgu, wd.contiguous())

    def load_hf(self, path: str) -> "LlamaModel":
        ck = Checkpoint(path)
        pre = strip_prefixes(ck)
        dev, dt = self.device, self.dtype

        def get(name):
            return ck.get(name).to(device=dev, dtype=dt, copy=True)   # never alias the mmap

        self.embed = get(f"{pre}embed_tokens.weight")
        self.final_norm = get(f"{pre}norm.weight")
        for i in range(self.cfg.n_layers):
            p = f"{pre}layers.{i}."
            self.layers.append(self._pack_layer(
                get(p + "input_layernorm.weight"), get(p + "self_attn.q_proj.weight"),
                get(p + "self_attn.k_proj.weight"), get(p + "self_attn.v_proj.weight"),
                get(p + "self_attn.o_proj.weight"), get(p + "post_attention_layernorm.weight"),
                get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight"), get(p + "mlp.down_proj.weight")))
        if "lm_head.weight" in ck and not self.cfg.tie_embeddings:
            head = get("lm_head.weight")
        else:
            head = self.embed
        self.lm_head = self._shard_vocab(head)
        ck.close()
        return self

    # ---- plain-PyTorch forward ---------------------------------------------------
    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1 and self.tp_group is not None:
            import torch.distributed as dist
            dist.all_reduce(x, group=self.tp_group)
        return x

    def forward_torch(self, batch: ExtendBatch, kv, block_table: torch.Tensor, state=None) -> torch.Tensor:
        """Runs all layers, writes the new tokens' K/V into ``kv`` and returns post-norm hidden [T, d]."""
        c = self.cfg
        h = self.embed[batch.input_ids.long()]
        T = h.shape[0]
        for li, L in enumerate(self.layers):
            x = rmsnorm(h, L.ln1, c.rms_eps)
            qkv = x @ L.wqkv.t()
            q = qkv[:, :self.n_heads * c.head_dim].view(T, self.n_heads, c.head_dim)
            k = qkv[:, self.n_heads * c.head_dim:(self.n_heads + self.n_kv_heads) * c.head_dim].view(T, self.n_kv_heads, c.head_dim)
            v = qkv[:, (self.n_heads + self.n_kv_heads) * c.head_dim:].view(T, self.n_kv_heads, c.head_dim)
            q = apply_rope(q, batch.positions, self.rope)
            k = apply_rope(k, batch.positions, self.rope)
            kv.write(li, batch.cache_locs, k, v)
            a = paged_attention_reference(q, kv.k[li], kv.v[li], block_table, batch, self.n_kv_heads)
            o = self._all_reduce(a.reshape(T, -1) @ L.wo.t())
            h = h + o
            x = rmsnorm(h, L.ln2, c.rms_eps)
            gate, up = split_gate_up(x @ L.wgu.t(), self.gu_block)
            d = self._all_reduce(swiglu(gate, up) @ L.wdown.t())
            h = h + d
        return rmsnorm(h, self.final_norm, c.rms_eps)

    def logits_torch(self, hidden: torch.Tensor) -> torch.Tensor:
        """fp32 logits over the full vocabulary (all-gathered across TP ranks on the baseline path)."""
        lg = (hidden @ self.lm_head.t()).float()
        if self.tp_size > 1 and self.tp_group is not None:
            import torch.distributed as dist
            parts = [torch.empty_like(lg) for _ in range(self.tp_size)]
            dist.all_gather(parts, lg, group=self.tp_group)
            lg = torch.cat(parts, dim=-1)[:, :self.cfg.vocab_size]
        if self.cfg.logit_softcap > 0:
            cap = self.cfg.logit_softcap
            lg = torch.tanh(lg / cap) * cap
        return lg

    def fold_norms(self) -> "LlamaModel":
        """Multiply every RMSNorm weight into the matrix that consumes the normalised activations (W <- W diag(w),
        w <- 1).  The function computed is unchanged; afterwards a GEMM can take the raw residual stream as its
        operand and apply only the per-token 1/rms factor in its epilogue."""
        if getattr(self, "_folded", False):
            return self
        for L in self.layers:
            L.wqkv = (L.wqkv.float() * L.ln1.float().unsqueeze(0)).to(self.dtype)
            L.wgu = (L.wgu.float() * L.ln2.float().unsqueeze(0)).to(self.dtype)
            L.ln1 = torch.ones_like(L.ln1)
            L.ln2 = torch.ones_like(L.ln2)
        if self.lm_head.data_ptr() == self.embed.data_ptr():
            self.lm_head = self.lm_head.clone()            # tied embeddings: the folded head needs its own copy
        self.lm_head = (self.lm_head.float() * self.final_norm.float().unsqueeze(0)).to(self.dtype)
        self.final_norm = torch.ones_like(self.final_norm)
        self._folded = True
        return self

    # recurrent-state hooks (no-ops for dense models)
    has_state = False

    def state_spec(self):
        return None
