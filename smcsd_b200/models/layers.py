"""Plain-PyTorch layer math: the fp32 oracle for the sm_100a kernels, the CPU path and
the cuBLAS baseline.  Also the batch descriptor shared by every forward mode.

One descriptor covers prefill, single-token decode, the two-token draft head and the
(gamma+1)-token verify pass: each sequence row has ``prefix_len`` tokens already in the
paged cache and ``extend_len`` new tokens, attended causally (the reference expresses
the same thing as EXTEND / TARGET_VERIFY forward modes, smcsd/core/info.py:206-365).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F


@dataclass
class ExtendBatch:
    input_ids: torch.Tensor        # [T]
    positions: torch.Tensor        # [T]
    cache_locs: torch.Tensor       # [T] page id each new token's K/V is written to
    rows: torch.Tensor             # [bs] block-table row of each sequence
    prefix_lens: torch.Tensor      # [bs] tokens already cached per row
    extend_len: int = 1            # uniform new tokens per row (0 => use extend_lens)
    extend_lens: Optional[List[int]] = None   # varlen (prefill) new tokens per row
    prefix_lens_host: Optional[List[int]] = None
    state_rows: Optional[torch.Tensor] = None  # [bs] recurrent-state rows (hybrids); defaults to rows
    save_steps: bool = False       # hybrids: keep per-position intermediate recurrent states
    logits_rows: Optional[torch.Tensor] = None  # token indices whose logits are wanted (None = all)

    @property
    def bs(self) -> int:
        return int(self.rows.shape[0])

    @property
    def uniform(self) -> bool:
        return self.extend_lens is None

    def lens(self) -> List[int]:
        return [self.extend_len] * self.bs if self.extend_lens is None else list(self.extend_lens)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, plus_one: bool = False) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + 1.0 if plus_one else w.float()
    return (y * wf).to(x.dtype)


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        if kind == "llama3":
            factor = scaling["factor"]
            lo, hi = scaling["low_freq_factor"], scaling["high_freq_factor"]
            old = scaling["original_max_position_embeddings"]
            wavelen = 2 * math.pi / inv
            smooth = ((old / wavelen) - lo) / (hi - lo)
            scaled = torch.where(wavelen > old / lo, inv / factor, inv)
            mid = (wavelen <= old / lo) & (wavelen >= old / hi)
            inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
        elif kind == "linear":
            inv = inv / scaling["factor"]
    return inv.float()


def rope_table(rotary_dim: int, theta: float, scaling: Optional[dict], max_pos: int, device) -> torch.Tensor:
    """[max_pos, rotary_dim] fp32: cos in the first half of each row, sin in the second."""
    inv = rope_inv_freq(rotary_dim, theta, scaling).to(device)
    ang = torch.arange(max_pos, device=device, dtype=torch.float32).unsqueeze(1) * inv.unsqueeze(0)
    return torch.cat([ang.cos(), ang.sin()], dim=-1).contiguous()


def apply_rope(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x [T, H, D]; rotates the first ``table.shape[1]`` dims (HF half-split convention)."""
    rd = table.shape[1]
    half = rd // 2
    cs = table[positions.long()]
    cos, sin = cs[:, :half].unsqueeze(1), cs[:, half:].unsqueeze(1)
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:rd]
    out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, xf[..., rd:]], dim=-1)
    return out.to(x.dtype)


def kv_rows_to_float(rows: torch.Tensor, n_kv_heads: int, head_dim: int) -> torch.Tensor:
    from ..memory.pools import kv_rows_to_float as f       # e4m3 page rows carry their scales (memory/pools.py)
    return f(rows, n_kv_heads, head_dim)


def paged_attention_reference(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                              block_table: torch.Tensor, batch: ExtendBatch, n_kv_heads: int,
                              scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention of the new tokens over [cached prefix + new tokens], all read through
    the block table (the new tokens' K/V must already be written).  q [T, Hq, D] -> [T, Hq, D]."""
    T, Hq, D = q.shape
    G = Hq // n_kv_heads
    scale = scale if scale is not None else D ** -0.5
    out = torch.empty_like(q)
    lens = batch.lens()
    pref = batch.prefix_lens_host if batch.prefix_lens_host is not None else batch.prefix_lens.tolist()
    t0 = 0
    for b, (p, e) in enumerate(zip(pref, lens)):
        if e == 0:
            continue
        L = p + e
        pages = block_table[batch.rows[b].long(), :L].long()
        k = kv_rows_to_float(k_pool[pages], n_kv_heads, D)
        v = kv_rows_to_float(v_pool[pages], n_kv_heads, D)
        qb = q[t0:t0 + e].float().view(e, n_kv_heads, G, D)
        s = torch.einsum("ehgd,lhd->hgel", qb, k) * scale
        causal = torch.arange(L, device=q.device).unsqueeze(0) <= (p + torch.arange(e, device=q.device)).unsqueeze(1)
        s = s.masked_fill(~causal.view(1, 1, e, L), float("-inf"))
        o = torch.einsum("hgel,lhd->ehgd", torch.softmax(s, dim=-1), v)
        out[t0:t0 + e] = o.reshape(e, Hq, D).to(q.dtype)
        t0 += e
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate.float()).mul(up.float()).to(gate.dtype)
