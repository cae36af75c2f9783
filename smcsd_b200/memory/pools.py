"""Paged memory for SMC particles: refcounted page allocator, block table, KV pool,
recurrent-state pool and the co-budget rule that sizes them.

The allocator is *device resident*: the free list is a stack in device memory with
its cursor beside it, so pages are popped by the cycle-prologue kernel and pushed
back by the resample kernel inside the captured cycle graph, without a host round
trip.  The host only keeps a conservative lower bound of the free count for
admission.  Semantics (token-granular pages, per-page reference counts shared by
the particles of a group, ``alloc / free / inc_ref / dec_ref_and_free /
copy_block_table``) follow the reference's allocator
(smcsd/mem_cache/allocator.py:18-76); the KV cell sizing follows
smcsd/model_executor/smc_model_runner.py:109-239.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


class PageAllocator:
    """Refcounted allocator of token pages 1..size (page 0 is a scratch page that
    padding rows and exhausted allocations write to)."""

    def __init__(self, size: int, device):
        self.size = int(size)
        self.device = torch.device(device)
        self.refcount = torch.zeros(self.size + 1, dtype=torch.int32, device=self.device)
        # stack of free page ids; free_stack[:free_count] are free
        self.free_stack = torch.arange(self.size, 0, -1, dtype=torch.int32, device=self.device).contiguous()
        self.free_count = torch.full((1,), self.size, dtype=torch.int32, device=self.device)
        # set to 1 by device code when an allocation ran dry
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ---- torch implementations (CPU path, oracle, and rare host-driven events) ----
    def available(self) -> int:
        return int(self.free_count.item())

    def alloc(self, n: int) -> Optional[torch.Tensor]:
        """Pop n pages (refcount set to 1).  Returns None when fewer than n are free."""
        n = int(n)
        cnt = int(self.free_count.item())
        if n > cnt:
            return None
        pages = self.free_stack[cnt - n:cnt].flip(0).clone()
        self.free_count.fill_(cnt - n)
        self.refcount.index_fill_(0, pages.long(), 1)
        return pages

    def free(self, pages: torch.Tensor) -> None:
        """Push pages back unconditionally (refcount forced to 0)."""
        if pages.numel() == 0:
            return
        pages = pages.to(torch.int32).reshape(-1)
        cnt = int(self.free_count.item())
        self.free_stack[cnt:cnt + pages.numel()] = pages
        self.free_count.fill_(cnt + pages.numel())
        self.refcount.index_fill_(0, pages.long(), 0)

    def inc_ref(self, pages: torch.Tensor) -> None:
        if pages.numel() == 0:
            return
        ones = torch.ones(pages.numel(), dtype=torch.int32, device=self.device)
        self.refcount.index_add_(0, pages.long().reshape(-1), ones)

    def dec_ref_and_free(self, pages: torch.Tensor) -> int:
        """Drop one reference from each page; pages that reach zero return to the stack."""
        if pages.numel() == 0:
            return 0
        idx = pages.long().reshape(-1)
        ones = torch.ones(idx.numel(), dtype=torch.int32, device=self.device)
        self.refcount.index_add_(0, idx, -ones)
        uniq = torch.unique(idx)
        dead = uniq[(self.refcount[uniq] <= 0) & (uniq > 0)]
        if dead.numel():
            self.refcount.index_fill_(0, dead, 0)
            cnt = int(self.free_count.item())
            self.free_stack[cnt:cnt + dead.numel()] = dead.to(torch.int32)
            self.free_count.fill_(cnt + dead.numel())
        return int(dead.numel())

    def pages_in_use(self) -> int:
        return self.size - self.available()

    def check_conservation(self) -> None:
        """free pages and referenced pages partition 1..size; used by the tests after every scenario."""
        cnt = self.available()
        free = self.free_stack[:cnt].long()
        assert torch.unique(free).numel() == cnt, "duplicate page on the free stack"
        assert int((self.refcount[free] != 0).sum()) == 0, "free page with a live reference"
        live = int((self.refcount[1:] > 0).sum())
        assert live + cnt == self.size, f"leak: {live} live + {cnt} free != {self.size}"
        assert int((self.refcount < 0).sum()) == 0, "negative refcount"


class BlockTable:
    """Row-per-sequence table of page ids: ``table[row, pos]`` is the page of token ``pos``.

    Particle slot ``s`` owns row ``s``; rows ``[n_slots, n_slots + n_parent_rows)`` serve
    parents during prefill, so no second indirection is needed on the device.
    """

    def __init__(self, n_slots: int, n_parent_rows: int, max_context: int, device):
        self.n_slots = n_slots
        self.n_parent_rows = n_parent_rows
        self.max_context = int(max_context)
        self.table = torch.zeros(n_slots + n_parent_rows, self.max_context, dtype=torch.int32, device=device)
        self._free_parent_rows: List[int] = list(range(n_slots + n_parent_rows - 1, n_slots - 1, -1))

    def alloc_parent_row(self) -> Optional[int]:
        return self._free_parent_rows.pop() if self._free_parent_rows else None

    def free_parent_row(self, row: int) -> None:
        self._free_parent_rows.append(row)

    def copy_row(self, src: int, dst_rows: torch.Tensor, length: int, alloc: PageAllocator) -> None:
        """Fan a parent's first ``length`` entries out to ``dst_rows`` and take one reference per copy."""
        pages = self.table[src, :length]
        self.table[dst_rows.long(), :length] = pages.unsqueeze(0)
        n = int(dst_rows.numel())
        alloc.refcount.index_add_(0, pages.long(), torch.full((length,), n, dtype=torch.int32,
                                                              device=alloc.device))


@dataclass
class KVSpec:
    n_layers: int        # layers that own a KV cache (attention layers only for hybrids)
    n_kv_heads: int
    head_dim: int
    dtype: torch.dtype = torch.bfloat16
    fp8: bool = False    # e4m3 cache: a page row holds Hkv * D value bytes + one fp32 scale per kv head (padded to 16)

    @property
    def row_width(self) -> int:
        """Elements of one page row of the K (or V) tensor."""
        if self.fp8:
            return (self.n_kv_heads * self.head_dim + self.n_kv_heads * 4 + 15) // 16 * 16
        return self.n_kv_heads * self.head_dim

    @property
    def store_dtype(self) -> torch.dtype:
        return torch.uint8 if self.fp8 else self.dtype

    @property
    def cell_bytes(self) -> int:
        return 2 * self.n_layers * self.row_width * torch.empty((), dtype=self.store_dtype).element_size()


def kv_rows_to_float(rows: torch.Tensor, n_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Page rows of a K or V pool -> fp32 [L, Hkv, D]; e4m3 rows (uint8) are dequantised with their per-head scales."""
    L = rows.shape[0]
    if rows.dtype != torch.uint8:
        return rows.view(L, n_kv_heads, head_dim).float()
    nv = n_kv_heads * head_dim
    vals = rows[:, :nv].contiguous().view(torch.float8_e4m3fn).float().view(L, n_kv_heads, head_dim)
    scales = rows[:, nv:nv + 4 * n_kv_heads].contiguous().view(torch.float32).view(L, n_kv_heads, 1)
    return vals * scales


def kv_rows_from_float(x: torch.Tensor, row_width: int) -> torch.Tensor:
    """fp32 / bf16 [T, Hkv, D] -> e4m3 page rows [T, row_width] (uint8) with per-(token, head) scales max|x| / 448."""
    T, H, D = x.shape
    xf = x.float()
    scale = xf.abs().amax(dim=-1).clamp_(min=1e-12) / 448.0                      # [T, H]
    q = (xf / scale.unsqueeze(-1)).to(torch.float8_e4m3fn).view(torch.uint8).reshape(T, H * D)
    out = torch.zeros(T, row_width, dtype=torch.uint8, device=x.device)
    out[:, :H * D] = q
    out[:, H * D:H * D + 4 * H] = scale.contiguous().view(torch.uint8).reshape(T, 4 * H)
    return out


class KVPool:
    """K and V as ``[layer, page, row]``; one row per token page (bf16 values, or the e4m3 layout of ``KVSpec``)."""

    def __init__(self, spec: KVSpec, n_pages: int, device):
        self.spec = spec
        self.n_pages = n_pages
        self.k = torch.zeros(spec.n_layers, n_pages + 1, spec.row_width, dtype=spec.store_dtype, device=device)
        self.v = torch.zeros(spec.n_layers, n_pages + 1, spec.row_width, dtype=spec.store_dtype, device=device)

    def write(self, layer: int, locs: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        if self.spec.fp8:
            H, D = self.spec.n_kv_heads, self.spec.head_dim
            self.k[layer].index_copy_(0, locs.long(), kv_rows_from_float(k.reshape(k.shape[0], H, D), self.spec.row_width))
            self.v[layer].index_copy_(0, locs.long(), kv_rows_from_float(v.reshape(v.shape[0], H, D), self.spec.row_width))
            return
        self.k[layer].index_copy_(0, locs.long(), k.reshape(k.shape[0], -1).to(self.k.dtype))
        self.v[layer].index_copy_(0, locs.long(), v.reshape(v.shape[0], -1).to(self.v.dtype))


@dataclass
class StateSpec:
    """Recurrent (Gated-DeltaNet) state per sequence row."""
    n_layers: int
    conv_dim: int
    conv_width: int
    n_heads: int
    head_k_dim: int
    head_v_dim: int
    conv_dtype: torch.dtype = torch.bfloat16
    state_dtype: torch.dtype = torch.float32

    @property
    def row_bytes(self) -> int:
        conv = self.conv_dim * (self.conv_width - 1) * torch.empty((), dtype=self.conv_dtype).element_size()
        temp = self.n_heads * self.head_k_dim * self.head_v_dim * torch.empty((), dtype=self.state_dtype).element_size()
        return self.n_layers * (conv + temp)


class StatePool:
    """Conv window and temporal state per (layer, row).  Multi-token passes advance the state in place (SMC accepts
    every token), so no per-position copies are kept."""

    def __init__(self, spec: StateSpec, n_rows: int, device):
        self.spec = spec
        self.n_rows = n_rows
        self.conv = torch.zeros(spec.n_layers, n_rows, spec.conv_dim, spec.conv_width - 1,
                                dtype=spec.conv_dtype, device=device)
        self.temporal = torch.zeros(spec.n_layers, n_rows, spec.n_heads, spec.head_k_dim, spec.head_v_dim,
                                    dtype=spec.state_dtype, device=device)

    def copy_rows(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        """dst[i] <- src[i] for every layer (fan-out at materialize, resample copies)."""
        if dst.numel() == 0:
            return
        d, s = dst.long(), src.long()
        self.conv[:, d] = self.conv[:, s]
        self.temporal[:, d] = self.temporal[:, s]

    def clear_rows(self, rows: torch.Tensor) -> None:
        if rows.numel() == 0:
            return
        r = rows.long()
        self.conv[:, r] = 0
        self.temporal[:, r] = 0


def cobudget_pages(available_bytes: int, target_cell: int, draft_cell: int,
                   draft_weight_bytes: int = 0, state_bytes: int = 0) -> int:
    """Pages that fit when target and draft KV share one page id space:
    (available - draft weights - recurrent state) // (target cell + draft cell)."""
    usable = available_bytes - draft_weight_bytes - state_bytes
    return max(int(usable // max(target_cell + draft_cell, 1)), 0)
