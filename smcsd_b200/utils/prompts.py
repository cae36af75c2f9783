"""Synthetic workloads named by the benchmark configs: uniform token ids with log-normal,
uniform-range or fixed prompt lengths (no dataset or tokenizer needed)."""
from __future__ import annotations

import math
from typing import List

import torch


def lognormal_lengths(n: int, median: float = 200.0, sigma: float = 1.0, lo: int = 4, hi: int = 2048,
                      seed: int = 0) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(n, generator=g)
    return [int(min(max(round(math.exp(math.log(median) + sigma * float(v))), lo), hi)) for v in z]


def uniform_lengths(n: int, lo: int = 700, hi: int = 900, seed: int = 0) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


def random_prompts(lengths: List[int], vocab_size: int, seed: int = 0) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed + 1)
    return [torch.randint(0, vocab_size, (L,), generator=g).tolist() for L in lengths]
