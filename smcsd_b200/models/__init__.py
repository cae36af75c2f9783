"""Model families: dense Llama-style decoders and Qwen3.5-style Gated-DeltaNet hybrids."""
from __future__ import annotations

import os

import torch

from .config import ModelConfig, preset, resolve_config


def build_model(spec, dtype=torch.bfloat16, device="cpu", tp_rank: int = 0, tp_size: int = 1, seed: int = 0,
                max_positions=None):
    """Build a model from a HF directory (weights loaded) or a config / preset (random init)."""
    cfg = resolve_config(spec)
    if cfg.arch == "hybrid_gdn":
        from .hybrid_gdn import HybridGDNModel as Cls
    else:
        from .llama import LlamaModel as Cls
    m = Cls(cfg, dtype=dtype, device=device, tp_rank=tp_rank, tp_size=tp_size, max_positions=max_positions)
    if isinstance(spec, str) and os.path.isdir(spec):
        m.load_hf(spec)
    else:
        m.init_random(seed)
    return m


__all__ = ["ModelConfig", "preset", "resolve_config", "build_model"]
