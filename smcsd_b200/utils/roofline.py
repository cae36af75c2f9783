"""Bandwidth floor of one decode cycle: the bytes a cycle cannot avoid reading from HBM, over the measured copy
bandwidth of the GPU.  The reported fraction is floor / measured time ("of measured" when the denominators come from
the measured-peaks record of the machine, "of fallback" otherwise)."""
from __future__ import annotations

import json
import os
from typing import Optional, Tuple

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks(path: Optional[str] = None) -> Tuple[float, float, str]:
    """(HBM copy GB/s, bf16 TFLOP/s, "measured" | "fallback").  The record is written beside the package's parent
    folder by whoever measured the machine; without it the stated fallback figures are used."""
    if path is None:
        here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            j = json.load(f)
        return float(j.get("hbm_gbs", FALLBACK_HBM_GBS)), float(j.get("bf16_tflops", FALLBACK_BF16_TFLOPS)), "measured"
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


def dense_weight_bytes(cfg, bytes_per_weight: float = 2.0) -> Optional[int]:
    """Bytes of the matrices a forward pass of a dense Llama-style model streams: the four projections of every
    layer and the output head (the input embedding is a row gather, not a stream; a tied head is counted once, as
    the head).  None for other architectures."""
    if getattr(cfg, "arch", "llama") != "llama":
        return None
    H, D = cfg.hidden_size, cfg.head_dim
    per_layer = (cfg.n_heads + 2 * cfg.n_kv_heads) * D * H + H * cfg.n_heads * D + 3 * cfg.ffn_size * H
    return int((per_layer * cfg.n_layers + cfg.vocab_size * H) * bytes_per_weight)


def kv_bytes_per_token(cfg, bytes_per_value: float = 2.0) -> int:
    return int(2 * cfg.n_layers * cfg.n_kv_heads * cfg.head_dim * bytes_per_value)


def decode_cycle_floor(target_cfg, draft_cfg, gamma: int, defer_bonus: bool = True, rows: int = 8, context: int = 0,
                       shared_prompt: int = 0, hbm_gbs: Optional[float] = None) -> Optional[dict]:
    """Floor of one SMC decode cycle on one GPU.  The target's weights are read once (one verify pass over gamma + 1
    tokens per particle), the draft's once per draft forward (gamma with the deferred bonus, gamma + 1 without).
    Cached keys and values are read once per pass: every particle row's own ``context - shared_prompt`` tokens plus the
    shared prompt once per request group (``rows`` particle rows are taken as one group)."""
    wt, wd = dense_weight_bytes(target_cfg), dense_weight_bytes(draft_cfg)
    if wt is None or wd is None:
        return None
    src = "given"
    if hbm_gbs is None:
        hbm_gbs, _, src = measured_peaks()
    n_draft = gamma if defer_bonus else gamma + 1
    own = max(0, context - shared_prompt)
    kv_tokens = rows * own + shared_prompt
    kv = kv_tokens * (kv_bytes_per_token(target_cfg) + n_draft * kv_bytes_per_token(draft_cfg))
    total = wt + n_draft * wd + kv
    return {"weight_bytes": wt + n_draft * wd, "kv_bytes": int(kv), "bytes": int(total),
            "hbm_gbs": hbm_gbs, "peaks": src, "floor_ms": total / (hbm_gbs * 1e9) * 1e3}
