"""Architecture descriptions: parsed from a HF ``config.json`` or built from presets.

Two families are served, the ones the reference runs: dense Llama-style decoders and
Qwen3.5-style hybrids that interleave Gated-DeltaNet layers with gated full attention
(reference: README.md model list; parameter names checked against the HF
implementation, transformers/models/qwen3_5/modeling_qwen3_5.py).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class ModelConfig:
    arch: str = "llama"                  # "llama" | "hybrid_gdn"
    vocab_size: int = 32000
    hidden_size: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn_size: int = 14336
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    max_position: int = 8192
    tie_embeddings: bool = False
    logit_softcap: float = 0.0
    eos_token_ids: List[int] = field(default_factory=list)
    # ---- hybrid (Gated DeltaNet) -------------------------------------------
    layer_types: Optional[List[str]] = None       # "linear_attention" | "full_attention"
    gdn_n_k_heads: int = 16
    gdn_n_v_heads: int = 16
    gdn_head_k_dim: int = 128
    gdn_head_v_dim: int = 128
    gdn_conv_width: int = 4
    partial_rotary: float = 1.0
    attn_output_gate: bool = False
    qk_norm: bool = False
    norm_plus_one: bool = False                    # RMSNorm weight stored as (w - 1)
    name: str = ""

    # ---- derived -------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary)

    def layer_type(self, i: int) -> str:
        if self.layer_types is None:
            return "full_attention"
        return self.layer_types[i]

    @property
    def attn_layers(self) -> List[int]:
        return [i for i in range(self.n_layers) if self.layer_type(i) == "full_attention"]

    @property
    def gdn_layers(self) -> List[int]:
        return [i for i in range(self.n_layers) if self.layer_type(i) == "linear_attention"]

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_n_k_heads * self.gdn_head_k_dim + self.gdn_n_v_heads * self.gdn_head_v_dim

    def param_count(self) -> int:
        d, f = self.hidden_size, self.ffn_size
        n = self.vocab_size * d * (1 if self.tie_embeddings else 2) + d
        for i in range(self.n_layers):
            n += 3 * d * f + 2 * d
            if self.layer_type(i) == "full_attention":
                qmul = 2 if self.attn_output_gate else 1
                n += d * (self.q_size * qmul + 2 * self.kv_size) + self.q_size * d
            else:
                kd = self.gdn_n_k_heads * self.gdn_head_k_dim
                vd = self.gdn_n_v_heads * self.gdn_head_v_dim
                n += d * (2 * kd + vd) + d * vd + 2 * d * self.gdn_n_v_heads + vd * d
        return n

    # ---- construction ----------------------------------------------------------
    @classmethod
    def from_hf_dict(cls, c: Dict[str, Any]) -> "ModelConfig":
        if "text_config" in c and isinstance(c["text_config"], dict):
            merged = dict(c["text_config"])
            merged.setdefault("architectures", c.get("architectures"))
            c = merged
        archs = c.get("architectures") or []
        mt = (c.get("model_type") or "").lower()
        is_hybrid = "layer_types" in c and any(t == "linear_attention" for t in c["layer_types"])
        is_hybrid = is_hybrid or "qwen3_5" in mt or "qwen3_next" in mt or any("Qwen3_5" in a or "Qwen3Next" in a for a in archs)
        n_heads = c["num_attention_heads"]
        head_dim = c.get("head_dim") or c["hidden_size"] // n_heads
        eos = c.get("eos_token_id")
        eos_ids = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        rope_params = c.get("rope_parameters") or {}
        rope_theta = c.get("rope_theta", rope_params.get("rope_theta", 10000.0))
        rope_scaling = c.get("rope_scaling")
        if rope_scaling is None and rope_params.get("rope_type", "default") not in ("default", None):
            rope_scaling = rope_params
        cfg = cls(
            arch="hybrid_gdn" if is_hybrid else "llama",
            vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], n_layers=c["num_hidden_layers"],
            n_heads=n_heads, n_kv_heads=c.get("num_key_value_heads", n_heads), head_dim=head_dim,
            ffn_size=c["intermediate_size"], rms_eps=c.get("rms_norm_eps", 1e-5), rope_theta=rope_theta,
            rope_scaling=rope_scaling, max_position=c.get("max_position_embeddings", 8192),
            tie_embeddings=bool(c.get("tie_word_embeddings", False)),
            logit_softcap=float(c.get("final_logit_softcapping") or 0.0), eos_token_ids=eos_ids,
            name=c.get("_name_or_path", ""))
        if is_hybrid:
            lt = c.get("layer_types")
            if lt is None:
                interval = c.get("full_attention_interval", 4)
                lt = ["full_attention" if (i + 1) % interval == 0 else "linear_attention"
                      for i in range(cfg.n_layers)]
            cfg.layer_types = list(lt)
            cfg.gdn_n_k_heads = c.get("linear_num_key_heads", 16)
            cfg.gdn_n_v_heads = c.get("linear_num_value_heads", 16)
            cfg.gdn_head_k_dim = c.get("linear_key_head_dim", 128)
            cfg.gdn_head_v_dim = c.get("linear_value_head_dim", 128)
            cfg.gdn_conv_width = c.get("linear_conv_kernel_dim", 4)
            cfg.partial_rotary = float(c.get("partial_rotary_factor", rope_params.get("partial_rotary_factor", 0.25)))
            cfg.attn_output_gate = bool(c.get("attn_output_gate", True))
            cfg.qk_norm = True
            cfg.norm_plus_one = True
        return cfg

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            cfg = cls.from_hf_dict(json.load(f))
        gen = os.path.join(path, "generation_config.json")
        if os.path.exists(gen):
            with open(gen) as f:
                g = json.load(f)
            eos = g.get("eos_token_id")
            if eos is not None:
                ids = [eos] if isinstance(eos, int) else list(eos)
                cfg.eos_token_ids = sorted(set(cfg.eos_token_ids) | set(ids))
        cfg.name = cfg.name or os.path.basename(os.path.normpath(path))
        return cfg


_LLAMA3_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                   "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}


def preset(name: str) -> ModelConfig:
    """Random-init architectures named by the benchmark configs."""
    n = name.lower()
    if n in ("llama-3.1-8b", "llama8b", "8b"):
        return ModelConfig(arch="llama", vocab_size=128256, hidden_size=4096, n_layers=32, n_heads=32,
                           n_kv_heads=8, head_dim=128, ffn_size=14336, rope_theta=500000.0,
                           rope_scaling=dict(_LLAMA3_SCALING), max_position=131072, name="llama-3.1-8b")
    if n in ("llama-3.2-1b", "llama1b", "1b"):
        sc = dict(_LLAMA3_SCALING, factor=32.0)
        return ModelConfig(arch="llama", vocab_size=128256, hidden_size=2048, n_layers=16, n_heads=32,
                           n_kv_heads=8, head_dim=64, ffn_size=8192, rope_theta=500000.0, rope_scaling=sc,
                           max_position=131072, tie_embeddings=True, name="llama-3.2-1b")
    if n in ("llama-3.1-70b", "70b"):
        return ModelConfig(arch="llama", vocab_size=128256, hidden_size=8192, n_layers=80, n_heads=64,
                           n_kv_heads=8, head_dim=128, ffn_size=28672, rope_theta=500000.0,
                           rope_scaling=dict(_LLAMA3_SCALING), max_position=131072, name="llama-3.1-70b")
    if n in ("tiny-target", "tiny"):
        return ModelConfig(arch="llama", vocab_size=4096, hidden_size=256, n_layers=4, n_heads=4, n_kv_heads=2,
                           head_dim=64, ffn_size=688, rope_theta=10000.0, max_position=2048, name="tiny-target")
    if n in ("tiny-draft",):
        return ModelConfig(arch="llama", vocab_size=4096, hidden_size=128, n_layers=1, n_heads=2, n_kv_heads=1,
                           head_dim=64, ffn_size=344, rope_theta=10000.0, max_position=2048, name="tiny-draft")
    if n in ("hybrid-gdn-target", "qwen3.5-hybrid"):
        lt = ["full_attention" if (i + 1) % 4 == 0 else "linear_attention" for i in range(48)]
        return ModelConfig(arch="hybrid_gdn", vocab_size=151936, hidden_size=2048, n_layers=48, n_heads=16,
                           n_kv_heads=2, head_dim=256, ffn_size=6144, rope_theta=10000000.0, max_position=32768,
                           layer_types=lt, gdn_n_k_heads=16, gdn_n_v_heads=16, gdn_head_k_dim=128,
                           gdn_head_v_dim=128, gdn_conv_width=4, partial_rotary=0.25, attn_output_gate=True,
                           qk_norm=True, norm_plus_one=True, rms_eps=1e-6, name="hybrid-gdn-target")
    if n in ("hybrid-gdn-draft", "dense-draft-1024"):
        return ModelConfig(arch="llama", vocab_size=151936, hidden_size=1024, n_layers=12, n_heads=16,
                           n_kv_heads=8, head_dim=64, ffn_size=3072, rope_theta=1000000.0, max_position=32768,
                           tie_embeddings=True, rms_eps=1e-6, name="hybrid-gdn-draft")
    if n in ("tiny-hybrid",):
        lt = ["linear_attention", "linear_attention", "linear_attention", "full_attention"]
        return ModelConfig(arch="hybrid_gdn", vocab_size=4096, hidden_size=128, n_layers=4, n_heads=4,
                           n_kv_heads=2, head_dim=64, ffn_size=256, rope_theta=10000.0, max_position=2048,
                           layer_types=lt, gdn_n_k_heads=2, gdn_n_v_heads=4, gdn_head_k_dim=32,
                           gdn_head_v_dim=32, gdn_conv_width=4, partial_rotary=0.25, attn_output_gate=True,
                           qk_norm=True, norm_plus_one=True, rms_eps=1e-6, name="tiny-hybrid")
    raise KeyError(f"unknown preset {name!r}")


def resolve_config(spec) -> ModelConfig:
    if isinstance(spec, ModelConfig):
        return spec
    if isinstance(spec, str) and spec.startswith("preset:"):
        return preset(spec[len("preset:"):])
    if isinstance(spec, str) and os.path.isdir(spec):
        return ModelConfig.from_pretrained(spec)
    if isinstance(spec, str):
        return preset(spec)
    raise TypeError(f"cannot resolve a model config from {spec!r}")
