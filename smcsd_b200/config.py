"""Engine configuration: one dataclass carrying every SMC and serving knob.

Precedence of the feature switches is ``SMC_*`` environment variable (kill
switch) > constructor keyword > default, the same three tiers the reference
documents (reference: docs/smc/performance.md:145-150, smcsd/core/worker.py:106-113,
smcsd/core/scheduler.py:263-274).  Knob inventory follows the reference's
constructor and CLI (smcsd/engine.py:60-82, smcsd/http_server.py:140-212).
"""
from __future__ import annotations

import argparse
import dataclasses
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

_TRUE = {"1", "true", "yes", "on"}
_FALSE = {"0", "false", "no", "off"}


def env_flag(name: str, kwarg: Optional[bool], default: bool) -> bool:
    """Resolve a boolean switch: env var beats the keyword, which beats the default."""
    raw = os.environ.get(name)
    if raw is not None:
        low = raw.strip().lower()
        if low in _TRUE:
            return True
        if low in _FALSE:
            return False
    if kwarg is not None:
        return bool(kwarg)
    return default


def env_int(name: str, kwarg: Optional[int], default: int) -> int:
    raw = os.environ.get(name)
    if raw is not None:
        try:
            return int(raw)
        except ValueError:
            pass
    return int(kwarg) if kwarg is not None else default


@dataclass
class EngineArgs:
    # ---- models -------------------------------------------------------------
    model_path: Any = None              # HF directory, or a ModelConfig for random-init
    draft_model_path: Any = None
    dtype: str = "bfloat16"
    device: str = "auto"                # "cuda", "cpu" or "auto"
    backend: str = "auto"               # "native" (sm_100a kernels) | "torch" (oracle / CPU / baseline)
    random_seed: int = 0
    trust_remote_code: bool = False
    context_length: Optional[int] = None
    skip_tokenizer_init: bool = False
    # ---- SMC ----------------------------------------------------------------
    n_particles: int = 4
    gamma: int = 4
    draft_temperature: float = 0.7
    target_temperature: float = 1.0
    power_alpha: float = 1.0
    resample_threshold: float = 0.5
    resample_method: str = "systematic"
    defer_bonus: Optional[bool] = None
    cycle_graph: Optional[bool] = None
    enable_overlap: Optional[bool] = None
    fused_sampling: Optional[bool] = None
    fused_write_back: Optional[bool] = None
    fast_verify: Optional[bool] = None
    draft_phase_graph: Optional[bool] = None
    graph_max_bs: Optional[int] = None
    graph_max_context: Optional[int] = None
    emit_particle_output: bool = True
    # ---- serving ------------------------------------------------------------
    max_running_requests: int = 8       # user-facing concurrent groups
    max_queued_requests: Optional[int] = None
    enable_priority_scheduling: bool = False          # requests may carry a priority; the waiting queue is ordered by it
    schedule_low_priority_values_first: bool = False  # smaller numbers are served first (default: larger first)
    mem_fraction_static: float = 0.6
    max_total_tokens: Optional[int] = None
    kv_cache_dtype: str = "auto"
    quantization: Optional[str] = None
    disable_cuda_graph: bool = False
    cuda_graph_max_bs: Optional[int] = None
    attention_num_kv_splits: int = 16   # upper bound of the key-range splits the attention planner may choose
    log_level: str = "error"
    # ---- parallelism --------------------------------------------------------
    tp_size: int = 1                    # tensor-parallel ranks for the target
    dp_size: int = 1                    # independent replicas
    pp_size: int = 1                    # particle-parallel ranks (particles of one group sharded)
    base_gpu_id: int = 0
    replicate_draft: bool = True
    dist_init_addr: str = "127.0.0.1"
    nccl_port: Optional[int] = None
    in_process: Optional[bool] = None   # run the scheduler in the caller's process (no ZMQ hop)
    extra: Dict[str, Any] = field(default_factory=dict)

    # resolved switches (filled by ``finalize``)
    def finalize(self) -> "EngineArgs":
        if self.n_particles < 1:
            raise ValueError("n_particles must be >= 1")
        if self.gamma < 1:
            raise ValueError("gamma must be >= 1")
        if self.power_alpha <= 0:
            raise ValueError("power_alpha must be > 0")
        if self.resample_method not in ("systematic", "multinomial"):
            raise ValueError(f"unknown resample_method {self.resample_method!r}")
        if self.quantization in ("", "none"):
            self.quantization = None
        if self.quantization not in (None, "fp8"):
            raise ValueError(f"quantization={self.quantization!r} is not supported: weights are served in bf16 or, with "
                             "quantization='fp8', as e4m3 with per-row scales (dense models, kernel backend)")
        if self.kv_cache_dtype in ("fp8", "fp8_e4m3"):
            self.kv_cache_dtype = "fp8_e4m3"
        if self.kv_cache_dtype not in ("auto", "bf16", "bfloat16", "fp8_e4m3"):
            raise ValueError(f"kv_cache_dtype={self.kv_cache_dtype!r} is not supported: the KV cache holds bf16 rows or, "
                             "with kv_cache_dtype='fp8_e4m3', e4m3 rows with one scale per token and kv head")
        self.target_temperature = max(float(self.target_temperature), 1e-5)
        self.defer_bonus = env_flag("SMC_DEFER_BONUS", self.defer_bonus, True)
        self.cycle_graph = env_flag("SMC_CYCLE_GRAPH", self.cycle_graph, True)
        self.enable_overlap = env_flag("SMC_ENABLE_OVERLAP", self.enable_overlap, True)
        self.fused_sampling = env_flag("SMC_FUSED_SAMPLING", self.fused_sampling, True)
        self.fused_write_back = env_flag("SMC_FUSED_WRITE_BACK", self.fused_write_back, True)
        self.fast_verify = env_flag("SMC_FAST_VERIFY", self.fast_verify, True)
        self.draft_phase_graph = env_flag("SMC_DRAFT_PHASE_GRAPH", self.draft_phase_graph, False)
        self.graph_max_bs = env_int("SMC_DRAFT_GRAPH_MAX_BS", self.graph_max_bs, 64)
        if self.cuda_graph_max_bs:          # the sweeps size the capture cap as batch x particles
            self.graph_max_bs = max(self.graph_max_bs, int(self.cuda_graph_max_bs))
        # the reference caps graph replay at 8192 tokens because of its index buffers; the cycle graph here has no
        # per-context buffers, so the default cap is far out and the knob only exists to force the eager path
        self.graph_max_context = env_int("SMC_DRAFT_GRAPH_MAX_CONTEXT", self.graph_max_context, 131072)
        if self.disable_cuda_graph or self.draft_temperature <= 0.0:
            # greedy proposals take the eager path, like the reference (worker.py:299-300)
            self.cycle_graph = False
            self.draft_phase_graph = False
        return self

    @property
    def max_slots(self) -> int:
        return self.max_running_requests * self.n_particles

    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        for k in ("model_path", "draft_model_path"):
            if not isinstance(d[k], (str, type(None))):
                d[k] = repr(d[k])
        return d

    # ---- CLI ----------------------------------------------------------------
    @staticmethod
    def add_cli_args(p: argparse.ArgumentParser) -> None:
        p.add_argument("--model", "--model-path", dest="model_path", required=True)
        p.add_argument("--draft-model", "--speculative-draft-model-path", dest="draft_model_path", required=True)
        p.add_argument("-N", "--smc-n-particles", dest="n_particles", type=int, default=4)
        p.add_argument("-g", "--smc-gamma", dest="gamma", type=int, default=4)
        p.add_argument("--smc-draft-temperature", dest="draft_temperature", type=float, default=0.7)
        p.add_argument("--smc-target-temperature", dest="target_temperature", type=float, default=1.0)
        p.add_argument("--smc-power-alpha", dest="power_alpha", type=float, default=1.0)
        p.add_argument("--smc-resample-threshold", dest="resample_threshold", type=float, default=0.5)
        p.add_argument("--smc-resample-method", dest="resample_method", default="systematic",
                       choices=["systematic", "multinomial"])
        p.add_argument("--no-defer-bonus", dest="defer_bonus", action="store_false", default=None)
        p.add_argument("--no-cycle-graph", dest="cycle_graph", action="store_false", default=None)
        p.add_argument("--no-overlap", dest="enable_overlap", action="store_false", default=None)
        p.add_argument("--tp-size", type=int, default=1)
        p.add_argument("--dp-size", type=int, default=1)
        p.add_argument("--pp-size", "--particle-parallel-size", dest="pp_size", type=int, default=1)
        p.add_argument("--base-gpu-id", type=int, default=0)
        p.add_argument("--mem-fraction-static", type=float, default=0.4)
        p.add_argument("--max-running-requests", type=int, default=8)
        p.add_argument("--max-queued-requests", type=int, default=None)
        p.add_argument("--enable-priority-scheduling", action="store_true")
        p.add_argument("--schedule-low-priority-values-first", action="store_true")
        p.add_argument("--max-total-tokens", type=int, default=None)
        p.add_argument("--context-length", type=int, default=None)
        p.add_argument("--cuda-graph-max-bs", type=int, default=None)
        p.add_argument("--disable-cuda-graph", action="store_true")
        p.add_argument("--attention-backend", default="native", help="accepted for CLI parity; one native backend exists")
        p.add_argument("--kv-cache-dtype", default="auto")
        p.add_argument("--quantization", default=None)
        p.add_argument("--dtype", default="bfloat16")
        p.add_argument("--device", default="auto")
        p.add_argument("--backend", default="auto", choices=["auto", "native", "torch"])
        p.add_argument("--random-seed", type=int, default=0)
        p.add_argument("--trust-remote-code", action="store_true")
        p.add_argument("--log-level", default="info")

    @classmethod
    def from_cli_args(cls, ns: argparse.Namespace) -> "EngineArgs":
        names = {f.name for f in dataclasses.fields(cls)}
        kw = {k: v for k, v in vars(ns).items() if k in names}
        return cls(**kw)
