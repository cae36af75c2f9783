"""Messages between the API process and the scheduler processes, and request validation.

The message set mirrors what the reference exchanges over its three sockets
(smcsd/engine.py:20-29: tokenized generate request, batched token output, abort,
profile and RPC requests, and the particle side channel smcsd/core/info.py:38-52);
the rejected request features are those of smcsd/common/utils.py:150-167.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class SamplingParams:
    max_new_tokens: int = 128
    ignore_eos: bool = False
    stop_token_ids: Optional[List[int]] = None
    # accepted for API compatibility; SMC uses the engine-wide draft/target temperatures
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    stop: Optional[Any] = None
    stop_regex: Optional[Any] = None
    n: int = 1

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> "SamplingParams":
        d = dict(d or {})
        known = {k: d.pop(k) for k in list(d) if k in cls.__dataclass_fields__}
        sp = cls(**known)
        sp.extra = d
        return sp

    def normalize(self) -> "SamplingParams":
        if self.max_new_tokens is None or self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        return self


@dataclass
class GenerateRequest:
    rid: str
    input_ids: List[int]
    sampling_params: SamplingParams
    eos_token_ids: List[int] = field(default_factory=list)
    return_logprob: bool = False
    return_hidden_states: bool = False
    return_routed_experts: bool = False
    input_embeds: Any = None
    image_data: Any = None
    grammar: Any = None
    arrival_time: float = 0.0
    priority: Optional[int] = None     # only with priority scheduling switched on (otherwise the request is refused)


@dataclass
class RequestOutput:
    """One (possibly partial) slice of a request's output tokens."""
    rid: str
    output_ids: List[int]
    finished: bool
    finish_reason: Optional[Dict[str, Any]] = None
    prompt_tokens: int = 0
    completion_tokens: int = 0
    aborted: bool = False
    error: Optional[str] = None
    # request time stats in seconds (set on the final slice): time in the queue, arrival to first token
    # (end of prefill), arrival to completion; and the number of decode cycles the group ran
    time_stats: Optional[Dict[str, float]] = None


@dataclass
class ParticleOutput:
    """Side channel with every particle of a finished group (offline engine only)."""
    rid: str
    particle_output_ids: List[List[int]]
    log_Z_hat: float
    log_w_tilde: List[float]
    picked: int = 0


@dataclass
class AbortReq:
    rid: str


@dataclass
class ProfileReq:
    action: str                       # "start" | "stop"
    output_dir: Optional[str] = None
    num_steps: Optional[int] = None
    activities: Optional[List[str]] = None
    with_stack: bool = False
    record_shapes: bool = False
    profile_by_stage: bool = False
    profile_stages: Optional[List[str]] = None


@dataclass
class RpcReq:
    method: str
    kwargs: Dict[str, Any] = field(default_factory=dict)
    req_id: int = 0


@dataclass
class RpcResp:
    req_id: int
    rank: int
    ok: bool
    value: Any = None


@dataclass
class ShutdownReq:
    pass


def validate_request(req: GenerateRequest, max_context: int, gamma: int) -> Optional[str]:
    """Returns an error string for requests SMC cannot serve, else None."""
    sp = req.sampling_params
    if req.image_data is not None:
        return "SMC does not support multimodal inputs"
    if req.input_embeds is not None:
        return "SMC does not support input_embeds"
    if req.grammar is not None:
        return "SMC does not support grammar-constrained decoding"
    if req.return_logprob:
        return "SMC does not support return_logprob"
    if req.return_hidden_states:
        return "SMC does not support return_hidden_states"
    if req.return_routed_experts:
        return "SMC does not support return_routed_experts"
    if sp.stop:
        return "SMC does not support stop strings (use stop_token_ids)"
    if sp.stop_regex:
        return "SMC does not support stop regex"
    if len(req.input_ids) == 0:
        return "empty prompt"
    # a group that hits its length limit can run one more cycle under the overlapped loop before the host sees the
    # finished mask, so two cycles of gamma + 1 tokens of slack are kept inside the block-table row
    if len(req.input_ids) + sp.max_new_tokens + 2 * (gamma + 1) > max_context:
        return (f"prompt ({len(req.input_ids)}) + max_new_tokens ({sp.max_new_tokens}) exceeds "
                f"the context length ({max_context})")
    return None
