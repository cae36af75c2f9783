"""SMC arithmetic in plain PyTorch: the oracle for every fused kernel and the CPU path.

Covers the sampling identities, the per-cycle importance-weight increment with its
EOS / length gating, ESS, systematic resampling and the logZ estimator.
Behaviour follows the reference (smcsd/core/worker.py:721-778 samplers,
smcsd/core/kernels/fused_write_back.py:24-144 gating,
smcsd/core/kernels/fused_collect.py:156-227 resampling,
smcsd/common/utils.py:324-378 torch helpers); the code is an independent restatement.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

FINISH_NONE = 0
FINISH_LENGTH = 1
FINISH_EOS = 2
MAX_EOS = 8
EMPTY_SLOT = -1

# ----------------------------------------------------------------------------------
# counter-based RNG shared by the CPU path and the CUDA kernels (Philox4x32-10)
# ----------------------------------------------------------------------------------
_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32(counter: Tuple[int, int, int, int], key: Tuple[int, int]) -> Tuple[int, int, int, int]:
    c0, c1, c2, c3 = (x & _MASK for x in counter)
    k0, k1 = (x & _MASK for x in key)
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = (p0 >> 32) & _MASK, p0 & _MASK
        hi1, lo1 = (p1 >> 32) & _MASK, p1 & _MASK
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & _MASK, lo1, (hi0 ^ c3 ^ k1) & _MASK, lo0
        k0 = (k0 + _W0) & _MASK
        k1 = (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def philox_uniform(seed: int, step: int, row: int, stream: int = 0) -> float:
    """Uniform in (0,1) keyed by (seed, stream) and counted by (step, row).

    The CUDA collect kernel evaluates the same function, so a CPU run and a GPU run
    with the same seed draw the same systematic-resampling offsets.
    """
    r = philox4x32((step & _MASK, (step >> 32) & _MASK, row & _MASK, stream & _MASK),
                   (seed & _MASK, (seed >> 32) & _MASK))
    return (r[0] + 0.5) * (1.0 / 4294967296.0)


# ----------------------------------------------------------------------------------
# sampling identities
# ----------------------------------------------------------------------------------
def chosen_logprob(logits: torch.Tensor, tokens: torch.Tensor, temperature: float) -> torch.Tensor:
    """log softmax(logits/T)[tokens] without materialising the full log-softmax."""
    scaled = logits.float() / temperature
    picked = scaled.gather(-1, tokens.long().unsqueeze(-1)).squeeze(-1)
    return picked - torch.logsumexp(scaled, dim=-1)


def gumbel_noise(shape, device, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    u = torch.rand(shape, device=device, generator=generator, dtype=torch.float32)
    u = u.clamp_min(torch.finfo(torch.float32).tiny)
    return -torch.log((-torch.log(u)).clamp_min(torch.finfo(torch.float32).tiny))


def gumbel_sample(logits: torch.Tensor, temperature: float, alpha: float = 1.0,
                  generator: Optional[torch.Generator] = None,
                  noise: Optional[torch.Tensor] = None):
    """Draw from softmax(alpha*logits/T) by Gumbel-max.

    Returns (token, logp, logz): ``logp`` is the noise-free log-probability of the
    token under softmax(alpha*logits/T) and ``logz = lse(alpha*l/T) - alpha*lse(l/T)``,
    which is exactly zero at alpha == 1.  ``temperature <= 0`` means greedy argmax.
    """
    x = logits.float()
    if temperature <= 0.0:
        tok = torch.argmax(x, dim=-1)
        zeros = torch.zeros(tok.shape, dtype=torch.float32, device=x.device)
        return tok, zeros, zeros.clone()
    base = x / temperature
    scaled = base * alpha
    if noise is None:
        noise = gumbel_noise(scaled.shape, scaled.device, generator)
    tok = torch.argmax(scaled + noise, dim=-1)
    lse_scaled = torch.logsumexp(scaled, dim=-1)
    logp = scaled.gather(-1, tok.unsqueeze(-1)).squeeze(-1) - lse_scaled
    if alpha == 1.0:
        logz = torch.zeros_like(logp)
    else:
        logz = lse_scaled - alpha * torch.logsumexp(base, dim=-1)
    return tok, logp, logz


def bonus_logz(logits: torch.Tensor, alpha: float, temperature: float) -> torch.Tensor:
    base = logits.float() / temperature
    return torch.logsumexp(alpha * base, dim=-1) - alpha * torch.logsumexp(base, dim=-1)


# ----------------------------------------------------------------------------------
# weights / ESS / resampling
# ----------------------------------------------------------------------------------
def normalize_log_weights(log_w: torch.Tensor) -> torch.Tensor:
    lw = log_w.double()
    return torch.exp(lw - torch.logsumexp(lw, dim=-1, keepdim=True))


def effective_sample_size(log_w: torch.Tensor) -> torch.Tensor:
    w = normalize_log_weights(log_w)
    return 1.0 / (w * w).sum(dim=-1)


def should_resample(log_w: torch.Tensor, threshold: float) -> torch.Tensor:
    n = log_w.shape[-1]
    if n < 2 or threshold <= 0.0:
        return torch.zeros(log_w.shape[:-1], dtype=torch.bool, device=log_w.device)
    return effective_sample_size(log_w) < threshold * n


def systematic_ancestors(weights: torch.Tensor, u: float) -> torch.Tensor:
    """Ancestor index per offspring for one group: ancestor_k = #{j : cdf_j < (u+k)/N}."""
    n = weights.shape[-1]
    cdf = torch.cumsum(weights.double(), dim=-1)
    cdf = cdf / cdf[-1]
    pos = (u + torch.arange(n, dtype=torch.float64, device=weights.device)) / n
    anc = (cdf.unsqueeze(0) < pos.unsqueeze(1)).sum(dim=1)
    return anc.clamp_max(n - 1)


def resample_plan(weights: torch.Tensor, u: float) -> Tuple[list, list]:
    """(dst, src) particle-index pairs that realise a systematic resample.

    Ancestors that keep at least one offspring stay in place; each particle with no
    offspring becomes the destination of one surplus copy of an ancestor with more
    than one.  Destinations are unique and disjoint from sources, so the copies can
    run in parallel.
    """
    n = weights.shape[-1]
    anc = systematic_ancestors(weights, u)
    counts = torch.bincount(anc, minlength=n).tolist()
    dead = [i for i in range(n) if counts[i] == 0]
    surplus = []
    for i in range(n):
        surplus.extend([i] * max(counts[i] - 1, 0))
    assert len(dead) == len(surplus)
    return dead, surplus


def multinomial_plan(weights: torch.Tensor, generator: Optional[torch.Generator] = None) -> Tuple[list, list]:
    """Multinomial resampling expressed as the same (dst, src) plan."""
    n = weights.shape[-1]
    anc = torch.multinomial(weights.float(), n, replacement=True, generator=generator)
    counts = torch.bincount(anc, minlength=n).tolist()
    dead = [i for i in range(n) if counts[i] == 0]
    surplus = []
    for i in range(n):
        surplus.extend([i] * max(counts[i] - 1, 0))
    return dead, surplus


def logz_increment(interval_log_w: torch.Tensor) -> torch.Tensor:
    """logsumexp(interval weights) - log N per group row."""
    n = interval_log_w.shape[-1]
    return torch.logsumexp(interval_log_w.double(), dim=-1) - math.log(n)


# ----------------------------------------------------------------------------------
# write-back gating (per row), vectorised
# ----------------------------------------------------------------------------------
def write_back_reference(tokens: torch.Tensor, logprob_diff: torch.Tensor,
                         bonus_logz_: Optional[torch.Tensor],
                         token_counts: torch.Tensor, finished: torch.Tensor,
                         max_new_tokens: torch.Tensor, ignore_eos: torch.Tensor,
                         eos_ids: torch.Tensor):
    """Pure function form of the cycle write-back for ``bs`` rows.

    tokens [bs, G] (G = gamma+1: gamma drafts then the bonus), logprob_diff [bs, gamma].
    Returns a dict with new_counts, newly_finished, finish_code, finished_len,
    matched_eos, weight_inc (float64).
    """
    bs, G = tokens.shape
    gamma = G - 1
    dev = tokens.device
    new_counts = token_counts + G
    length_hit = new_counts >= max_new_tokens
    is_eos = (tokens.unsqueeze(-1).long() == eos_ids.unsqueeze(1).long()).logical_and(
        (eos_ids >= 0).unsqueeze(1)).any(-1)
    is_eos = is_eos & (~ignore_eos).unsqueeze(-1)
    eos_hit = is_eos.any(-1)
    idx = torch.arange(G, device=dev).unsqueeze(0).expand(bs, G)
    first_eos = torch.where(is_eos, idx, torch.full_like(idx, G)).min(dim=-1).values
    newly = (~finished) & (length_hit | eos_hit)
    code = torch.where(length_hit, torch.full_like(first_eos, FINISH_LENGTH),
                       torch.full_like(first_eos, FINISH_EOS))
    fin_len = torch.where(length_hit, max_new_tokens.long(), (token_counts + first_eos + 1).long())
    matched = torch.where(eos_hit & ~length_hit,
                          tokens.gather(1, first_eos.clamp_max(G - 1).unsqueeze(1)).squeeze(1),
                          torch.full_like(tokens[:, 0], -1))
    # weight increment
    cutoff = torch.full((bs,), gamma - 1, device=dev, dtype=torch.long)
    eos_new = newly & eos_hit
    cutoff = torch.where(eos_new, torch.minimum(first_eos, cutoff), cutoff)
    cutoff = torch.where(finished, torch.full_like(cutoff, -1), cutoff)
    kidx = torch.arange(gamma, device=dev).unsqueeze(0)
    mask = kidx <= cutoff.unsqueeze(1)
    inc = (logprob_diff.double() * mask).sum(-1)
    if bonus_logz_ is not None:
        eos_in_draft = eos_new & (first_eos < gamma)
        add_bonus = (~finished) & (~eos_in_draft)
        inc = inc + torch.where(add_bonus, bonus_logz_.double(), torch.zeros_like(inc))
    return dict(new_counts=new_counts, newly_finished=newly, finish_code=code, finished_len=fin_len,
                matched_eos=matched, weight_inc=inc, first_eos=first_eos)
