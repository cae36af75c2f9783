// Per-row partial result of one slice of the vocabulary, shared by the sampling kernels: running
// log-sum-exp of the scaled and of the base logits and the best Gumbel-perturbed candidate.
#pragma once
#include "common.cuh"

namespace smc {

struct RowPartial {
  float max_s, sum_s;      // running max / sum of exp for scaled = alpha * x / T
  float max_b, sum_b;      // same for base = x / T
  float best, best_scaled; // best perturbed score and its unperturbed scaled value
  int best_idx;
  int pad;
};
static_assert(sizeof(RowPartial) == 32, "partials are exchanged as two 16-byte words");

__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  const float M = fmaxf(m, m2);
  if (M == -INFINITY) { m = M; s = 0.f; return; }
  s = s * __expf(m - M) + s2 * __expf(m2 - M);
  m = M;
}

// Sampling / scoring parameters of a fused lm_head epilogue.
struct SampleArgs {
  float inv_temp, alpha, softcap;
  int V;                          // vocabulary size (weight rows past it are padding)
  int rows, call_id;              // logit rows; call id mixed into the noise counter
  const int* tokens_in;           // per row: >= 0 score that token, < 0 sample (null: every row samples)
  unsigned long long seed;
  const long long* cycle_counter;
};

__device__ __forceinline__ RowPartial row_partial_neutral() {
  return RowPartial{-INFINITY, 0.f, -INFINITY, 0.f, -INFINITY, 0.f, 0, __float_as_int(-INFINITY)};
}

// One chunk of 16 logit rows x 128 vocabulary entries of a weight slab, reduced to per-row partials.
// tr[j * 129 + i] holds the (already normalised) logit of vocabulary entry row0 + i for logit row m0 + c0 + j; the
// 128 calling threads (t = 0..127) have synchronised after writing it.  Eight threads share a row (16 entries each)
// and merge through shuffles inside their group of eight lanes; the group's first lane folds the result into
// rp[c0 + j] (shared memory, touched by that one thread only).  The noise is the Philox stream of the stand-alone
// sampler, (entry / 4, row, call id, cycle counter), so both produce the same draws from the same logits.  The chosen
// token's logit of a scored row is carried in the partial's last field.
__device__ __forceinline__ void lm_reduce_chunk(const SampleArgs& a, const float* tr, int row0, int c0, int m0, int t,
                                                RowPartial* rp) {
  const int lane = t & 31;
  const int col = t >> 3, sub = t & 7, m = m0 + c0 + col;
  const unsigned int gmask = 0xFFu << (lane & 24);
  if (m >= a.rows) return;                 // whole groups of eight lanes leave together
  const int given = a.tokens_in != nullptr ? a.tokens_in[m] : -1;
  const bool sampling = given < 0;
  const Philox rng(a.seed);
  const long long cyc = *a.cycle_counter;
  const uint32_t ctr_lo = (uint32_t)cyc, ctr_hi = (uint32_t)(cyc >> 32);
  float max_s = -INFINITY, sum_s = 0.f, max_b = -INFINITY, sum_b = 0.f, best = -INFINITY, best_scaled = 0.f;
  float given_logit = -INFINITY;
  const int nb = row0 + sub * 16;
  int best_idx = nb < a.V ? nb : 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t rnd[4] = {0u, 0u, 0u, 0u};
    const int c4 = nb + q * 4;
    if (sampling && c4 < a.V) rng.run((uint32_t)(c4 >> 2), (uint32_t)m, (uint32_t)a.call_id ^ (ctr_hi << 8), ctr_lo, rnd);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = c4 + i;
      if (c >= a.V) continue;
      float x = tr[col * 129 + sub * 16 + q * 4 + i];
      if (a.softcap > 0.f) x = tanhf(x / a.softcap) * a.softcap;
      const float b = x * a.inv_temp, sc = b * a.alpha;
      if (sc > max_s) { sum_s = sum_s * __expf(max_s - sc) + 1.f; max_s = sc; } else { sum_s += __expf(sc - max_s); }
      if (a.alpha != 1.f) {
        if (b > max_b) { sum_b = sum_b * __expf(max_b - b) + 1.f; max_b = b; } else { sum_b += __expf(b - max_b); }
      }
      if (sampling) {
        const float u = u32_to_unit(rnd[i]);
        const float pert = sc + (-__logf(-__logf(u)));
        if (pert > best) { best = pert; best_scaled = sc; best_idx = c; }
      } else if (c == given) {
        given_logit = x;
      }
    }
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    lse_merge(max_s, sum_s, __shfl_xor_sync(gmask, max_s, o), __shfl_xor_sync(gmask, sum_s, o));
    lse_merge(max_b, sum_b, __shfl_xor_sync(gmask, max_b, o), __shfl_xor_sync(gmask, sum_b, o));
    const float b2 = __shfl_xor_sync(gmask, best, o), bs2 = __shfl_xor_sync(gmask, best_scaled, o);
    const int i2 = __shfl_xor_sync(gmask, best_idx, o);
    if (b2 > best || (b2 == best && i2 < best_idx)) { best = b2; best_scaled = bs2; best_idx = i2; }
    given_logit = fmaxf(given_logit, __shfl_xor_sync(gmask, given_logit, o));
  }
  if (sub == 0) {
    RowPartial r = rp[c0 + col];
    lse_merge(r.max_s, r.sum_s, max_s, sum_s);
    lse_merge(r.max_b, r.sum_b, max_b, sum_b);
    if (best > r.best || (best == r.best && best_idx < r.best_idx)) {
      r.best = best; r.best_scaled = best_scaled; r.best_idx = best_idx;
    }
    if (given_logit != -INFINITY) r.pad = __float_as_int(given_logit);
    rp[c0 + col] = r;
  }
}

// One warp merges the n partials of a logit row (global memory, stride in partials) and writes the row's result.
__device__ __forceinline__ void sample_merge_row(const SampleArgs& a, const RowPartial* parts, int n, int stride, int row,
                                                 int lane, int* tok_out, float* logp_out, float* logz_out) {
  RowPartial r = row_partial_neutral();
  float given_logit = -INFINITY;
  // two 16-byte loads per partial, four partials in flight per lane (the loop is bound by load latency)
#pragma unroll 4
  for (int c = lane; c < n; c += 32) {
    const float4* src = reinterpret_cast<const float4*>(parts + (size_t)c * stride);
    const float4 lo = __ldcg(src), hi = __ldcg(src + 1);
    RowPartial b;
    b.max_s = lo.x; b.sum_s = lo.y; b.max_b = lo.z; b.sum_b = lo.w;
    b.best = hi.x; b.best_scaled = hi.y; b.best_idx = __float_as_int(hi.z); b.pad = __float_as_int(hi.w);
    lse_merge(r.max_s, r.sum_s, b.max_s, b.sum_s);
    lse_merge(r.max_b, r.sum_b, b.max_b, b.sum_b);
    if (b.best > r.best || (b.best == r.best && b.best_idx < r.best_idx)) {
      r.best = b.best; r.best_scaled = b.best_scaled; r.best_idx = b.best_idx;
    }
    given_logit = fmaxf(given_logit, __int_as_float(b.pad));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lse_merge(r.max_s, r.sum_s, __shfl_xor_sync(0xffffffffu, r.max_s, o), __shfl_xor_sync(0xffffffffu, r.sum_s, o));
    lse_merge(r.max_b, r.sum_b, __shfl_xor_sync(0xffffffffu, r.max_b, o), __shfl_xor_sync(0xffffffffu, r.sum_b, o));
    const float b2 = __shfl_xor_sync(0xffffffffu, r.best, o), bs2 = __shfl_xor_sync(0xffffffffu, r.best_scaled, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, r.best_idx, o);
    if (b2 > r.best || (b2 == r.best && i2 < r.best_idx)) { r.best = b2; r.best_scaled = bs2; r.best_idx = i2; }
    given_logit = fmaxf(given_logit, __shfl_xor_sync(0xffffffffu, given_logit, o));
  }
  if (lane == 0) {
    const float lse_s = r.max_s + __logf(r.sum_s);
    const int given = a.tokens_in != nullptr ? a.tokens_in[row] : -1;
    if (given >= 0) {
      // score mode reports log softmax(x / T)[token] (alpha is applied by the caller)
      const float lse_b = (a.alpha != 1.f) ? r.max_b + __logf(r.sum_b) : lse_s;
      tok_out[row] = given;
      logp_out[row] = given_logit * a.inv_temp - lse_b;
      if (logz_out) logz_out[row] = 0.f;
    } else {
      tok_out[row] = r.best_idx;
      logp_out[row] = r.best_scaled - lse_s;
      if (logz_out) logz_out[row] = (a.alpha != 1.f) ? lse_s - a.alpha * (r.max_b + __logf(r.sum_b)) : 0.f;
    }
  }
}

}  // namespace smc
