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

__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  const float M = fmaxf(m, m2);
  if (M == -INFINITY) { m = M; s = 0.f; return; }
  s = s * __expf(m - M) + s2 * __expf(m2 - M);
  m = M;
}

}  // namespace smc
