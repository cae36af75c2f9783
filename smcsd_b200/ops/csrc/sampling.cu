// Fused vocabulary pass: one read of the logits gives, per row, either
//   sample mode : Gumbel-max draw from softmax(alpha * x / T), its noise-free log-probability and
//                 logZ = lse(alpha x / T) - alpha * lse(x / T)   (zero when alpha == 1), or
//   score mode  : log softmax(x / T)[token] for a given token.
// Rows choose their mode through tokens_in (>= 0: score that token, < 0: sample).  The RNG is
// Philox keyed by a seed and counted by (column, row, call id, *cycle counter); the cycle counter
// lives in device memory so captured graphs draw fresh noise on every replay.
// Logits arrive as fp32 split-K partials [splits, rows, V] straight from the lm_head GEMM.
#include "common.cuh"
#include "sample_core.cuh"

namespace smc {

constexpr int S1_THREADS = 256;

__global__ void __launch_bounds__(S1_THREADS)
sample_stage1_kernel(const float* __restrict__ logits, int splits, long long split_stride, long long row_stride, int V,
                     float inv_temp, float alpha, const int* __restrict__ tokens_in, uint64_t seed,
                     const long long* __restrict__ cycle_counter, int call_id, float softcap,
                     RowPartial* __restrict__ parts, int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int row = blockIdx.x, chunk = blockIdx.y, nchunks = gridDim.y;
  const int per = (((V + nchunks - 1) / nchunks) + 3) & ~3;
  const int c_begin = chunk * per, c_end = min(V, c_begin + per);
  const bool sampling = tokens_in == nullptr || tokens_in[row] < 0;
  const float* base = logits + (size_t)row * row_stride;
  const Philox rng(seed);
  const uint32_t ctr_lo = (uint32_t)(*cycle_counter), ctr_hi = (uint32_t)((*cycle_counter) >> 32);
  float max_s = -INFINITY, sum_s = 0.f, max_b = -INFINITY, sum_b = 0.f, best = -INFINITY, best_scaled = 0.f;
  int best_idx = c_begin < V ? c_begin : 0;
  for (int c = c_begin + threadIdx.x * 4; c < c_end; c += S1_THREADS * 4) {
    float x[4];
    if (c + 3 < V) {
      float4 a = *reinterpret_cast<const float4*>(base + c);
      for (int s = 1; s < splits; ++s) {
        const float4 b2 = *reinterpret_cast<const float4*>(base + (size_t)s * split_stride + c);
        a.x += b2.x; a.y += b2.y; a.z += b2.z; a.w += b2.w;
      }
      x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    } else {
      for (int j = 0; j < 4; ++j) {
        float a = -INFINITY;
        if (c + j < V) {
          a = 0.f;
          for (int s = 0; s < splits; ++s) a += base[(size_t)s * split_stride + c + j];
        }
        x[j] = a;
      }
    }
    uint32_t rnd[4] = {0, 0, 0, 0};
    if (sampling) rng.run((uint32_t)(c >> 2), (uint32_t)row, (uint32_t)call_id ^ (ctr_hi << 8), ctr_lo, rnd);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (c + j >= c_end) continue;
      float v = x[j];
      if (softcap > 0.f) v = tanhf(v / softcap) * softcap;
      const float b = v * inv_temp;
      const float sc = b * alpha;
      if (sc > max_s) { sum_s = sum_s * __expf(max_s - sc) + 1.f; max_s = sc; } else { sum_s += __expf(sc - max_s); }
      if (alpha != 1.f) {
        if (b > max_b) { sum_b = sum_b * __expf(max_b - b) + 1.f; max_b = b; } else { sum_b += __expf(b - max_b); }
      }
      if (sampling) {
        const float u = u32_to_unit(rnd[j]);
        const float g = -__logf(-__logf(u));
        const float pert = sc + g;
        if (pert > best) { best = pert; best_scaled = sc; best_idx = c + j; }
      }
    }
  }
  // block reduction
  __shared__ RowPartial red[S1_THREADS / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, max_s, o), s2 = __shfl_xor_sync(0xffffffffu, sum_s, o);
    lse_merge(max_s, sum_s, m2, s2);
    const float mb2 = __shfl_xor_sync(0xffffffffu, max_b, o), sb2 = __shfl_xor_sync(0xffffffffu, sum_b, o);
    lse_merge(max_b, sum_b, mb2, sb2);
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o), bs2 = __shfl_xor_sync(0xffffffffu, best_scaled, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_idx, o);
    if (b2 > best || (b2 == best && i2 < best_idx)) { best = b2; best_scaled = bs2; best_idx = i2; }
  }
  if (lane == 0) red[warp] = RowPartial{max_s, sum_s, max_b, sum_b, best, best_scaled, best_idx, 0};
  __syncthreads();
  if (threadIdx.x == 0) {
    RowPartial a = red[0];
    for (int w = 1; w < S1_THREADS / 32; ++w) {
      const RowPartial b2 = red[w];
      lse_merge(a.max_s, a.sum_s, b2.max_s, b2.sum_s);
      lse_merge(a.max_b, a.sum_b, b2.max_b, b2.sum_b);
      if (b2.best > a.best || (b2.best == a.best && b2.best_idx < a.best_idx)) {
        a.best = b2.best; a.best_scaled = b2.best_scaled; a.best_idx = b2.best_idx;
      }
    }
    parts[(size_t)row * nchunks + chunk] = a;
  }
}

__global__ void sample_stage2_kernel(const RowPartial* __restrict__ parts, int nchunks, const float* __restrict__ logits,
                                     int splits, long long split_stride, long long row_stride, float inv_temp,
                                     float alpha, float softcap, const int* __restrict__ tokens_in,
                                     int* __restrict__ tok_out, float* __restrict__ logp_out,
                                     float* __restrict__ logz_out, int rows, int pdl) {
  if (pdl) { pdl_launch_dependents(); pdl_wait_prior_grid(); }
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < rows) {
    RowPartial a = parts[(size_t)row * nchunks];
    for (int c = 1; c < nchunks; ++c) {
      const RowPartial b2 = parts[(size_t)row * nchunks + c];
      lse_merge(a.max_s, a.sum_s, b2.max_s, b2.sum_s);
      lse_merge(a.max_b, a.sum_b, b2.max_b, b2.sum_b);
      if (b2.best > a.best || (b2.best == a.best && b2.best_idx < a.best_idx)) {
        a.best = b2.best; a.best_scaled = b2.best_scaled; a.best_idx = b2.best_idx;
      }
    }
    const float lse_s = a.max_s + __logf(a.sum_s);
    const int given = tokens_in ? tokens_in[row] : -1;
    if (given >= 0) {
      float v = 0.f;
      for (int s = 0; s < splits; ++s) v += logits[(size_t)s * split_stride + (size_t)row * row_stride + given];
      if (softcap > 0.f) v = tanhf(v / softcap) * softcap;
      // score mode reports log softmax(x / T)[token] (alpha is applied by the caller)
      const float lse_b = (alpha != 1.f) ? a.max_b + __logf(a.sum_b) : lse_s;
      tok_out[row] = given;
      logp_out[row] = v * inv_temp - lse_b;
      if (logz_out) logz_out[row] = 0.f;
    } else {
      tok_out[row] = a.best_idx;
      logp_out[row] = a.best_scaled - lse_s;
      if (logz_out) logz_out[row] = (alpha != 1.f) ? lse_s - alpha * (a.max_b + __logf(a.sum_b)) : 0.f;
    }
  }
}

}  // namespace smc

// Host-side view of the uniform mapping used for the Gumbel noise (for tests of its open-interval property).
SMC_API float smc_u32_to_unit(unsigned int x) { return smc::u32_to_unit(x); }

SMC_API int smc_sample_scratch_bytes(int rows, int nchunks) { return rows * nchunks * (int)sizeof(smc::RowPartial); }

// logits fp32 partials [splits, rows(row_stride), V]; tokens_in may be null (all rows sample).
SMC_API int smc_sample_or_score(const float* logits, int splits, long long split_stride, long long row_stride, int rows,
                                int V, float temperature, float alpha, float softcap, const int* tokens_in,
                                unsigned long long seed, const long long* cycle_counter, int call_id, void* scratch,
                                int nchunks, int* tok_out, float* logp_out, float* logz_out, int pdl,
                                cudaStream_t st) {
  using namespace smc;
  if (rows <= 0) return 0;
  if ((row_stride & 3) || (split_stride & 3)) return -50;
  const float inv_temp = 1.0f / temperature;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows, nchunks);
  cfg.blockDim = dim3(S1_THREADS);
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, sample_stage1_kernel, logits, splits, split_stride, row_stride, V, inv_temp,
                                    alpha, tokens_in, (uint64_t)seed, cycle_counter, call_id, softcap,
                                    (RowPartial*)scratch, pdl));
  cfg.gridDim = dim3((rows + 63) / 64);
  cfg.blockDim = dim3(64);
  CUDA_CHECK_RET(cudaLaunchKernelEx(&cfg, sample_stage2_kernel, (const RowPartial*)scratch, nchunks, logits, splits,
                                    split_stride, row_stride, inv_temp, alpha, softcap, tokens_in, tok_out, logp_out,
                                    logz_out, rows, pdl));
  return 0;
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in smc_no_alloc.h).
// ---------------------------------------------------------------------------------------------------
#include <stdio.h>

#include "smc_no_alloc.h"

namespace smc {
constexpr int STATIC_NCHUNKS = 32;
// Scratch for the per-(row, chunk) partial results.  In host code this name is only a handle for the
// symbol: the address kernels can use is obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) RowPartial g_static_sample_scratch[SMC_STATIC_SAMPLE_MAX_ROWS * STATIC_NCHUNKS];
static RowPartial* g_static_scratch_addr[64] = {nullptr};
static thread_local char g_no_alloc_error[256] = "";
}  // namespace smc

SMC_API const char* smc_no_alloc_last_error(void) { return smc::g_no_alloc_error; }

SMC_API int smc_sample_or_score_static(const float* logits, int splits, long long split_stride, long long row_stride,
                                       int rows, int V, float temperature, float alpha, float softcap,
                                       const int* tokens_in, unsigned long long seed, const long long* cycle_counter,
                                       int call_id, int* tok_out, float* logp_out, float* logz_out,
                                       cudaStream_t stream) {
  using namespace smc;
  g_no_alloc_error[0] = '\0';
  if (rows <= 0) return 0;
  if (rows > SMC_STATIC_SAMPLE_MAX_ROWS) {
    snprintf(g_no_alloc_error, sizeof(g_no_alloc_error),
             "smc_sample_or_score_static: %d rows requested, the built-in scratch holds at most %d", rows,
             SMC_STATIC_SAMPLE_MAX_ROWS);
    return SMC_STATIC_ERR_TOO_LARGE;
  }
  if ((row_stride & 3) || (split_stride & 3) || temperature <= 0.f || V <= 0 || splits < 1) {
    snprintf(g_no_alloc_error, sizeof(g_no_alloc_error),
             "smc_sample_or_score_static: bad argument (strides must be multiples of 4, temperature > 0)");
    return SMC_STATIC_ERR_ARG;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    snprintf(g_no_alloc_error, sizeof(g_no_alloc_error), "smc_sample_or_score_static: cannot identify the device");
    return SMC_STATIC_ERR_SETUP;
  }
  if (g_static_scratch_addr[dev] == nullptr) {
    // once per device, with that device current: resolve the device address of the scratch array
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_sample_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      snprintf(g_no_alloc_error, sizeof(g_no_alloc_error),
               "smc_sample_or_score_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return SMC_STATIC_ERR_SETUP;
    }
    g_static_scratch_addr[dev] = static_cast<RowPartial*>(ptr);
  }
  RowPartial* scratch = g_static_scratch_addr[dev];
  const float inv_temp = 1.0f / temperature;
  sample_stage1_kernel<<<dim3(rows, STATIC_NCHUNKS), S1_THREADS, 0, stream>>>(
      logits, splits, split_stride, row_stride, V, inv_temp, alpha, tokens_in, (uint64_t)seed, cycle_counter, call_id,
      softcap, scratch, 0);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  sample_stage2_kernel<<<(rows + 63) / 64, 64, 0, stream>>>(scratch, STATIC_NCHUNKS, logits, splits, split_stride,
                                                            row_stride, inv_temp, alpha, softcap, tokens_in, tok_out,
                                                            logp_out, logz_out, rows, 0);
  return (int)cudaGetLastError();
}
